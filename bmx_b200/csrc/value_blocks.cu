// Value-only page blocks for caches whose keys live in another pool (the K4 spectral key codec):
// quantize-on-append of the per-head Hadamard + 2-bit Lloyd value codec, and the exporter that rewrites
// blocks into the reference's containers.
//   n = fp16(max(||v||, 1e-12)); u = v / n; y = fwht(u * signs); idx = #{mid_k < y * sqrt(128)}
//   (bmx: src/bmx/cache/codecs.py:616-636)
// Block per (slot, head), 4352 bytes: [ V codes, 4096 B | V norms, 128 fp16 ], both in the "row order" of
// the k2b page block (layout.cuh, layout 1), so that the tcgen05 decode kernels read either pool alike.
// Compiled with -fmad=false; the arithmetic is the one of k2b_quant_page_kernel, step for step.
#include "common.cuh"

namespace bmxk {

constexpr int VBLOCK_BYTES = 128 * 32 + 128 * 2;

template <typename T>
__global__ void __launch_bounds__(128) vblock_quant_kernel(int h_kv, const T* __restrict__ v, int64_t stride_seq, int64_t stride_head,
                                                           int64_t stride_tok, const float* __restrict__ signs,
                                                           const float* __restrict__ codebook, const int32_t* __restrict__ slots,
                                                           int n_pages, uint8_t* __restrict__ vpages) {
  __shared__ __align__(16) uint8_t vcode[128 * HEAD_DIM];  // [token][channel]
  const int item = blockIdx.x / h_kv, h = blockIdx.x % h_kv;
  const int seq = item / n_pages, pg = item % n_pages;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* blk = vpages + ((int64_t)slots[item] * h_kv + h) * VBLOCK_BYTES;
  const T* vsrc = v + seq * stride_seq + h * stride_head + (int64_t)pg * 128 * stride_tok;
  const float c0 = codebook[0], c1 = codebook[1], c2 = codebook[2], c3 = codebook[3];
  const float m0 = (c0 + c1) / 2.f, m1 = (c1 + c2) / 2.f, m2 = (c2 + c3) / 2.f;
  float sg[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) sg[k] = signs[4 * lane + k];
  __half* vnorm = reinterpret_cast<__half*>(blk + 128 * 32);
  for (int r = warp; r < 128; r += 4) {  // warp = token
    float x[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) x[k] = load_as_float<T>(vsrc + r * stride_tok + 4 * lane + k);
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) ss = fmaf(x[k], x[k], ss);
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) ss = ss + __shfl_xor_sync(0xffffffffu, ss, m);
    const float n = __half2float(__float2half_rn(fmaxf(sqrtf(ss), 1e-12f)));
#pragma unroll
    for (int k = 0; k < 4; ++k) x[k] = (x[k] / n) * sg[k];
    fwht128_warp(x, lane);
    const float sqrt_d = 11.313708498984761f;
    uint32_t packed4 = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float y = x[k] * sqrt_d;
      packed4 |= (uint32_t)((y > m0) + (y > m1) + (y > m2)) << (8 * k);
    }
    *reinterpret_cast<uint32_t*>(vcode + r * HEAD_DIM + 4 * lane) = packed4;
    if (lane == 0) vnorm[r] = __float2half_rn(n);
  }
  __syncthreads();
  // word w = (chunk cc, channel c, word j) holds tokens 64cc + 16j .. + 15 of channel c
  uint32_t* vw = reinterpret_cast<uint32_t*>(blk);
  for (int w = tid; w < 128 * 8; w += 128) {
    const int j = w & 3, c = (w >> 2) & 127, cc = w >> 9;
    uint32_t word = 0;
#pragma unroll
    for (int tau = 0; tau < 16; ++tau)
      word |= (uint32_t)vcode[(64 * cc + 16 * j + tau) * HEAD_DIM + c] << (tau < 8 ? 4 * tau : 4 * (tau - 8) + 2);
    vw[w] = word;
  }
}

// v_idx_packed[n][r][(h*128 + c)/4] (four 2-bit codes per byte, channel-minor) and v_norm[n][r][h], as
// bmx's build_kv_stacked_k2b stacks them (src/bmx/cache/triton_dequant_attention.py:1118-1229).
__global__ void vblock_export_kernel(int h_kv, const uint8_t* __restrict__ vpages, const int32_t* __restrict__ slots,
                                     uint8_t* __restrict__ v_idx_packed, __half* __restrict__ v_norm) {
  const int n = blockIdx.x / h_kv, h = blockIdx.x % h_kv, C = h_kv * HEAD_DIM;
  const uint8_t* blk = vpages + ((int64_t)slots[n] * h_kv + h) * VBLOCK_BYTES;
  const uint32_t* vw = reinterpret_cast<const uint32_t*>(blk);
  const __half* vn = reinterpret_cast<const __half*>(blk + 128 * 32);
  for (int o = threadIdx.x; o < 128 * HEAD_DIM / 4; o += blockDim.x) {
    const int r = o / (HEAD_DIM / 4), cb = o % (HEAD_DIM / 4);
    uint32_t b = 0;
    for (int k = 0; k < 4; ++k) {
      int w, bit;
      k2b_vcode_loc(1, r, 4 * cb + k, w, bit);
      b |= ((vw[w] >> bit) & 3u) << (2 * k);
    }
    v_idx_packed[((int64_t)n * 128 + r) * (C / 4) + h * (HEAD_DIM / 4) + cb] = (uint8_t)b;
  }
  for (int r = threadIdx.x; r < 128; r += blockDim.x) v_norm[((int64_t)n * 128 + r) * h_kv + h] = vn[r];
}

}  // namespace bmxk

using namespace bmxk;

extern "C" {

size_t bmxk_vblock_bytes(void) { return (size_t)VBLOCK_BYTES; }

int bmxk_vblock_append(int h_kv, const void* v, int src_dtype, int64_t stride_seq, int64_t stride_head, int64_t stride_tok,
                       const float* signs, const float* codebook, const int32_t* slots, int n_seq, int n_pages, void* vpages,
                       void* stream) {
  BMXK_REQUIRE(h_kv >= 1 && h_kv <= 64, "bmxk_vblock_append: h_kv=%d", h_kv);
  BMXK_REQUIRE(n_seq >= 0 && n_pages >= 0, "bmxk_vblock_append: negative counts");
  if (n_seq == 0 || n_pages == 0) return BMXK_OK;
  BMXK_REQUIRE(v && signs && codebook && slots && vpages, "bmxk_vblock_append: null pointer");
  BMXK_REQUIRE(stride_tok >= HEAD_DIM, "bmxk_vblock_append: stride_tok=%lld < 128", (long long)stride_tok);
  BMXK_REQUIRE((int64_t)n_seq * n_pages * h_kv < (1LL << 31), "bmxk_vblock_append: too many pages in one call");
  const int blocks = n_seq * n_pages * h_kv;
  cudaStream_t s = (cudaStream_t)stream;
  if (src_dtype == BMXK_DTYPE_F16)
    vblock_quant_kernel<__half><<<blocks, 128, 0, s>>>(h_kv, (const __half*)v, stride_seq, stride_head, stride_tok, signs, codebook,
                                                        slots, n_pages, (uint8_t*)vpages);
  else if (src_dtype == BMXK_DTYPE_BF16)
    vblock_quant_kernel<__nv_bfloat16><<<blocks, 128, 0, s>>>(h_kv, (const __nv_bfloat16*)v, stride_seq, stride_head, stride_tok, signs,
                                                               codebook, slots, n_pages, (uint8_t*)vpages);
  else if (src_dtype == BMXK_DTYPE_F32)
    vblock_quant_kernel<float><<<blocks, 128, 0, s>>>(h_kv, (const float*)v, stride_seq, stride_head, stride_tok, signs, codebook, slots,
                                                       n_pages, (uint8_t*)vpages);
  else {
    set_error("bmxk_vblock_append: unknown src_dtype %d", src_dtype);
    return BMXK_ERR_INVALID;
  }
  return check_launch("bmxk_vblock_append");
}

int bmxk_vblock_export(int h_kv, const void* vpages, const int32_t* slots, int n, uint8_t* v_idx_packed, void* v_norm, void* stream) {
  BMXK_REQUIRE(h_kv >= 1 && h_kv <= 64 && n >= 0, "bmxk_vblock_export: h_kv=%d n=%d", h_kv, n);
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(vpages && slots && v_idx_packed && v_norm, "bmxk_vblock_export: null pointer");
  vblock_export_kernel<<<n * h_kv, 256, 0, (cudaStream_t)stream>>>(h_kv, (const uint8_t*)vpages, slots, v_idx_packed, (__half*)v_norm);
  return check_launch("bmxk_vblock_export");
}

}  // extern "C"
