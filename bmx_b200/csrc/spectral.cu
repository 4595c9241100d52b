// K4 spectral key codec, per-head packs (128 x 128 encoder / decoder, per-direction bit tiers):
// quantize-on-append and page dequantizer.
//   encode   Y = M @ enc                                   (bmx: src/bmx/cache/spectral.py:798)
//   per direction j with b_j > 0 bits, per group of `group` tokens: symmetric RTN with the step refined
//   by 10 alternating-minimisation rounds                  (bmx: src/bmx/quant/rtn.py:10-44, mse_scale=True)
//   decode   M_hat = Y_hat @ dec^T                          (bmx: src/bmx/cache/spectral.py:812-839)
// Containers follow bmx (spectral.py:703-739): 2- and 4-bit tiers offset-binary at exact width, the 3-bit
// tier as two's-complement nibbles, 5/6/8-bit tiers as int8; all packed along tokens.
//
// Page block per (slot, head): for every direction with bits, its code row (page * container_bits / 8
// bytes) at the byte offset the host assigns (directions sorted by tier), then float32 scales
// [direction][page / group].  Sums run in ascending index order with one accumulator (fmaf for the two
// matrix products; separate multiply and add inside the step refinement, as the reference does), which
// makes the result independent of launch shape.  Compiled with -fmad=false.
#include "common.cuh"

namespace bmxk {

struct SpectralGeom {
  int h_kv, page, group, block_bytes, scale_off;
};

__device__ __forceinline__ int container_bits(int b) { return b == 0 ? 0 : (b == 2 ? 2 : (b <= 4 ? 4 : 8)); }

template <typename T>
__global__ void __launch_bounds__(128) spectral_quant_page_kernel(SpectralGeom g, const T* __restrict__ k,
                                                                  int64_t stride_seq, int64_t stride_head, int64_t stride_tok,
                                                                  const float* __restrict__ enc, const int32_t* __restrict__ col_bits,
                                                                  const int32_t* __restrict__ col_off, const int32_t* __restrict__ slots,
                                                                  int n_pages, uint8_t* __restrict__ pages) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* Ms = reinterpret_cast<float*>(smem);  // [page][128] keys, then Y in place
  const int item = blockIdx.x / g.h_kv, h = blockIdx.x % g.h_kv;
  const int seq = item / n_pages, pg = item % n_pages, page = g.page, j = threadIdx.x;
  const T* src = k + seq * stride_seq + h * stride_head + (int64_t)pg * page * stride_tok;
  for (int o = threadIdx.x; o < page * HEAD_DIM; o += 128) Ms[o] = load_as_float<T>(src + (o / HEAD_DIM) * stride_tok + o % HEAD_DIM);
  __syncthreads();
  const float* e = enc + (int64_t)h * HEAD_DIM * HEAD_DIM;
  // Y[:, j]: thread j walks the rows; every thread reads the same key row (shared-memory broadcast)
  float y[128];
#pragma unroll 1
  for (int r = 0; r < page; ++r) {
    float acc = 0.f;
    for (int c = 0; c < HEAD_DIM; ++c) acc = fmaf(Ms[r * HEAD_DIM + c], e[c * HEAD_DIM + j], acc);
    y[r & 127] = acc;
  }
  __syncthreads();
  for (int r = 0; r < page; ++r) Ms[r * HEAD_DIM + j] = y[r];
  __syncthreads();
  const int b = col_bits[h * HEAD_DIM + j];
  if (b == 0) return;
  uint8_t* blk = pages + ((int64_t)slots[item] * g.h_kv + h) * g.block_bytes;
  uint8_t* row = blk + col_off[h * HEAD_DIM + j];
  float* scales = reinterpret_cast<float*>(blk + g.scale_off) + j * (page / g.group);
  const float qmax = (float)((1 << (b - 1)) - 1);
  const int cb = container_bits(b);
  for (int grp = 0; grp < page / g.group; ++grp) {
    const int r0 = grp * g.group;
    float amax = 0.f;
    for (int r = r0; r < r0 + g.group; ++r) amax = fmaxf(amax, fabsf(Ms[r * HEAD_DIM + j]));
    float scale = fmaxf(amax, 1e-12f) / qmax;
    for (int it = 0; it < 10; ++it) {
      float num = 0.f, den = 0.f;
      for (int r = r0; r < r0 + g.group; ++r) {
        const float x = Ms[r * HEAD_DIM + j];
        const float q = fminf(fmaxf(rintf(x / scale), -qmax - 1.f), qmax);
        num = num + x * q;
        den = den + q * q;
      }
      scale = fmaxf(num / fmaxf(den, 1e-12f), 1e-12f);
    }
    scales[grp] = scale;
    for (int r = r0; r < r0 + g.group; r += 8 / cb) {
      uint32_t byte = 0;
      for (int u = 0; u < 8 / cb; ++u) {
        const int q = (int)fminf(fmaxf(rintf(Ms[(r + u) * HEAD_DIM + j] / scale), -qmax - 1.f), qmax);
        const uint32_t field = (b == 2 || b == 4) ? (uint32_t)(q + (1 << (b - 1))) : ((uint32_t)q & ((1u << cb) - 1u));
        byte |= field << (cb * u);
      }
      row[r * cb / 8] = (uint8_t)byte;
    }
  }
}

__device__ __forceinline__ int spectral_code(const uint8_t* row, int r, int b) {
  const int cb = container_bits(b);
  if (cb == 8) return (int)(int8_t)row[r];
  const uint32_t f = (row[r * cb / 8] >> (cb * (r % (8 / cb)))) & ((1u << cb) - 1u);
  if (b == 3) return (int)((f ^ 8u)) - 8;          // two's-complement nibble
  return (int)f - (1 << (b - 1));                  // offset binary (2- and 4-bit tiers)
}

// One block per (page, head): codes as int8 (n, h, 128 directions, page), scales float32, and/or
// M_hat = Y_hat @ dec^T as float32 (n, page, h*128).
__global__ void __launch_bounds__(128) spectral_dequant_kernel(SpectralGeom g, const uint8_t* __restrict__ pages,
                                                               const float* __restrict__ dec, const int32_t* __restrict__ col_bits,
                                                               const int32_t* __restrict__ col_off, const int32_t* __restrict__ slots,
                                                               int8_t* __restrict__ codes, float* __restrict__ scales_out,
                                                               float* __restrict__ k_out) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* Ys = reinterpret_cast<float*>(smem);  // [page][128]
  const int n = blockIdx.x / g.h_kv, h = blockIdx.x % g.h_kv, page = g.page, j = threadIdx.x, ngrp = page / g.group;
  const uint8_t* blk = pages + ((int64_t)slots[n] * g.h_kv + h) * g.block_bytes;
  const int b = col_bits[h * HEAD_DIM + j];
  const uint8_t* row = blk + col_off[h * HEAD_DIM + j];
  const float* sc = reinterpret_cast<const float*>(blk + g.scale_off) + j * ngrp;
  for (int r = 0; r < page; ++r) {
    const int q = b ? spectral_code(row, r, b) : 0;
    Ys[r * HEAD_DIM + j] = b ? (float)q * sc[r / g.group] : 0.f;
    if (codes) codes[(((int64_t)n * g.h_kv + h) * HEAD_DIM + j) * page + r] = (int8_t)q;
  }
  if (scales_out)
    for (int grp = 0; grp < ngrp; ++grp) scales_out[(((int64_t)n * g.h_kv + h) * HEAD_DIM + j) * ngrp + grp] = b ? sc[grp] : 0.f;
  __syncthreads();
  if (k_out) {
    const float* d = dec + (int64_t)h * HEAD_DIM * HEAD_DIM + (int64_t)j * HEAD_DIM;  // dec[c = j][:]
    for (int r = 0; r < page; ++r) {
      float acc = 0.f;
      for (int i = 0; i < HEAD_DIM; ++i) acc = fmaf(Ys[r * HEAD_DIM + i], d[i], acc);
      k_out[((int64_t)n * page + r) * (g.h_kv * HEAD_DIM) + h * HEAD_DIM + j] = acc;
    }
  }
}

static int check_sgeom(const bmxk_spectral_geom* g, const char* who) {
  BMXK_REQUIRE(g != nullptr, "%s: null geometry", who);
  BMXK_REQUIRE(g->h_kv >= 1 && g->h_kv <= 64, "%s: h_kv=%d", who, g->h_kv);
  BMXK_REQUIRE(g->page == 64 || g->page == 128, "%s: page=%d must be 64 or 128", who, g->page);
  BMXK_REQUIRE(g->group >= 8 && g->page % g->group == 0 && g->group % 8 == 0, "%s: group=%d must divide page and be a multiple of 8", who,
               g->group);
  BMXK_REQUIRE(g->block_bytes > 0 && g->scale_off >= 0 && g->scale_off % 4 == 0 &&
                   g->scale_off + HEAD_DIM * (g->page / g->group) * 4 <= g->block_bytes,
               "%s: inconsistent block_bytes=%d / scale_off=%d", who, g->block_bytes, g->scale_off);
  return BMXK_OK;
}
static SpectralGeom to_s(const bmxk_spectral_geom* g) {
  SpectralGeom o;
  o.h_kv = g->h_kv, o.page = g->page, o.group = g->group, o.block_bytes = g->block_bytes, o.scale_off = g->scale_off;
  return o;
}

}  // namespace bmxk

using namespace bmxk;

extern "C" {

int bmxk_spectral_append(const bmxk_spectral_geom* g, const void* k_pre, int src_dtype, int64_t stride_seq, int64_t stride_head,
                         int64_t stride_tok, const float* enc, const int32_t* col_bits, const int32_t* col_off,
                         const int32_t* slots, int n_seq, int n_pages, void* pages, void* stream) {
  int rc = check_sgeom(g, "bmxk_spectral_append");
  if (rc) return rc;
  BMXK_REQUIRE(n_seq >= 0 && n_pages >= 0, "bmxk_spectral_append: negative counts");
  if (n_seq == 0 || n_pages == 0) return BMXK_OK;
  BMXK_REQUIRE(k_pre && enc && col_bits && col_off && slots && pages, "bmxk_spectral_append: null pointer");
  const SpectralGeom gg = to_s(g);
  const int blocks = n_seq * n_pages * g->h_kv;
  const size_t smem = (size_t)g->page * HEAD_DIM * 4;
  cudaStream_t s = (cudaStream_t)stream;
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaFuncSetAttribute(spectral_quant_page_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    cudaFuncSetAttribute(spectral_quant_page_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    cudaFuncSetAttribute(spectral_quant_page_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  }
  if (src_dtype == BMXK_DTYPE_F16)
    spectral_quant_page_kernel<__half><<<blocks, 128, smem, s>>>(gg, (const __half*)k_pre, stride_seq, stride_head, stride_tok, enc,
                                                                  col_bits, col_off, slots, n_pages, (uint8_t*)pages);
  else if (src_dtype == BMXK_DTYPE_BF16)
    spectral_quant_page_kernel<__nv_bfloat16><<<blocks, 128, smem, s>>>(gg, (const __nv_bfloat16*)k_pre, stride_seq, stride_head,
                                                                         stride_tok, enc, col_bits, col_off, slots, n_pages,
                                                                         (uint8_t*)pages);
  else if (src_dtype == BMXK_DTYPE_F32)
    spectral_quant_page_kernel<float><<<blocks, 128, smem, s>>>(gg, (const float*)k_pre, stride_seq, stride_head, stride_tok, enc,
                                                                 col_bits, col_off, slots, n_pages, (uint8_t*)pages);
  else {
    set_error("bmxk_spectral_append: unknown src_dtype %d", src_dtype);
    return BMXK_ERR_INVALID;
  }
  return check_launch("bmxk_spectral_append");
}

int bmxk_spectral_dequant_pages(const bmxk_spectral_geom* g, const void* pages, const float* dec, const int32_t* col_bits,
                                const int32_t* col_off, const int32_t* slots, int n, int8_t* codes, float* scales, float* k_out,
                                void* stream) {
  int rc = check_sgeom(g, "bmxk_spectral_dequant_pages");
  if (rc) return rc;
  BMXK_REQUIRE(n >= 0, "bmxk_spectral_dequant_pages: n < 0");
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(pages && col_bits && col_off && slots && (!k_out || dec), "bmxk_spectral_dequant_pages: null pointer");
  static PerDeviceOnce configured;
  if (configured.first()) cudaFuncSetAttribute(spectral_dequant_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  spectral_dequant_kernel<<<n * g->h_kv, 128, (size_t)g->page * HEAD_DIM * 4, (cudaStream_t)stream>>>(
      to_s(g), (const uint8_t*)pages, dec, col_bits, col_off, slots, codes, scales, k_out);
  return check_launch("bmxk_spectral_dequant_pages");
}

}  // extern "C"
