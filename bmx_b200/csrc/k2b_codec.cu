// k2b write side: quantize-on-append into the native page layout, the exporter that rewrites
// pages into the reference's stacked tensors, and the page dequantizer.
//
// Compiled with -fmad=false: every multiply-then-add that the reference performs as two
// float32 operations stays two operations here; the sums that ARE fused use fmaf explicitly
// and run in a fixed order (ascending index, one accumulator), which `oracle/cpu_ref.c`
// repeats step for step.
#include "common.cuh"

namespace bmxk {

__device__ __forceinline__ float half_round(float x) { return __half2float(__float2half_rn(x)); }

// ---------------------------------------------------------------------------------------------
// Projection  Us = M @ V  (bmx: src/bmx/cache/packed_streaming.py:518-520), rounded to fp16 and
// written to the coefficient block.  One block per (item, coef head); thread -> (row, i).
// Order: acc = 0; for c ascending: acc = fmaf(M[r,c], V[c,i], acc).
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void k2b_project_kernel(K2bGeom g, const T* __restrict__ k_pre, int64_t stride_seq, int64_t stride_head,
                                   int64_t stride_tok, const float* __restrict__ basis, const int32_t* __restrict__ slots,
                                   int n_pages, __half* __restrict__ coefs) {
  const int item = blockIdx.x / g.n_coef_heads, ch = blockIdx.x % g.n_coef_heads;
  const int seq = item / n_pages, pg = item % n_pages;
  const int slot = slots[item];
  const int h0 = (g.n_coef_heads == 1) ? 0 : ch, nh = (g.n_coef_heads == 1) ? g.h_kv : 1;
  __half* out = coefs + ((int64_t)slot * g.n_coef_heads + ch) * (g.page * g.rank);
  const T* src = k_pre + seq * stride_seq + (int64_t)pg * g.page * stride_tok;
  for (int o = threadIdx.x; o < g.page * g.rank; o += blockDim.x) {
    const int r = o / g.rank, i = o % g.rank;
    float acc = 0.f;
    for (int h = h0; h < h0 + nh; ++h) {
      const T* row = src + h * stride_head + r * stride_tok;
      const float* b = basis + (int64_t)h * HEAD_DIM * g.rank + i;
      for (int c = 0; c < HEAD_DIM; ++c) acc = fmaf(load_as_float<T>(row + c), b[(int64_t)c * g.rank], acc);
    }
    out[k2b_coef_idx(g.layout, r, i, g.rank)] = __float2half_rn(acc);
  }
}

// ---------------------------------------------------------------------------------------------
// Page quantizer.  One block of 128 threads per (item, kv head).
//   keys  : thread = channel.  L[r,c] = sum_i Us16[r,i] V16[c,i] (fmaf, i ascending), R = M - L,
//           per group of `group` tokens scale = max(absmax, 1e-12) / qmax, code = rint(R / scale)
//           clamped to [-qmax-1, qmax]   (bmx: src/bmx/cache/codecs.py:677-695, src/bmx/quant/rtn.py:34-44)
//   values: warp = token.   n = fp16(max(sqrt(sum v^2), 1e-12)); u = v / n; y = fwht(u * signs);
//           idx = #{mid_k < y * sqrt(128)}        (bmx: src/bmx/cache/codecs.py:616-636)
// Codes are staged in shared memory and then assembled into whole 32-bit words of the native layout.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) k2b_quant_page_kernel(K2bGeom g, const T* __restrict__ k_pre,
                                                             const T* __restrict__ v, int64_t stride_seq,
                                                             int64_t stride_head, int64_t stride_tok,
                                                             const float* __restrict__ basis,
                                                             const float* __restrict__ signs,
                                                             const float* __restrict__ codebook,
                                                             const int32_t* __restrict__ slots, int n_pages,
                                                             uint8_t* __restrict__ pages, const __half* __restrict__ coefs) {
  extern __shared__ __align__(16) uint8_t smem[];
  int8_t* kcode = reinterpret_cast<int8_t*>(smem);                     // [page][128]
  uint8_t* vcode = smem + g.page * HEAD_DIM;                            // [page][128]
  float* us = reinterpret_cast<float*>(smem + 2 * g.page * HEAD_DIM);   // [page][rank]

  const int item = blockIdx.x / g.h_kv, h = blockIdx.x % g.h_kv;
  const int seq = item / n_pages, pg = item % n_pages;
  const int slot = slots[item];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int page = g.page, rank = g.rank, group = g.group;
  const int ch = (g.n_coef_heads == 1) ? 0 : h;
  const __half* cblk = coefs + ((int64_t)slot * g.n_coef_heads + ch) * (page * rank);
  uint8_t* blk = pages + ((int64_t)slot * g.h_kv + h) * k2b_page_block_bytes(page, group);
  const T* ksrc = k_pre + seq * stride_seq + h * stride_head + (int64_t)pg * page * stride_tok;
  const T* vsrc = v + seq * stride_seq + h * stride_head + (int64_t)pg * page * stride_tok;

  for (int o = tid; o < page * rank; o += blockDim.x) us[o] = __half2float(cblk[k2b_coef_idx(g.layout, o / rank, o % rank, rank)]);
  __syncthreads();

  // ---- keys: thread = channel ----
  {
    const int c = tid;
    float vb[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) vb[i] = (i < rank) ? half_round(basis[((int64_t)h * HEAD_DIM + c) * rank + i]) : 0.f;
    const float qmax = (float)((1 << (g.kbits - 1)) - 1);
    __half* kscale = reinterpret_cast<__half*>(blk + k2b_off_kscale(page));
    for (int grp = 0; grp < page / group; ++grp) {
      float amax = 0.f;
      for (int r = grp * group; r < (grp + 1) * group; ++r) {
        float L = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < rank) L = fmaf(us[r * rank + i], vb[i], L);
        const float R = load_as_float<T>(ksrc + r * stride_tok + c) - L;
        amax = fmaxf(amax, fabsf(R));
      }
      const float scale = fmaxf(amax, 1e-12f) / qmax;
      kscale[k2b_kscale_idx(g.layout, grp, c)] = __float2half_rn(scale);
      for (int r = grp * group; r < (grp + 1) * group; ++r) {
        float L = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i < rank) L = fmaf(us[r * rank + i], vb[i], L);
        const float R = load_as_float<T>(ksrc + r * stride_tok + c) - L;
        float q = rintf(R / scale);
        q = fminf(fmaxf(q, -qmax - 1.f), qmax);
        kcode[r * HEAD_DIM + c] = (int8_t)q;
      }
    }
  }
  // ---- values: warp = token ----
  {
    const float c0 = codebook[0], c1 = codebook[1], c2 = codebook[2], c3 = codebook[3];
    const float m0 = (c0 + c1) / 2.f, m1 = (c1 + c2) / 2.f, m2 = (c2 + c3) / 2.f;
    float sg[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) sg[k] = signs[4 * lane + k];
    __half* vnorm = reinterpret_cast<__half*>(blk + k2b_off_vnorm(page, group));
    for (int r = warp; r < page; r += 4) {
      float x[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = load_as_float<T>(vsrc + r * stride_tok + 4 * lane + k);
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) ss = fmaf(x[k], x[k], ss);
#pragma unroll
      for (int m = 16; m >= 1; m >>= 1) ss = ss + __shfl_xor_sync(0xffffffffu, ss, m);
      const float n = half_round(fmaxf(sqrtf(ss), 1e-12f));
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = (x[k] / n) * sg[k];
      fwht128_warp(x, lane);
      const float sqrt_d = 11.313708498984761f;
      uint32_t packed4 = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float y = x[k] * sqrt_d;
        const uint32_t idx = (y > m0) + (y > m1) + (y > m2);
        packed4 |= idx << (8 * k);
      }
      *reinterpret_cast<uint32_t*>(vcode + r * HEAD_DIM + 4 * lane) = packed4;
      if (lane == 0) vnorm[r] = __float2half_rn(n);
    }
  }
  __syncthreads();
  // ---- assemble native words ----
  uint32_t* kres = reinterpret_cast<uint32_t*>(blk);
  if (g.layout == 1) {
    // row order: word w of the K residual = (chunk k, token r, word j); of the V codes = (chunk cc, channel c, word j)
    for (int w = tid; w < page * 16; w += blockDim.x) {
      const int j = w & 3, r = (w >> 2) & 127, k = w >> 9;
      const int base = (j < 2) ? 16 * k + 8 * j : 64 + 16 * k + 8 * (j - 2);
      uint32_t word = 0;
#pragma unroll
      for (int e = 0; e < 2; ++e)
#pragma unroll
        for (int i = 0; i < 4; ++i) word |= ((uint32_t)kcode[r * HEAD_DIM + base + 2 * i + e] & 0xFu) << (16 * e + 4 * i);
      kres[w] = word;
    }
    uint32_t* vw1 = reinterpret_cast<uint32_t*>(blk + k2b_off_vcode(page, group));
    for (int w = tid; w < page * 8; w += blockDim.x) {
      const int j = w & 3, c = (w >> 2) & 127, cc = w >> 9;
      uint32_t word = 0;
#pragma unroll
      for (int tau = 0; tau < 16; ++tau)
        word |= (uint32_t)vcode[(64 * cc + 16 * j + tau) * HEAD_DIM + c] << (tau < 8 ? 4 * tau : 4 * (tau - 8) + 2);
      vw1[w] = word;
    }
    return;
  }
  for (int w = tid; w < page * 16; w += blockDim.x) {
    const int q = w & 3, ln = (w >> 2) & 31, th = (w >> 7) & 1, wr = w >> 8;
    const int gg = ln >> 2, t = ln & 3;
    const int r = wr * 16 + th * 8 + gg;
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 2; ++e)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = 8 * (4 * q + i) + 2 * t + e;
        word |= ((uint32_t)kcode[r * HEAD_DIM + c] & 0xFu) << (16 * e + 4 * i);
      }
    kres[w] = word;
  }
  uint32_t* vw = reinterpret_cast<uint32_t*>(blk + k2b_off_vcode(page, group));
  for (int w = tid; w < page * 8; w += blockDim.x) {
    const int j = w & 3, ln = (w >> 2) & 31, wr = w >> 7;
    const int gg = ln >> 2, t = ln & 3;
    uint32_t word = 0;
#pragma unroll
    for (int hs = 0; hs < 2; ++hs)
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int mt = 2 * j + hs, c = 16 * mt + 8 * (a & 1) + gg;
          const int r = wr * 16 + 8 * (a >> 1) + 2 * t + e;
          word |= (uint32_t)vcode[r * HEAD_DIM + c] << (16 * hs + 4 * (2 * (a & 1) + e) + 2 * (a >> 1));
        }
    vw[w] = word;
  }
}

// ---------------------------------------------------------------------------------------------
// Exporter: native page -> the reference's stacked tensors.  One block per (page, head).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int k2b_read_kcode(int lay, const uint32_t* kres, int r, int c) {
  int w, b;
  k2b_kres_loc(lay, r, c, w, b);
  const int nib = (kres[w] >> b) & 0xF;
  return (nib ^ 8) - 8;
}
__device__ __forceinline__ int k2b_read_vcode(int lay, const uint32_t* vw, int r, int c) {
  int w, b;
  k2b_vcode_loc(lay, r, c, w, b);
  return (vw[w] >> b) & 3;
}

__global__ void k2b_export_kernel(K2bGeom g, const uint8_t* __restrict__ pages, const __half* __restrict__ coefs,
                                  const int32_t* __restrict__ slots, __half* __restrict__ us,
                                  uint8_t* __restrict__ res_int_packed, __half* __restrict__ res_scale,
                                  uint8_t* __restrict__ v_idx_packed, __half* __restrict__ v_norm) {
  const int n = blockIdx.x / g.h_kv, h = blockIdx.x % g.h_kv;
  const int slot = slots[n], page = g.page, group = g.group, rank = g.rank;
  const int C = g.h_kv * HEAD_DIM, ngrp = page / group;
  const uint8_t* blk = pages + ((int64_t)slot * g.h_kv + h) * k2b_page_block_bytes(page, group);
  const uint32_t* kres = reinterpret_cast<const uint32_t*>(blk);
  const __half* kscale = reinterpret_cast<const __half*>(blk + k2b_off_kscale(page));
  const uint32_t* vw = reinterpret_cast<const uint32_t*>(blk + k2b_off_vcode(page, group));
  const __half* vn = reinterpret_cast<const __half*>(blk + k2b_off_vnorm(page, group));
  // res_int_packed[n][h*128 + c][r/2]
  for (int o = threadIdx.x; o < HEAD_DIM * page / 2; o += blockDim.x) {
    const int c = o / (page / 2), rb = o % (page / 2);
    const uint32_t lo = k2b_read_kcode(g.layout, kres, 2 * rb, c) & 0xF, hi = k2b_read_kcode(g.layout, kres, 2 * rb + 1, c) & 0xF;
    res_int_packed[((int64_t)n * C + h * HEAD_DIM + c) * (page / 2) + rb] = (uint8_t)(lo | (hi << 4));
  }
  for (int o = threadIdx.x; o < HEAD_DIM * ngrp; o += blockDim.x) {
    const int c = o / ngrp, gi = o % ngrp;
    res_scale[((int64_t)n * C + h * HEAD_DIM + c) * ngrp + gi] = kscale[k2b_kscale_idx(g.layout, gi, c)];
  }
  // v_idx_packed[n][r][(h*128 + c)/4]
  for (int o = threadIdx.x; o < page * HEAD_DIM / 4; o += blockDim.x) {
    const int r = o / (HEAD_DIM / 4), cb = o % (HEAD_DIM / 4);
    uint32_t b = 0;
    for (int k = 0; k < 4; ++k) b |= (uint32_t)k2b_read_vcode(g.layout, vw, r, 4 * cb + k) << (2 * k);
    v_idx_packed[((int64_t)n * page + r) * (C / 4) + h * (HEAD_DIM / 4) + cb] = (uint8_t)b;
  }
  for (int r = threadIdx.x; r < page; r += blockDim.x) v_norm[((int64_t)n * page + r) * g.h_kv + h] = vn[r];
  if (h < g.n_coef_heads) {
    const __half* cblk = coefs + ((int64_t)slot * g.n_coef_heads + h) * (page * rank);
    for (int o = threadIdx.x; o < page * rank; o += blockDim.x)
      us[((int64_t)n * g.n_coef_heads + h) * (page * rank) + o] = cblk[k2b_coef_idx(g.layout, o / rank, o % rank, rank)];
  }
}

// ---------------------------------------------------------------------------------------------
// Page dequantizer (bmx: src/bmx/cache/codecs.py:639-649, 837-842).  One block per (page, head).
//   K[r,c] = L[r,c] + float(code) * float(scale16)   with L as in the quantizer
//   V[r,:] = (fwht(cb[idx] / sqrt(128)) * signs) * norm
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128) k2b_dequant_kernel(K2bGeom g, const uint8_t* __restrict__ pages,
                                                          const __half* __restrict__ coefs,
                                                          const __half* __restrict__ basis16,
                                                          const float* __restrict__ signs,
                                                          const float* __restrict__ codebook,
                                                          const int32_t* __restrict__ slots, float* __restrict__ k_out,
                                                          float* __restrict__ v_out) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* us = reinterpret_cast<float*>(smem);
  const int n = blockIdx.x / g.h_kv, h = blockIdx.x % g.h_kv;
  const int slot = slots[n], page = g.page, group = g.group, rank = g.rank;
  const int C = g.h_kv * HEAD_DIM;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint8_t* blk = pages + ((int64_t)slot * g.h_kv + h) * k2b_page_block_bytes(page, group);
  const uint32_t* kres = reinterpret_cast<const uint32_t*>(blk);
  const __half* kscale = reinterpret_cast<const __half*>(blk + k2b_off_kscale(page));
  const uint32_t* vw = reinterpret_cast<const uint32_t*>(blk + k2b_off_vcode(page, group));
  const __half* vn = reinterpret_cast<const __half*>(blk + k2b_off_vnorm(page, group));
  const int ch = (g.n_coef_heads == 1) ? 0 : h;
  const __half* cblk = coefs + ((int64_t)slot * g.n_coef_heads + ch) * (page * rank);
  if (k_out) {
    for (int o = tid; o < page * rank; o += blockDim.x) us[o] = __half2float(cblk[k2b_coef_idx(g.layout, o / rank, o % rank, rank)]);
    __syncthreads();
    const int c = tid;
    float vb[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) vb[i] = (i < rank) ? __half2float(basis16[((int64_t)h * HEAD_DIM + c) * rank + i]) : 0.f;
    for (int r = 0; r < page; ++r) {
      float L = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i < rank) L = fmaf(us[r * rank + i], vb[i], L);
      const float res = (float)k2b_read_kcode(g.layout, kres, r, c) * __half2float(kscale[k2b_kscale_idx(g.layout, r / group, c)]);
      k_out[((int64_t)n * page + r) * C + h * HEAD_DIM + c] = L + res;
    }
  }
  if (v_out) {
    float sg[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) sg[k] = signs[4 * lane + k];
    const float sqrt_d = 11.313708498984761f;
    for (int r = warp; r < page; r += 4) {
      float x[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = codebook[k2b_read_vcode(g.layout, vw, r, 4 * lane + k)] / sqrt_d;
      fwht128_warp(x, lane);
      const float nn = __half2float(vn[r]);
#pragma unroll
      for (int k = 0; k < 4; ++k) v_out[((int64_t)n * page + r) * C + h * HEAD_DIM + 4 * lane + k] = (x[k] * sg[k]) * nn;
    }
  }
}

static int check_geom(const bmxk_k2b_geom* g, const char* who) {
  BMXK_REQUIRE(g != nullptr, "%s: null geometry", who);
  BMXK_REQUIRE(g->h_kv >= 1 && g->h_kv <= 64, "%s: h_kv=%d out of range", who, g->h_kv);
  BMXK_REQUIRE(g->n_q_groups >= 1 && g->n_q_groups <= 8, "%s: n_q_groups=%d must be in 1..8", who, g->n_q_groups);
  BMXK_REQUIRE(g->page == 64 || g->page == 128, "%s: page=%d must be 64 or 128", who, g->page);
  BMXK_REQUIRE(g->rank == 16 || g->rank == 32, "%s: rank=%d must be 16 or 32", who, g->rank);
  BMXK_REQUIRE((g->group == 32 || g->group == 64 || g->group == 128) && g->page % g->group == 0,
               "%s: group=%d must be 32/64/128 and divide page=%d", who, g->group, g->page);
  BMXK_REQUIRE(g->n_coef_heads == 1 || g->n_coef_heads == g->h_kv, "%s: n_coef_heads=%d must be 1 or h_kv", who,
               g->n_coef_heads);
  BMXK_REQUIRE(g->kbits >= 2 && g->kbits <= 4, "%s: kbits=%d must be in 2..4", who, g->kbits);
  BMXK_REQUIRE(g->vbits == 2, "%s: vbits=%d (only 2-bit value codes have a kernel)", who, g->vbits);
  BMXK_REQUIRE(g->layout == 0 || (g->layout == 1 && g->page == 128), "%s: layout=%d must be 0, or 1 with page=128", who,
               g->layout);
  return BMXK_OK;
}

static K2bGeom to_geom(const bmxk_k2b_geom* g) {
  K2bGeom o;
  o.h_kv = g->h_kv, o.n_q_groups = g->n_q_groups, o.page = g->page, o.rank = g->rank, o.group = g->group;
  o.n_coef_heads = g->n_coef_heads, o.kbits = g->kbits, o.vbits = g->vbits, o.layout = g->layout;
  return o;
}

template <typename T>
static int append_impl(const bmxk_k2b_geom* g, const void* k_pre, const void* v, int64_t ss, int64_t sh, int64_t st,
                       const float* basis, const float* signs, const float* codebook, const int32_t* slots, int n_seq,
                       int n_pages, void* pages, void* coefs, cudaStream_t s) {
  const K2bGeom gg = to_geom(g);
  const int items = n_seq * n_pages;
  k2b_project_kernel<T><<<items * g->n_coef_heads, 256, 0, s>>>(gg, (const T*)k_pre, ss, sh, st, basis, slots, n_pages,
                                                                 (__half*)coefs);
  int rc = check_launch("bmxk_k2b_append(project)");
  if (rc) return rc;
  const size_t smem = 2 * g->page * HEAD_DIM + (size_t)g->page * g->rank * 4;
  k2b_quant_page_kernel<T><<<items * g->h_kv, 128, smem, s>>>(gg, (const T*)k_pre, (const T*)v, ss, sh, st, basis, signs,
                                                              codebook, slots, n_pages, (uint8_t*)pages,
                                                              (const __half*)coefs);
  return check_launch("bmxk_k2b_append(quantize)");
}

}  // namespace bmxk

using namespace bmxk;

extern "C" {

size_t bmxk_k2b_page_block_bytes(const bmxk_k2b_geom* g) {
  return g ? (size_t)k2b_page_block_bytes(g->page, g->group) : 0;
}
size_t bmxk_k2b_coef_block_bytes(const bmxk_k2b_geom* g) { return g ? (size_t)k2b_coef_block_bytes(g->page, g->rank) : 0; }

int bmxk_k2b_append(const bmxk_k2b_geom* g, const void* k_pre, const void* v, int src_dtype, int64_t stride_seq,
                    int64_t stride_head, int64_t stride_tok, const float* basis_f32, const float* signs,
                    const float* codebook, const int32_t* slots, int n_seq, int n_pages, void* pages, void* coefs,
                    void* stream) {
  int rc = check_geom(g, "bmxk_k2b_append");
  if (rc) return rc;
  BMXK_REQUIRE(n_seq >= 0 && n_pages >= 0, "bmxk_k2b_append: negative counts");
  if (n_seq == 0 || n_pages == 0) return BMXK_OK;
  BMXK_REQUIRE(k_pre && v && basis_f32 && signs && codebook && slots && pages && coefs, "bmxk_k2b_append: null pointer");
  BMXK_REQUIRE(stride_tok >= HEAD_DIM, "bmxk_k2b_append: stride_tok=%lld < 128", (long long)stride_tok);
  BMXK_REQUIRE((int64_t)n_seq * n_pages * g->h_kv < (1LL << 31), "bmxk_k2b_append: too many pages in one call");
  cudaStream_t s = (cudaStream_t)stream;
  switch (src_dtype) {
    case BMXK_DTYPE_F16:
      return append_impl<__half>(g, k_pre, v, stride_seq, stride_head, stride_tok, basis_f32, signs, codebook, slots,
                                 n_seq, n_pages, pages, coefs, s);
    case BMXK_DTYPE_BF16:
      return append_impl<__nv_bfloat16>(g, k_pre, v, stride_seq, stride_head, stride_tok, basis_f32, signs, codebook,
                                        slots, n_seq, n_pages, pages, coefs, s);
    case BMXK_DTYPE_F32:
      return append_impl<float>(g, k_pre, v, stride_seq, stride_head, stride_tok, basis_f32, signs, codebook, slots,
                                n_seq, n_pages, pages, coefs, s);
    default:
      set_error("bmxk_k2b_append: unknown src_dtype %d", src_dtype);
      return BMXK_ERR_INVALID;
  }
}

int bmxk_k2b_export_stacks(const bmxk_k2b_geom* g, const void* pages, const void* coefs, const int32_t* slots, int n,
                           void* us, uint8_t* res_int_packed, void* res_scale, uint8_t* v_idx_packed, void* v_norm,
                           void* stream) {
  int rc = check_geom(g, "bmxk_k2b_export_stacks");
  if (rc) return rc;
  BMXK_REQUIRE(n >= 0, "bmxk_k2b_export_stacks: n < 0");
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(pages && coefs && slots && us && res_int_packed && res_scale && v_idx_packed && v_norm,
               "bmxk_k2b_export_stacks: null pointer");
  k2b_export_kernel<<<n * g->h_kv, 256, 0, (cudaStream_t)stream>>>(to_geom(g), (const uint8_t*)pages,
                                                                  (const __half*)coefs, slots, (__half*)us,
                                                                  res_int_packed, (__half*)res_scale, v_idx_packed,
                                                                  (__half*)v_norm);
  return check_launch("bmxk_k2b_export_stacks");
}

int bmxk_k2b_dequant_pages(const bmxk_k2b_geom* g, const void* pages, const void* coefs, const void* basis_f16,
                           const float* signs, const float* codebook, const int32_t* slots, int n, float* k_out,
                           float* v_out, void* stream) {
  int rc = check_geom(g, "bmxk_k2b_dequant_pages");
  if (rc) return rc;
  BMXK_REQUIRE(n >= 0, "bmxk_k2b_dequant_pages: n < 0");
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(pages && coefs && slots, "bmxk_k2b_dequant_pages: null pointer");
  BMXK_REQUIRE(!k_out || basis_f16, "bmxk_k2b_dequant_pages: keys need basis_f16");
  BMXK_REQUIRE(!v_out || (signs && codebook), "bmxk_k2b_dequant_pages: values need signs and codebook");
  const size_t smem = (size_t)g->page * g->rank * 4;
  k2b_dequant_kernel<<<n * g->h_kv, 128, smem, (cudaStream_t)stream>>>(to_geom(g), (const uint8_t*)pages,
                                                                      (const __half*)coefs, (const __half*)basis_f16,
                                                                      signs, codebook, slots, k_out, v_out);
  return check_launch("bmxk_k2b_dequant_pages");
}

}  // extern "C"
