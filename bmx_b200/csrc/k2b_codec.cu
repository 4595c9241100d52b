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

// Four consecutive source elements as float32 (exact for every source type).  `vec`: the address is aligned for one
// wide load (the host checks base pointer and strides once per call).
template <typename T>
__device__ __forceinline__ void load4_as_float(const T* p, bool vec, float (&f)[4]);
template <>
__device__ __forceinline__ void load4_as_float<__half>(const __half* p, bool vec, float (&f)[4]) {
  if (vec) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __half22float2(u32_as_h2(u.x)), b = __half22float2(u32_as_h2(u.y));
    f[0] = a.x, f[1] = a.y, f[2] = b.x, f[3] = b.y;
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) f[k] = __half2float(p[k]);
  }
}
template <>
__device__ __forceinline__ void load4_as_float<__nv_bfloat16>(const __nv_bfloat16* p, bool vec, float (&f)[4]) {
  if (vec) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    f[0] = __uint_as_float(u.x << 16), f[1] = __uint_as_float(u.x & 0xFFFF0000u);
    f[2] = __uint_as_float(u.y << 16), f[3] = __uint_as_float(u.y & 0xFFFF0000u);
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) f[k] = __bfloat162float(p[k]);
  }
}
template <>
__device__ __forceinline__ void load4_as_float<float>(const float* p, bool vec, float (&f)[4]) {
  if (vec) {
    const float4 u = *reinterpret_cast<const float4*>(p);
    f[0] = u.x, f[1] = u.y, f[2] = u.z, f[3] = u.w;
  } else {
#pragma unroll
    for (int k = 0; k < 4; ++k) f[k] = p[k];
  }
}

constexpr int KF_STRIDE = 132;  // floats per staged key row: consecutive rows start 16 bytes apart modulo 128
                                // (4 consecutive rows x one 128-bit load each fall in distinct bank groups)

// ---------------------------------------------------------------------------------------------
// Projection  Us = M @ V  (bmx: src/bmx/cache/packed_streaming.py:518-520), rounded to fp16 and
// written to the coefficient block, for a basis that spans several heads (the fused page kernel below
// projects by itself when every head has its own basis).  One block per (item, coef head, 32 rows);
// thread -> (row, four consecutive i).  Order per output: acc = 0; heads ascending, c ascending:
// acc = fmaf(M[r,c], V[c,i], acc).  Each head's 32 x 128 key rows and 128 x rank basis slice are staged
// in shared memory so that global loads are coalesced and every operand is read with 128-bit loads.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void k2b_project_kernel(K2bGeom g, const T* __restrict__ k_pre, int64_t stride_seq, int64_t stride_head,
                                   int64_t stride_tok, const float* __restrict__ basis, const int32_t* __restrict__ slots,
                                   int n_pages, __half* __restrict__ coefs, int vec) {
  extern __shared__ __align__(16) uint8_t smem[];
  float* ks = reinterpret_cast<float*>(smem);   // [32][KF_STRIDE]
  float* bs = ks + 32 * KF_STRIDE;              // [128][rank]
  const int rank = g.rank, IQ = rank >> 2, n_rb = g.page >> 5;
  int blk = blockIdx.x;
  const int rb = blk % n_rb;
  blk /= n_rb;
  const int ch = blk % g.n_coef_heads, item = blk / g.n_coef_heads;
  const int seq = item / n_pages, pg = item % n_pages;
  const int slot = slots[item];
  const int h0 = (g.n_coef_heads == 1) ? 0 : ch, nh = (g.n_coef_heads == 1) ? g.h_kv : 1;
  const int tid = threadIdx.x, rl = tid / IQ, iq = tid % IQ;
  const T* src = k_pre + seq * stride_seq + ((int64_t)pg * g.page + rb * 32) * stride_tok;
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  for (int h = h0; h < h0 + nh; ++h) {
    for (int o = tid; o < 32 * 32; o += blockDim.x) {
      const int r = o >> 5, c4 = o & 31;
      float f[4];
      load4_as_float<T>(src + h * stride_head + r * stride_tok + 4 * c4, vec != 0, f);
      *reinterpret_cast<float4*>(ks + r * KF_STRIDE + 4 * c4) = make_float4(f[0], f[1], f[2], f[3]);
    }
    const float4* bsrc = reinterpret_cast<const float4*>(basis + (int64_t)h * HEAD_DIM * rank);
    for (int o = tid; o < HEAD_DIM * IQ; o += blockDim.x) reinterpret_cast<float4*>(bs)[o] = bsrc[o];
    __syncthreads();
#pragma unroll 4
    for (int c4 = 0; c4 < 32; ++c4) {
      const float4 m = *reinterpret_cast<const float4*>(ks + rl * KF_STRIDE + 4 * c4);
      const float mm[4] = {m.x, m.y, m.z, m.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float4 vv = *reinterpret_cast<const float4*>(bs + (4 * c4 + k) * rank + 4 * iq);
        acc[0] = fmaf(mm[k], vv.x, acc[0]), acc[1] = fmaf(mm[k], vv.y, acc[1]);
        acc[2] = fmaf(mm[k], vv.z, acc[2]), acc[3] = fmaf(mm[k], vv.w, acc[3]);
      }
    }
    __syncthreads();
  }
  __half* out = coefs + ((int64_t)slot * g.n_coef_heads + ch) * (g.page * rank);
  const int r = rb * 32 + rl;
#pragma unroll
  for (int j = 0; j < 4; ++j) out[k2b_coef_idx(g.layout, r, 4 * iq + j, rank)] = __float2half_rn(acc[j]);
}

// Coefficients computed elsewhere (a projection summed over the GPUs that hold the other heads of a basis spanning all
// heads): us (n_seq, n_pages * page, rank) float32, rounded to fp16 into the coefficient blocks.  One block per page.
__global__ void k2b_store_coefs_kernel(K2bGeom g, const float* __restrict__ us, const int32_t* __restrict__ slots, int n_pages,
                                       __half* __restrict__ coefs) {
  const int item = blockIdx.x, seq = item / n_pages, pg = item % n_pages, rank = g.rank;
  const float* src = us + ((int64_t)seq * n_pages + pg) * g.page * rank;
  __half* out = coefs + (int64_t)slots[item] * (g.page * rank);  // one coefficient block per slot (n_coef_heads == 1)
  for (int o = threadIdx.x; o < g.page * rank; o += blockDim.x) out[k2b_coef_idx(g.layout, o / rank, o % rank, rank)] = __float2half_rn(src[o]);
}

// ---------------------------------------------------------------------------------------------
// Page quantizer.  One block of 256 threads per (item, kv head); two blocks share an SM.
//   staging: the head's key page (float32, KF_STRIDE per row) and its basis slice go to shared memory.
//   coefficients (FUSED: one basis per head): thread = (row slot, four i), ROWS rows each;
//           Us[r,i] = fmaf chain over c ascending, rounded to fp16, written to the coefficient block.
//           Otherwise the coefficients come from the coefficient block the projection kernel wrote.
//   keys  : thread = (channel, half of the page).  L[r,c] = sum_i Us16[r,i] V16[c,i] (fmaf, i ascending), R = M - L
//           is computed ONCE and kept in registers; per group of `group` tokens scale = max(absmax, 1e-12) / qmax,
//           code = rint(R / scale) clamped to [-qmax-1, qmax]
//           (bmx: src/bmx/cache/codecs.py:677-695, src/bmx/quant/rtn.py:34-44)
//   values: warp = token, two tokens in flight.  n = fp16(max(sqrt(sum v^2), 1e-12)); u = v / n; y = fwht(u * signs);
//           idx = #{mid_k < y * sqrt(128)}        (bmx: src/bmx/cache/codecs.py:616-636)
// Codes are staged in shared memory (over the key page, which is dead by then) and assembled into whole
// 32-bit words of the native layout.
// ---------------------------------------------------------------------------------------------
constexpr int QP_THREADS = 256;
// floats of the region that first holds the basis slice and the coefficients and later the two code buffers
__host__ __device__ constexpr int quant_region_floats(int page, int rank) {
  return (HEAD_DIM * (rank + 4) + page * rank) > (2 * page * HEAD_DIM / 4) ? (HEAD_DIM * (rank + 4) + page * rank) : (2 * page * HEAD_DIM / 4);
}

template <typename T, int PAGE, bool FUSED>
__global__ void __launch_bounds__(QP_THREADS, 2) k2b_quant_page_kernel(K2bGeom g, const T* __restrict__ k_pre,
                                                                        const T* __restrict__ v, int64_t stride_seq,
                                                                        int64_t stride_head, int64_t stride_tok,
                                                                        const float* __restrict__ basis,
                                                                        const float* __restrict__ signs,
                                                                        const float* __restrict__ codebook,
                                                                        const int32_t* __restrict__ slots, int n_pages,
                                                                        uint8_t* __restrict__ pages, __half* __restrict__ coefs,
                                                                        int vec) {
  extern __shared__ __align__(16) uint8_t smem[];
  constexpr int HALF_ROWS = PAGE / 2, SUBS = PAGE / 32;  // rows per thread in the key phase; 32-row sub-blocks
  const int rank = g.rank, group = g.group, BS = rank + 4;  // basis rows padded: eight consecutive rows, one 128-bit load each, conflict free
  float* kf = reinterpret_cast<float*>(smem);                 // [PAGE][KF_STRIDE] key page, overwritten in place by the residual
  float* bs = kf + PAGE * KF_STRIDE;                           // [128][rank + 4] basis slice (float32)
  float* us = bs + HEAD_DIM * BS;                              // [PAGE][rank] fp16-valued coefficients
  int8_t* kcode = reinterpret_cast<int8_t*>(bs);               // [PAGE][128]   } over the basis and the coefficients
  uint8_t* vcode = reinterpret_cast<uint8_t*>(bs) + PAGE * HEAD_DIM;  // [PAGE][128] } once they are dead
  float* amax_s = bs + quant_region_floats(PAGE, rank);        // [SUBS][128] absmax of 32-row sub-blocks

  const int item = blockIdx.x / g.h_kv, h = blockIdx.x % g.h_kv;
  const int seq = item / n_pages, pg = item % n_pages;
  const int slot = slots[item];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ch = (g.n_coef_heads == 1) ? 0 : h;
  __half* cblk = coefs + ((int64_t)slot * g.n_coef_heads + ch) * (PAGE * rank);
  uint8_t* blk = pages + ((int64_t)slot * g.h_kv + h) * k2b_page_block_bytes(PAGE, group);
  const T* ksrc = k_pre + seq * stride_seq + h * stride_head + (int64_t)pg * PAGE * stride_tok;
  const T* vsrc = v + seq * stride_seq + h * stride_head + (int64_t)pg * PAGE * stride_tok;

  // ---- staging ----
  for (int o0 = 0; o0 < PAGE * 32; o0 += QP_THREADS * 8) {
    float f[8][4];
#pragma unroll
    for (int u = 0; u < 8; ++u) {  // eight wide loads in flight per thread
      const int o = o0 + u * QP_THREADS + tid, r = o >> 5, c4 = o & 31;
      load4_as_float<T>(ksrc + r * stride_tok + 4 * c4, vec != 0, f[u]);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int o = o0 + u * QP_THREADS + tid, r = o >> 5, c4 = o & 31;
      *reinterpret_cast<float4*>(kf + r * KF_STRIDE + 4 * c4) = make_float4(f[u][0], f[u][1], f[u][2], f[u][3]);
    }
  }
  {
    const float4* bsrc = reinterpret_cast<const float4*>(basis + (int64_t)h * HEAD_DIM * rank);
    const int IQ = rank >> 2;
    for (int o = tid; o < HEAD_DIM * IQ; o += QP_THREADS) {
      const int c = o / IQ, i4 = o % IQ;
      *reinterpret_cast<float4*>(bs + c * BS + 4 * i4) = bsrc[o];
    }
  }
  if (!FUSED)
    for (int o = tid; o < PAGE * rank; o += QP_THREADS) us[o] = __half2float(cblk[k2b_coef_idx(g.layout, o / rank, o % rank, rank)]);
  __syncthreads();

  // ---- coefficients (one basis per head) ----
  if (FUSED) {
    const int IQ = rank >> 2, slots_r = QP_THREADS / IQ;  // 32 (rank 32) or 64 (rank 16) rows in flight
    const int rs = tid / IQ, iq = tid % IQ;
    for (int r0 = 0; r0 < PAGE; r0 += 4 * slots_r) {      // up to four rows per thread and pass
      float acc[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a) acc[a][0] = acc[a][1] = acc[a][2] = acc[a][3] = 0.f;
#pragma unroll 2
      for (int c4 = 0; c4 < 32; ++c4) {
        float mm[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const int r = min(r0 + a * slots_r + rs, PAGE - 1);
          const float4 m = *reinterpret_cast<const float4*>(kf + r * KF_STRIDE + 4 * c4);
          mm[a][0] = m.x, mm[a][1] = m.y, mm[a][2] = m.z, mm[a][3] = m.w;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float4 vv = *reinterpret_cast<const float4*>(bs + (4 * c4 + k) * BS + 4 * iq);
#pragma unroll
          for (int a = 0; a < 4; ++a) {
            acc[a][0] = fmaf(mm[a][k], vv.x, acc[a][0]), acc[a][1] = fmaf(mm[a][k], vv.y, acc[a][1]);
            acc[a][2] = fmaf(mm[a][k], vv.z, acc[a][2]), acc[a][3] = fmaf(mm[a][k], vv.w, acc[a][3]);
          }
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const int r = r0 + a * slots_r + rs;
        if (r < PAGE) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __half hv = __float2half_rn(acc[a][j]);
            us[r * rank + 4 * iq + j] = __half2float(hv);
            cblk[k2b_coef_idx(g.layout, r, 4 * iq + j, rank)] = hv;
          }
        }
      }
    }
    __syncthreads();
  }

  // ---- keys: thread = (channel, half of the page); the residuals stay in registers ----
  {
    const int c = tid & 127, hf = tid >> 7, r_base = hf * HALF_ROWS;
    float vb[32];
#pragma unroll
    for (int i4 = 0; i4 < 8; ++i4) {
      if (4 * i4 < rank) {
        const float4 t = *reinterpret_cast<const float4*>(bs + c * BS + 4 * i4);
        vb[4 * i4] = half_round(t.x), vb[4 * i4 + 1] = half_round(t.y), vb[4 * i4 + 2] = half_round(t.z), vb[4 * i4 + 3] = half_round(t.w);
      } else {
        vb[4 * i4] = vb[4 * i4 + 1] = vb[4 * i4 + 2] = vb[4 * i4 + 3] = 0.f;
      }
    }
#pragma unroll
    for (int sb = 0; sb < HALF_ROWS / 32; ++sb) {
      float am = 0.f;
#pragma unroll 4
      for (int rr = 0; rr < 32; ++rr) {
        const int r = r_base + 32 * sb + rr;
        float L = 0.f;
#pragma unroll
        for (int i4 = 0; i4 < 8; ++i4)
          if (4 * i4 < rank) {
            const float4 u = *reinterpret_cast<const float4*>(us + r * rank + 4 * i4);
            L = fmaf(u.x, vb[4 * i4], L), L = fmaf(u.y, vb[4 * i4 + 1], L), L = fmaf(u.z, vb[4 * i4 + 2], L), L = fmaf(u.w, vb[4 * i4 + 3], L);
          }
        const float res = kf[r * KF_STRIDE + c] - L;
        kf[r * KF_STRIDE + c] = res;  // this thread is the only one that touches column c of these rows
        am = fmaxf(am, fabsf(res));
      }
      amax_s[(hf * (HALF_ROWS / 32) + sb) * HEAD_DIM + c] = am;
    }
    __syncthreads();  // basis and coefficients are dead from here on: the code buffers may overwrite them
    const float qmax = (float)((1 << (g.kbits - 1)) - 1);
    __half* kscale = reinterpret_cast<__half*>(blk + k2b_off_kscale(PAGE));
    const int subs_per_group = group >> 5;
#pragma unroll
    for (int sb = 0; sb < HALF_ROWS / 32; ++sb) {
      const int gsb = hf * (HALF_ROWS / 32) + sb, grp = gsb / subs_per_group;
      float amax = 0.f;
      for (int k = 0; k < subs_per_group; ++k) amax = fmaxf(amax, amax_s[(grp * subs_per_group + k) * HEAD_DIM + c]);
      const float scale = fmaxf(amax, 1e-12f) / qmax;
      if (gsb == grp * subs_per_group) kscale[k2b_kscale_idx(g.layout, grp, c)] = __float2half_rn(scale);
#pragma unroll 8
      for (int rr = 0; rr < 32; ++rr) {
        const int r = r_base + 32 * sb + rr;
        float q = rintf(kf[r * KF_STRIDE + c] / scale);
        q = fminf(fmaxf(q, -qmax - 1.f), qmax);
        kcode[r * HEAD_DIM + c] = (int8_t)q;
      }
    }
    (void)SUBS;
  }
  // ---- values: warp = token, two tokens in flight ----
  {
    const float c0 = codebook[0], c1 = codebook[1], c2 = codebook[2], c3 = codebook[3];
    const float m0 = (c0 + c1) / 2.f, m1 = (c1 + c2) / 2.f, m2 = (c2 + c3) / 2.f;
    float sg[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) sg[k] = signs[4 * lane + k];
    __half* vnorm = reinterpret_cast<__half*>(blk + k2b_off_vnorm(PAGE, group));
    constexpr int NW = QP_THREADS / 32;
    for (int r0 = warp; r0 < PAGE; r0 += 2 * NW) {
      float x[2][4];
#pragma unroll
      for (int u = 0; u < 2; ++u) load4_as_float<T>(vsrc + (r0 + u * NW) * stride_tok + 4 * lane, vec != 0, x[u]);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int r = r0 + u * NW;
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < 4; ++k) ss = fmaf(x[u][k], x[u][k], ss);
#pragma unroll
        for (int m = 16; m >= 1; m >>= 1) ss = ss + __shfl_xor_sync(0xffffffffu, ss, m);
        const float n = half_round(fmaxf(sqrtf(ss), 1e-12f));
#pragma unroll
        for (int k = 0; k < 4; ++k) x[u][k] = (x[u][k] / n) * sg[k];
        fwht128_warp(x[u], lane);
        const float sqrt_d = 11.313708498984761f;
        uint32_t packed4 = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float y = x[u][k] * sqrt_d;
          const uint32_t idx = (y > m0) + (y > m1) + (y > m2);
          packed4 |= idx << (8 * k);
        }
        *reinterpret_cast<uint32_t*>(vcode + r * HEAD_DIM + 4 * lane) = packed4;
        if (lane == 0) vnorm[r] = __float2half_rn(n);
      }
    }
  }
  const int page = PAGE;
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

// ---------------------------------------------------------------------------------------------
// Page dequantizer of the dense prefill route: the same arithmetic as above, then the rotation of the keys at their
// absolute positions in float32 and ONE rounding to the model's 16-bit type, written straight into
// (batch, h_kv, row_stride, 128) tensors whose tail the caller fills with the fp16 window.  What bmx builds in float32,
// rotates and casts (src/bmx/cache/chunked_attention.py:320-395) costs 20 bytes of transient per element this way; here 4.
// One block per (sequence, page, head).
// ---------------------------------------------------------------------------------------------
template <typename OutT>
__device__ __forceinline__ OutT to_out(float x);
template <>
__device__ __forceinline__ __half to_out<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 to_out<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

constexpr int DD_THREADS = 256, DD_BP = 40, DD_KP = 136;  // halves per staged coefficient / basis row and per staged key row

template <typename OutT>
__device__ __forceinline__ uint32_t pack2_out(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2_out<__half>(float lo, float hi) {
  const __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2_out<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// The page block, the coefficients (as plain rows) and the head's basis are staged in shared memory; the low-rank
// product runs as mma.sync (fp16 operands are the stored values, fp32 accumulators), each warp 16 token rows; a
// thread then holds both channels of every rotary pair of its rows, adds code x scale, rotates and stages the rows
// for 16-byte stores.  Values: one warp per token row (butterflies over the lanes), 8-byte stores.
template <typename OutT>
__global__ void __launch_bounds__(DD_THREADS) k2b_dequant_dense_kernel(K2bGeom g, const uint8_t* __restrict__ pages,
                                                                       const __half* __restrict__ coefs, const __half* __restrict__ basis16,
                                                                       const float* __restrict__ signs, const float* __restrict__ codebook,
                                                                       const int32_t* __restrict__ page_table, int table_stride, int n_pg,
                                                                       const __half* __restrict__ rope_cos, const __half* __restrict__ rope_sin,
                                                                       int64_t pos_offset, OutT* __restrict__ k_out, OutT* __restrict__ v_out,
                                                                       int64_t row_stride) {
  extern __shared__ __align__(16) uint8_t smem[];
  const int b = blockIdx.x / n_pg, j = blockIdx.x % n_pg, h = blockIdx.y;
  const int slot = page_table[(int64_t)b * table_stride + j], page = g.page, group = g.group, rank = g.rank;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
  const int PB = k2b_page_block_bytes(page, group);
  uint8_t* raw = smem;
  __half* ca = reinterpret_cast<__half*>(raw + ((PB + 15) & ~15));  // [page][DD_BP]
  __half* bb = ca + 128 * DD_BP;                                     // [128][DD_BP]
  OutT* kt = reinterpret_cast<OutT*>(bb + 128 * DD_BP);              // [page][DD_KP]
  const uint8_t* blk = pages + ((int64_t)slot * g.h_kv + h) * PB;
  const int ch = (g.n_coef_heads == 1) ? 0 : h;
  const __half* cblk = coefs + ((int64_t)slot * g.n_coef_heads + ch) * (page * rank);
  for (int o = tid; o < PB / 16; o += DD_THREADS) reinterpret_cast<uint4*>(raw)[o] = reinterpret_cast<const uint4*>(blk)[o];
  if (k_out) {
    for (int o = tid; o < page * rank; o += DD_THREADS) ca[(o / rank) * DD_BP + o % rank] = cblk[k2b_coef_idx(g.layout, o / rank, o % rank, rank)];
    for (int o = tid; o < 128 * (rank / 8); o += DD_THREADS) {
      const int c = o / (rank / 8), i8 = o % (rank / 8);
      *reinterpret_cast<uint4*>(bb + c * DD_BP + 8 * i8) = reinterpret_cast<const uint4*>(basis16 + ((int64_t)h * HEAD_DIM + c) * rank)[i8];
    }
  }
  __syncthreads();
  const uint32_t* kres = reinterpret_cast<const uint32_t*>(raw);
  const __half* kscale = reinterpret_cast<const __half*>(raw + k2b_off_kscale(page));
  const uint32_t* vw = reinterpret_cast<const uint32_t*>(raw + k2b_off_vcode(page, group));
  const __half* vn = reinterpret_cast<const __half*>(raw + k2b_off_vnorm(page, group));
  const int64_t out_row0 = ((int64_t)b * g.h_kv + h) * row_stride + (int64_t)j * page;  // first row of this page in the outputs
  if (k_out && 16 * warp < page) {
    float c[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
    for (int ks = 0; ks < rank / 16; ++ks) {
      uint32_t a0, a1, a2, a3;
      ldmatrix_x4(a0, a1, a2, a3, smem_u32(ca + (16 * warp + (lane & 15)) * DD_BP + 16 * ks + 8 * (lane >> 4)));
#pragma unroll
      for (int n2 = 0; n2 < 8; ++n2) {
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, smem_u32(bb + (16 * n2 + (lane & 7) + ((lane >> 4) << 3)) * DD_BP + 16 * ks + (((lane >> 3) & 1) << 3)));
        mma_f32acc(c[2 * n2][0], c[2 * n2][1], c[2 * n2][2], c[2 * n2][3], a0, a1, a2, a3, b0, b1);
        mma_f32acc(c[2 * n2 + 1][0], c[2 * n2 + 1][1], c[2 * n2 + 1][2], c[2 * n2 + 1][3], a0, a1, a2, a3, b2, b3);
      }
    }
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int r = 16 * warp + gq + 8 * rr, grp = r / group;
      const int64_t pos = pos_offset + (int64_t)j * page + r;
#pragma unroll
      for (int n = 0; n < 8; ++n) {  // channels 8n + 2tq + {0, 1} and their rotary partners 64 further
        const int c1 = 8 * n + 2 * tq, c2 = c1 + 64;
        float x1[2], x2[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          x1[e] = c[n][2 * rr + e] + (float)k2b_read_kcode(g.layout, kres, r, c1 + e) * __half2float(kscale[k2b_kscale_idx(g.layout, grp, c1 + e)]);
          x2[e] = c[n + 8][2 * rr + e] + (float)k2b_read_kcode(g.layout, kres, r, c2 + e) * __half2float(kscale[k2b_kscale_idx(g.layout, grp, c2 + e)]);
        }
        if (rope_cos) {  // x * cos + rotate_half(x) * sin, tables (position, 128)
          const float2 cs1 = __half22float2(*reinterpret_cast<const __half2*>(rope_cos + pos * HEAD_DIM + c1));
          const float2 sn1 = __half22float2(*reinterpret_cast<const __half2*>(rope_sin + pos * HEAD_DIM + c1));
          const float2 cs2 = __half22float2(*reinterpret_cast<const __half2*>(rope_cos + pos * HEAD_DIM + c2));
          const float2 sn2 = __half22float2(*reinterpret_cast<const __half2*>(rope_sin + pos * HEAD_DIM + c2));
          const float y10 = x1[0] * cs1.x - x2[0] * sn1.x, y11 = x1[1] * cs1.y - x2[1] * sn1.y;
          const float y20 = x2[0] * cs2.x + x1[0] * sn2.x, y21 = x2[1] * cs2.y + x1[1] * sn2.y;
          x1[0] = y10, x1[1] = y11, x2[0] = y20, x2[1] = y21;
        }
        *reinterpret_cast<uint32_t*>(kt + r * DD_KP + c1) = pack2_out<OutT>(x1[0], x1[1]);
        *reinterpret_cast<uint32_t*>(kt + r * DD_KP + c2) = pack2_out<OutT>(x2[0], x2[1]);
      }
    }
  }
  __syncthreads();
  if (k_out)
    for (int o = tid; o < page * 16; o += DD_THREADS) {
      const int r = o >> 4, c8 = o & 15;
      reinterpret_cast<uint4*>(k_out + (out_row0 + r) * HEAD_DIM)[c8] = *reinterpret_cast<const uint4*>(kt + r * DD_KP + 8 * c8);
    }
  if (v_out) {
    float sg[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) sg[k] = signs[4 * lane + k];
    const float sqrt_d = 11.313708498984761f;
    for (int r = warp; r < page; r += DD_THREADS / 32) {
      float x[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = codebook[k2b_read_vcode(g.layout, vw, r, 4 * lane + k)] / sqrt_d;
      fwht128_warp(x, lane);
      const float nn = __half2float(vn[r]);
      const uint2 w = make_uint2(pack2_out<OutT>((x[0] * sg[0]) * nn, (x[1] * sg[1]) * nn), pack2_out<OutT>((x[2] * sg[2]) * nn, (x[3] * sg[3]) * nn));
      *reinterpret_cast<uint2*>(v_out + (out_row0 + r) * HEAD_DIM + 4 * lane) = w;
    }
  }
}

static size_t dequant_dense_smem(int page, int group) {
  return (size_t)((k2b_page_block_bytes(page, group) + 15) & ~15) + (size_t)2 * 128 * DD_BP * 2 + (size_t)page * DD_KP * 2;
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

static size_t quant_smem_bytes(int page, int rank) {
  return ((size_t)page * KF_STRIDE + (size_t)quant_region_floats(page, rank) + (size_t)(page / 32) * HEAD_DIM) * sizeof(float);
}

template <typename T, int PAGE, bool FUSED>
static int launch_quant(const K2bGeom& gg, const T* k_pre, const T* v, int64_t ss, int64_t sh, int64_t st, const float* basis,
                        const float* signs, const float* codebook, const int32_t* slots, int items, int n_pages, uint8_t* pages,
                        __half* coefs, int vec, cudaStream_t s) {
  const size_t smem = quant_smem_bytes(PAGE, gg.rank);
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(k2b_quant_page_kernel<T, PAGE, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024);
    if (e != cudaSuccess) {
      configured.retract();
      set_error("bmxk_k2b_append: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return BMXK_ERR_CUDA;
    }
  }
  k2b_quant_page_kernel<T, PAGE, FUSED><<<items * gg.h_kv, QP_THREADS, smem, s>>>(gg, k_pre, v, ss, sh, st, basis, signs, codebook, slots,
                                                                                n_pages, pages, coefs, vec);
  return check_launch("bmxk_k2b_append(quantize)");
}

template <typename T>
static int append_impl(const bmxk_k2b_geom* g, const void* k_pre, const void* v, int64_t ss, int64_t sh, int64_t st,
                       const float* basis, const float* signs, const float* codebook, const int32_t* slots, int n_seq,
                       int n_pages, void* pages, void* coefs, cudaStream_t s, const float* us_given = nullptr) {
  const K2bGeom gg = to_geom(g);
  const int items = n_seq * n_pages;
  // one wide load per four source elements needs every row start aligned to it
  const uintptr_t align = 4 * sizeof(T);
  const bool vec = ((uintptr_t)k_pre % align == 0) && ((uintptr_t)v % align == 0) && (ss * sizeof(T)) % align == 0 &&
                   (sh * sizeof(T)) % align == 0 && (st * sizeof(T)) % align == 0 && ((uintptr_t)basis % 16 == 0);
  const bool fused = g->n_coef_heads == g->h_kv && !us_given;  // one basis per head: the page kernel projects by itself
  if (us_given) {
    k2b_store_coefs_kernel<<<items, 256, 0, s>>>(gg, us_given, slots, n_pages, (__half*)coefs);
    int rc = check_launch("bmxk_k2b_append_coefs(store)");
    if (rc) return rc;
  } else if (!fused) {
    BMXK_REQUIRE((uintptr_t)basis % 16 == 0, "bmxk_k2b_append: basis must be 16-byte aligned");
    const size_t psmem = ((size_t)32 * KF_STRIDE + (size_t)HEAD_DIM * g->rank) * sizeof(float);
    k2b_project_kernel<T><<<items * g->n_coef_heads * (g->page / 32), 8 * g->rank, psmem, s>>>(
        gg, (const T*)k_pre, ss, sh, st, basis, slots, n_pages, (__half*)coefs, vec ? 1 : 0);
    int rc = check_launch("bmxk_k2b_append(project)");
    if (rc) return rc;
  }
  BMXK_REQUIRE((uintptr_t)basis % 16 == 0, "bmxk_k2b_append: basis must be 16-byte aligned");
#define BMXK_LAUNCH_QUANT(PAGE, FUSED)                                                                                              \
  launch_quant<T, PAGE, FUSED>(gg, (const T*)k_pre, (const T*)v, ss, sh, st, basis, signs, codebook, slots, items, n_pages, \
                               (uint8_t*)pages, (__half*)coefs, vec ? 1 : 0, s)
  if (g->page == 128) return fused ? BMXK_LAUNCH_QUANT(128, true) : BMXK_LAUNCH_QUANT(128, false);
  return fused ? BMXK_LAUNCH_QUANT(64, true) : BMXK_LAUNCH_QUANT(64, false);
#undef BMXK_LAUNCH_QUANT
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

int bmxk_k2b_append_coefs(const bmxk_k2b_geom* g, const void* k_pre, const void* v, int src_dtype, int64_t stride_seq,
                          int64_t stride_head, int64_t stride_tok, const float* us_f32, const float* basis_f32, const float* signs,
                          const float* codebook, const int32_t* slots, int n_seq, int n_pages, void* pages, void* coefs,
                          void* stream) {
  int rc = check_geom(g, "bmxk_k2b_append_coefs");
  if (rc) return rc;
  BMXK_REQUIRE(g->n_coef_heads == 1, "bmxk_k2b_append_coefs: n_coef_heads=%d (given coefficients belong to one basis over all heads)",
               g->n_coef_heads);
  BMXK_REQUIRE(n_seq >= 0 && n_pages >= 0, "bmxk_k2b_append_coefs: negative counts");
  if (n_seq == 0 || n_pages == 0) return BMXK_OK;
  BMXK_REQUIRE(k_pre && v && us_f32 && basis_f32 && signs && codebook && slots && pages && coefs, "bmxk_k2b_append_coefs: null pointer");
  BMXK_REQUIRE(stride_tok >= HEAD_DIM, "bmxk_k2b_append_coefs: stride_tok=%lld < 128", (long long)stride_tok);
  BMXK_REQUIRE((int64_t)n_seq * n_pages * g->h_kv < (1LL << 31), "bmxk_k2b_append_coefs: too many pages in one call");
  cudaStream_t s = (cudaStream_t)stream;
  switch (src_dtype) {
    case BMXK_DTYPE_F16:
      return append_impl<__half>(g, k_pre, v, stride_seq, stride_head, stride_tok, basis_f32, signs, codebook, slots, n_seq, n_pages, pages,
                                 coefs, s, us_f32);
    case BMXK_DTYPE_BF16:
      return append_impl<__nv_bfloat16>(g, k_pre, v, stride_seq, stride_head, stride_tok, basis_f32, signs, codebook, slots, n_seq, n_pages,
                                        pages, coefs, s, us_f32);
    case BMXK_DTYPE_F32:
      return append_impl<float>(g, k_pre, v, stride_seq, stride_head, stride_tok, basis_f32, signs, codebook, slots, n_seq, n_pages, pages,
                                coefs, s, us_f32);
    default:
      set_error("bmxk_k2b_append_coefs: unknown src_dtype %d", src_dtype);
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

int bmxk_k2b_dequant_dense(const bmxk_k2b_geom* g, const void* pages, const void* coefs, const void* basis_f16,
                           const float* signs, const float* codebook, const int32_t* page_table, int table_stride,
                           int n_pages, int batch, const void* rope_cos, const void* rope_sin, int64_t pos_offset,
                           void* k_out, void* v_out, int64_t row_stride, int out_dtype, void* stream) {
  int rc = check_geom(g, "bmxk_k2b_dequant_dense");
  if (rc) return rc;
  BMXK_REQUIRE(n_pages >= 0 && batch >= 1 && (int64_t)n_pages * batch <= 0x7fffffff, "bmxk_k2b_dequant_dense: n_pages=%d batch=%d", n_pages, batch);
  if (n_pages == 0) return BMXK_OK;
  BMXK_REQUIRE(pages && coefs && page_table && table_stride >= n_pages, "bmxk_k2b_dequant_dense: null pointer or table_stride=%d < n_pages", table_stride);
  BMXK_REQUIRE(!k_out || basis_f16, "bmxk_k2b_dequant_dense: keys need basis_f16");
  BMXK_REQUIRE(!v_out || (signs && codebook), "bmxk_k2b_dequant_dense: values need signs and codebook");
  BMXK_REQUIRE((rope_cos == nullptr) == (rope_sin == nullptr), "bmxk_k2b_dequant_dense: one rotation table without the other");
  BMXK_REQUIRE(row_stride >= (int64_t)n_pages * g->page, "bmxk_k2b_dequant_dense: row_stride=%lld below the %d committed rows",
               (long long)row_stride, n_pages * g->page);
  BMXK_REQUIRE(out_dtype == BMXK_DTYPE_F16 || out_dtype == BMXK_DTYPE_BF16, "bmxk_k2b_dequant_dense: out_dtype=%d (fp16 or bf16)", out_dtype);
  BMXK_REQUIRE(g->h_kv <= 65535, "bmxk_k2b_dequant_dense: h_kv=%d", g->h_kv);
  BMXK_REQUIRE(((uintptr_t)pages & 15) == 0 && ((uintptr_t)basis_f16 & 15) == 0 && (!k_out || ((uintptr_t)k_out & 15) == 0) &&
                   (!v_out || ((uintptr_t)v_out & 7) == 0) && (!rope_cos || (((uintptr_t)rope_cos | (uintptr_t)rope_sin) & 3) == 0),
               "bmxk_k2b_dequant_dense: misaligned buffer");
  const size_t smem = dequant_dense_smem(g->page, g->group);
  const dim3 grid((unsigned)(n_pages * batch), (unsigned)g->h_kv);
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e1 = cudaFuncSetAttribute(k2b_dequant_dense_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    cudaError_t e2 = cudaFuncSetAttribute(k2b_dequant_dense_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    if (e1 != cudaSuccess || e2 != cudaSuccess) {
      configured.retract();
      set_error("bmxk_k2b_dequant_dense: cudaFuncSetAttribute: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
      return BMXK_ERR_CUDA;
    }
  }
  if (out_dtype == BMXK_DTYPE_F16)
    k2b_dequant_dense_kernel<__half><<<grid, DD_THREADS, smem, (cudaStream_t)stream>>>(
        to_geom(g), (const uint8_t*)pages, (const __half*)coefs, (const __half*)basis_f16, signs, codebook, page_table, table_stride, n_pages,
        (const __half*)rope_cos, (const __half*)rope_sin, pos_offset, (__half*)k_out, (__half*)v_out, row_stride);
  else
    k2b_dequant_dense_kernel<__nv_bfloat16><<<grid, DD_THREADS, smem, (cudaStream_t)stream>>>(
        to_geom(g), (const uint8_t*)pages, (const __half*)coefs, (const __half*)basis_f16, signs, codebook, page_table, table_stride, n_pages,
        (const __half*)rope_cos, (const __half*)rope_sin, pos_offset, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out, row_stride);
  return check_launch("bmxk_k2b_dequant_dense");
}

}  // extern "C"
