// Plain RTN (round-to-nearest, symmetric, groupwise) packed cache: quantize-on-append, exporter,
// page dequantizer and the split-KV decode kernel.
//   keys  : `rtn_token`  (groups of k_group channels per token)  or
//           `rtn_channel` (groups of k_group tokens per channel, bmx's KIVI-style key arm); post-RoPE
//   values: `rtn_token`  (groups of v_group channels per token)
// Codes are bmx's signed integers (bmx: src/bmx/quant/rtn.py:23-44): keys in two's-complement nibbles,
// values in two's-complement 2-bit fields (a 2-bit symmetric code only takes -1, 0, 1).
//
// Page block per (slot, head), page = 64 or 128 tokens, head dim 128:
//   [ K nibbles page*64 | K scales | V codes page*32 | V scales page*8 ]
//   K nibbles and V codes use the same lane-fragment order as the k2b page (layout.cuh);
//   K scales: rtn_channel -> (page/k_group) x 128 fp16 in k2b_kscale_idx order
//             rtn_token   -> page x 4 fp16, [row][channel group] (unused groups zero)
//   V scales: page x 4 fp16, [row][channel group]
//
// The decode kernel needs no shared-memory staging: every lane's operands are contiguous 16-byte
// pieces of the page block, so a warp's global loads are fully coalesced and land directly in the
// mma fragment registers; the next tile is prefetched into registers while the current one is used.
#include "decode_common.cuh"

namespace bmxk {

struct RtnGeom {
  int h_kv, n_q_groups, page, k_arm, k_group, v_group, kbits, vbits;
};
constexpr int RTN_TOKEN = 0, RTN_CHANNEL = 1;

BMXK_HD int rtn_kscale_bytes(const RtnGeom& g) { return g.k_arm == RTN_CHANNEL ? (g.page / g.k_group) * 256 : g.page * 8; }
BMXK_HD int rtn_off_kscale(const RtnGeom& g) { return g.page * 64; }
BMXK_HD int rtn_off_vcode(const RtnGeom& g) { return rtn_off_kscale(g) + rtn_kscale_bytes(g); }
BMXK_HD int rtn_off_vscale(const RtnGeom& g) { return rtn_off_vcode(g) + g.page * 32; }
BMXK_HD int rtn_block_bytes(const RtnGeom& g) { return rtn_off_vscale(g) + g.page * 8; }

// ---------------------------------------------------------------------------------------------
// Quantize-on-append.  One block of 128 threads per (item, head).
//   scale = max(absmax, 1e-12) / qmax ; code = clamp(rint(x / scale), -qmax-1, qmax)   (float32)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128) rtn_quant_page_kernel(RtnGeom g, const T* __restrict__ k, const T* __restrict__ v,
                                                             int64_t stride_seq, int64_t stride_head, int64_t stride_tok,
                                                             const int32_t* __restrict__ slots, int n_pages,
                                                             uint8_t* __restrict__ pages) {
  extern __shared__ __align__(16) uint8_t smem[];
  int8_t* kcode = reinterpret_cast<int8_t*>(smem);            // [page][128]
  int8_t* vcode = kcode + g.page * HEAD_DIM;                   // [page][128]
  const int item = blockIdx.x / g.h_kv, h = blockIdx.x % g.h_kv;
  const int seq = item / n_pages, pg = item % n_pages;
  const int slot = slots[item], page = g.page;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* blk = pages + ((int64_t)slot * g.h_kv + h) * rtn_block_bytes(g);
  const T* ksrc = k + seq * stride_seq + h * stride_head + (int64_t)pg * page * stride_tok;
  const T* vsrc = v + seq * stride_seq + h * stride_head + (int64_t)pg * page * stride_tok;
  __half* kscale = reinterpret_cast<__half*>(blk + rtn_off_kscale(g));
  __half* vscale = reinterpret_cast<__half*>(blk + rtn_off_vscale(g));
  const float kq = (float)((1 << (g.kbits - 1)) - 1), vq = (float)((1 << (g.vbits - 1)) - 1);

  // token-grouped arms: warp = token, lane holds 4 channels, a group of `grp` channels spans grp/4 lanes
  auto quant_token_rows = [&](const T* src, int grp, float qmax, int8_t* code, __half* scale_out) {
    for (int r = warp; r < page; r += 4) {
      float x[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) x[i] = load_as_float<T>(src + r * stride_tok + 4 * lane + i);
      float am = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
      for (int m = 1; m < grp / 4; m <<= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, m));
      const float sc = fmaxf(am, 1e-12f) / qmax;
      uint32_t packed = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float q = rintf(x[i] / sc);
        q = fminf(fmaxf(q, -qmax - 1.f), qmax);
        packed |= ((uint32_t)(int)q & 0xFFu) << (8 * i);
      }
      *reinterpret_cast<uint32_t*>(code + r * HEAD_DIM + 4 * lane) = packed;
      const int gi = (4 * lane) / grp;
      if ((4 * lane) % grp == 0) scale_out[r * 4 + gi] = __float2half_rn(sc);
      if (lane < 4 && lane >= HEAD_DIM / grp) scale_out[r * 4 + lane] = __float2half_rn(0.f);
    }
  };
  if (g.k_arm == RTN_TOKEN) {
    quant_token_rows(ksrc, g.k_group, kq, kcode, kscale);
  } else {  // thread = channel, groups of k_group tokens
    const int c = tid;
    for (int grp = 0; grp < page / g.k_group; ++grp) {
      float am = 0.f;
      for (int r = grp * g.k_group; r < (grp + 1) * g.k_group; ++r) am = fmaxf(am, fabsf(load_as_float<T>(ksrc + r * stride_tok + c)));
      const float sc = fmaxf(am, 1e-12f) / kq;
      kscale[k2b_kscale_idx(grp, c)] = __float2half_rn(sc);
      for (int r = grp * g.k_group; r < (grp + 1) * g.k_group; ++r) {
        float q = rintf(load_as_float<T>(ksrc + r * stride_tok + c) / sc);
        kcode[r * HEAD_DIM + c] = (int8_t)fminf(fmaxf(q, -kq - 1.f), kq);
      }
    }
  }
  quant_token_rows(vsrc, g.v_group, vq, vcode, vscale);
  __syncthreads();
  uint32_t* kw = reinterpret_cast<uint32_t*>(blk);
  for (int w = tid; w < page * 16; w += blockDim.x) {
    const int q = w & 3, ln = (w >> 2) & 31, th = (w >> 7) & 1, wr = w >> 8;
    const int gg = ln >> 2, t = ln & 3, r = wr * 16 + th * 8 + gg;
    uint32_t word = 0;
#pragma unroll
    for (int e = 0; e < 2; ++e)
#pragma unroll
      for (int i = 0; i < 4; ++i) word |= ((uint32_t)kcode[r * HEAD_DIM + 8 * (4 * q + i) + 2 * t + e] & 0xFu) << (16 * e + 4 * i);
    kw[w] = word;
  }
  uint32_t* vw = reinterpret_cast<uint32_t*>(blk + rtn_off_vcode(g));
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
          const int c = 16 * (2 * j + hs) + 8 * (a & 1) + gg, r = wr * 16 + 8 * (a >> 1) + 2 * t + e;
          word |= ((uint32_t)vcode[r * HEAD_DIM + c] & 3u) << (16 * hs + 4 * (2 * (a & 1) + e) + 2 * (a >> 1));
        }
    vw[w] = word;
  }
}

__device__ __forceinline__ int rtn_read_kcode(const uint32_t* kw, int r, int c) {
  int w, b;
  k2b_kres_loc(r, c, w, b);
  return (((kw[w] >> b) & 0xF) ^ 8) - 8;
}
__device__ __forceinline__ int rtn_read_vcode(const uint32_t* vw, int r, int c) {
  int w, b;
  k2b_vcode_loc(r, c, w, b);
  return (((vw[w] >> b) & 3) ^ 2) - 2;
}
__device__ __forceinline__ float rtn_kscale_at(const RtnGeom& g, const __half* ks, int r, int c) {
  return __half2float(g.k_arm == RTN_CHANNEL ? ks[k2b_kscale_idx(r / g.k_group, c)] : ks[r * 4 + c / g.k_group]);
}

// Exporter / dequantizer: one block per (page, head).  Codes go out as int8 in bmx's containers
// (bmx: src/bmx/cache/triton_dequant_attention.py:1390-1451 for token arms; the (C, page) block-dict
// layout of src/bmx/cache/codecs.py:723-725 for channel-grouped keys); dequant = code * fp16 scale.
__global__ void rtn_export_kernel(RtnGeom g, const uint8_t* __restrict__ pages, const int32_t* __restrict__ slots,
                                  int8_t* __restrict__ k_codes, __half* __restrict__ k_scales, int8_t* __restrict__ v_codes,
                                  __half* __restrict__ v_scales, float* __restrict__ k_deq, float* __restrict__ v_deq) {
  const int n = blockIdx.x / g.h_kv, h = blockIdx.x % g.h_kv, page = g.page, C = g.h_kv * HEAD_DIM;
  const uint8_t* blk = pages + ((int64_t)slots[n] * g.h_kv + h) * rtn_block_bytes(g);
  const uint32_t* kw = reinterpret_cast<const uint32_t*>(blk);
  const __half* ks = reinterpret_cast<const __half*>(blk + rtn_off_kscale(g));
  const uint32_t* vw = reinterpret_cast<const uint32_t*>(blk + rtn_off_vcode(g));
  const __half* vs = reinterpret_cast<const __half*>(blk + rtn_off_vscale(g));
  const int nkg = HEAD_DIM / g.k_group, nvg = HEAD_DIM / g.v_group, ntg = page / g.k_group;
  for (int o = threadIdx.x; o < page * HEAD_DIM; o += blockDim.x) {
    const int r = o / HEAD_DIM, c = o % HEAD_DIM;
    const int kc = rtn_read_kcode(kw, r, c), vc = rtn_read_vcode(vw, r, c);
    if (k_codes) {
      if (g.k_arm == RTN_TOKEN) k_codes[(((int64_t)n * g.h_kv + h) * page + r) * HEAD_DIM + c] = (int8_t)kc;
      else k_codes[((int64_t)n * C + h * HEAD_DIM + c) * page + r] = (int8_t)kc;
    }
    if (v_codes) v_codes[(((int64_t)n * g.h_kv + h) * page + r) * HEAD_DIM + c] = (int8_t)vc;
    if (k_deq) k_deq[((int64_t)n * page + r) * C + h * HEAD_DIM + c] = (float)kc * rtn_kscale_at(g, ks, r, c);
    if (v_deq) v_deq[((int64_t)n * page + r) * C + h * HEAD_DIM + c] = (float)vc * __half2float(vs[r * 4 + c / g.v_group]);
  }
  if (k_scales) {
    if (g.k_arm == RTN_TOKEN) {
      for (int o = threadIdx.x; o < page * nkg; o += blockDim.x)
        k_scales[(((int64_t)n * g.h_kv + h) * page + o / nkg) * nkg + o % nkg] = ks[(o / nkg) * 4 + o % nkg];
    } else {
      for (int o = threadIdx.x; o < HEAD_DIM * ntg; o += blockDim.x)
        k_scales[((int64_t)n * C + h * HEAD_DIM + o / ntg) * ntg + o % ntg] = ks[k2b_kscale_idx(o % ntg, o / ntg)];
    }
  }
  if (v_scales)
    for (int o = threadIdx.x; o < page * nvg; o += blockDim.x)
      v_scales[(((int64_t)n * g.h_kv + h) * page + o / nvg) * nvg + o % nvg] = vs[(o / nvg) * 4 + o % nvg];
}

// ---------------------------------------------------------------------------------------------
// Split-KV decode.  Persistent grid, 8 warps per CTA, warp w owns token rows 16w..16w+15 of every
// 128-token tile of its CTA's range; same flat decomposition, partial record and merge kernel as k2b.
// ---------------------------------------------------------------------------------------------
struct RtnDecodeParams {
  RtnGeom g;
  const __half* q;
  const uint8_t* pages;
  const int32_t* page_table;
  int table_stride;
  const int32_t* n_pages;
  int batch;
  float scale_log2;
  float* part;
};

struct RtnFrag {   // one warp's operands of one tile, as loaded
  uint4 k0, k1, v, ks[4];
  uint2 vs0, vs1;
  bool valid;
};

template <int PAGE>
__global__ void __launch_bounds__(256, 1) rtn_decode_kernel(const RtnDecodeParams p) {
  constexpr int PAGES_PER_TILE = TILE_TOKENS / PAGE, WR_PER_PAGE = PAGE / 16;
  extern __shared__ __align__(16) uint8_t smem[];
  float* red = reinterpret_cast<float*>(smem);       // [8 warps][8 q][128]
  float* red_m = red + 8 * 8 * HEAD_DIM;              // [8][8]
  float* red_l = red_m + 64;
  int* cum = reinterpret_cast<int*>(red_l + 64);      // [batch + 1]
  int* npg_sm = cum + p.batch + 1;
  const RtnGeom g = p.g;
  const int G = g.n_q_groups, PB = rtn_block_bytes(g);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, t4 = lane & 3;
  asm volatile("griddepcontrol.launch_dependents;");  // the merge kernel is this kernel's programmatic dependent (see launch_merge)
  if (warp == 0) fill_cum(cum, p.n_pages, p.batch, g.h_kv, PAGE, lane);
  for (int i = tid; i < p.batch; i += 256) npg_sm[i] = p.n_pages[i];
  __syncthreads();
  const int total = cum[p.batch];
  const int per_cta = (total + gridDim.x - 1) / gridDim.x;
  const int f_begin = min(total, (int)blockIdx.x * per_cta), f_end = min(total, f_begin + per_cta);
  if (f_begin >= f_end) return;
  TileCursor cur;
  cur.init(cum, npg_sm, f_begin, PAGE);
  const int sub_page = warp / WR_PER_PAGE, wr = warp % WR_PER_PAGE;
  const int kgrp = (16 * wr) / g.k_group;  // token group of this warp's rows (channel-grouped keys)

  auto load = [&](const TileCursor& c) {
    RtnFrag f;
    const int valid_pages = min(PAGES_PER_TILE, npg_sm[c.b] - c.j * PAGES_PER_TILE);
    f.valid = sub_page < valid_pages;
    if (f.valid) {
      const int slot = p.page_table[(int64_t)c.b * p.table_stride + c.j * PAGES_PER_TILE + sub_page];
      const uint8_t* blk = p.pages + ((int64_t)slot * g.h_kv + c.h) * PB;
      f.k0 = *reinterpret_cast<const uint4*>(blk + ((wr * 2 + 0) * 32 + lane) * 16);
      f.k1 = *reinterpret_cast<const uint4*>(blk + ((wr * 2 + 1) * 32 + lane) * 16);
      f.v = *reinterpret_cast<const uint4*>(blk + rtn_off_vcode(g) + (wr * 32 + lane) * 16);
      const uint8_t* ks = blk + rtn_off_kscale(g);
      if (g.k_arm == RTN_CHANNEL) {
#pragma unroll
        for (int k = 0; k < 4; ++k) f.ks[k] = *reinterpret_cast<const uint4*>(ks + (kgrp * 128 + k * 32 + t4 * 8) * 2);
      } else {  // [row][4] halfs for rows g and g+8
        const uint2 a = *reinterpret_cast<const uint2*>(ks + (16 * wr + gq) * 8);
        const uint2 b = *reinterpret_cast<const uint2*>(ks + (16 * wr + gq + 8) * 8);
        f.ks[0] = make_uint4(a.x, a.y, b.x, b.y);
      }
      const uint8_t* vs = blk + rtn_off_vscale(g);
      f.vs0 = *reinterpret_cast<const uint2*>(vs + (16 * wr + gq) * 8);
      f.vs1 = *reinterpret_cast<const uint2*>(vs + (16 * wr + gq + 8) * 8);
    }
    return f;
  };

  uint32_t qb[8][2];
  float O[8][4];
  float m0 = 0.f, m1 = 0.f, l0 = 0.f, l1 = 0.f;
  int cur_bh = -1, cur_b = 0, cur_h = 0;
  const __half2 c1032 = __floats2half2_rn(1032.f, 1032.f), c16th = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 cm72 = __floats2half2_rn(-72.f, -72.f);
  // two's-complement 2-bit value codes as fp16: 0, 1, -2, -1  (low bytes / high bytes of the four halfs)
  const uint32_t lut_lo = 0x00000000u, lut_hi = 0xBCC03C00u;

  auto flush = [&](int b_, int h_) {
#pragma unroll
    for (int m = 4; m <= 16; m <<= 1) l0 += __shfl_xor_sync(0xffffffffu, l0, m), l1 += __shfl_xor_sync(0xffffffffu, l1, m);
    if (gq == 0) {
      red_m[warp * 8 + 2 * t4] = m0, red_m[warp * 8 + 2 * t4 + 1] = m1;
      red_l[warp * 8 + 2 * t4] = l0, red_l[warp * 8 + 2 * t4 + 1] = l1;
    }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      float* o = red + (warp * 8) * HEAD_DIM;
      o[(2 * t4) * HEAD_DIM + 16 * mt + gq] = O[mt][0];
      o[(2 * t4 + 1) * HEAD_DIM + 16 * mt + gq] = O[mt][1];
      o[(2 * t4) * HEAD_DIM + 16 * mt + gq + 8] = O[mt][2];
      o[(2 * t4 + 1) * HEAD_DIM + 16 * mt + gq + 8] = O[mt][3];
    }
    __syncthreads();
    float* dst = p.part + ((int64_t)(blockIdx.x + b_ * g.h_kv + h_) * G) * PART_STRIDE;
    for (int o = tid; o < G * HEAD_DIM; o += 256) {
      const int qi = o / HEAD_DIM, ch = o % HEAD_DIM;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < 8; ++w) M = fmaxf(M, red_m[w * 8 + qi]);
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < 8; ++w) {
        const float mw = red_m[w * 8 + qi];
        const float f = (mw == -INFINITY) ? 0.f : ex2_approx(mw - M);
        acc += red[(w * 8 + qi) * HEAD_DIM + ch] * f;
        l += red_l[w * 8 + qi] * f;
      }
      dst[qi * PART_STRIDE + 2 + ch] = acc;
      if (ch == 0) dst[qi * PART_STRIDE] = M, dst[qi * PART_STRIDE + 1] = l;
    }
    __syncthreads();
  };

  RtnFrag fr = load(cur);
  for (int f = f_begin; f < f_end; ++f) {
    const int b = cur.b, h = cur.h, bh = cur.b * g.h_kv + cur.h;
    TileCursor nxt = cur;
    nxt.next(npg_sm, g.h_kv, PAGE, p.batch);
    RtnFrag fn;
    fn.valid = false;
    if (f + 1 < f_end) fn = load(nxt);  // in flight while this tile is computed
    if (bh != cur_bh) {
      if (cur_bh >= 0) flush(cur_b, cur_h);
      cur_bh = bh, cur_b = b, cur_h = h;
      m0 = (2 * t4 < G) ? -INFINITY : 0.f, m1 = (2 * t4 + 1 < G) ? -INFINITY : 0.f, l0 = l1 = 0.f;
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) O[mt][0] = O[mt][1] = O[mt][2] = O[mt][3] = 0.f;
      const __half* qp = p.q + ((int64_t)bh * G + gq) * HEAD_DIM + 2 * t4;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qb[ks][0] = (gq < G) ? *reinterpret_cast<const uint32_t*>(qp + 16 * ks) : 0u;
        qb[ks][1] = (gq < G) ? *reinterpret_cast<const uint32_t*>(qp + 16 * ks + 8) : 0u;
      }
    }
    if (fr.valid) {
      // ---- keys: nibble -> half2 (one LOP3 + one exact fix-up), times the group scale ----
      uint32_t acc[16][2];
      const uint32_t ww[2][4] = {{fr.k0.x, fr.k0.y, fr.k0.z, fr.k0.w}, {fr.k1.x, fr.k1.y, fr.k1.z, fr.k1.w}};
      const uint32_t scw[16] = {fr.ks[0].x, fr.ks[0].y, fr.ks[0].z, fr.ks[0].w, fr.ks[1].x, fr.ks[1].y, fr.ks[1].z, fr.ks[1].w,
                                fr.ks[2].x, fr.ks[2].y, fr.ks[2].z, fr.ks[2].w, fr.ks[3].x, fr.ks[3].y, fr.ks[3].z, fr.ks[3].w};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
          const uint32_t wlo = ww[c][qd], whi = ww[c][qd] >> 8;
          const __half2 k0 = __hsub2(u32_as_h2(lop3<0x6A>(wlo, 0x000F000Fu, 0x64086408u)), c1032);
          const __half2 k1 = __hfma2(u32_as_h2(lop3<0x6A>(wlo, 0x00F000F0u, 0x64806480u)), c16th, cm72);
          const __half2 k2 = __hsub2(u32_as_h2(lop3<0x6A>(whi, 0x000F000Fu, 0x64086408u)), c1032);
          const __half2 k3 = __hfma2(u32_as_h2(lop3<0x6A>(whi, 0x00F000F0u, 0x64806480u)), c16th, cm72);
          __half2 s0, s1, s2, s3;
          if (g.k_arm == RTN_CHANNEL) {
            s0 = u32_as_h2(scw[4 * qd]), s1 = u32_as_h2(scw[4 * qd + 1]), s2 = u32_as_h2(scw[4 * qd + 2]), s3 = u32_as_h2(scw[4 * qd + 3]);
          } else {  // per (row, channel group): words 0,1 hold row g's four scales, words 2,3 row g+8's
            const int gi = (32 * qd) / g.k_group;
            const uint32_t wsel = scw[2 * c + (gi >> 1)];
            const __half sc = __ushort_as_half((unsigned short)((gi & 1) ? (wsel >> 16) : (wsel & 0xFFFFu)));
            s0 = s1 = s2 = s3 = __half2half2(sc);
          }
          acc[4 * qd + 0][c] = h2_as_u32(__hmul2(k0, s0));
          acc[4 * qd + 1][c] = h2_as_u32(__hmul2(k1, s1));
          acc[4 * qd + 2][c] = h2_as_u32(__hmul2(k2, s2));
          acc[4 * qd + 3][c] = h2_as_u32(__hmul2(k3, s3));
        }
      float S[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int ks = 0; ks < 8; ++ks)
        mma_f32acc(S[0], S[1], S[2], S[3], acc[2 * ks][0], acc[2 * ks][1], acc[2 * ks + 1][0], acc[2 * ks + 1][1], qb[ks][0], qb[ks][1]);
#pragma unroll
      for (int i = 0; i < 4; ++i) S[i] *= p.scale_log2;
      // ---- online softmax (base 2, lazy rescale), this lane owns queries 2t and 2t+1 ----
      {
        __half2 tm = __floats2half2_rn(fmaxf(S[0], S[2]), fmaxf(S[1], S[3]));
        tm = __hmax2(tm, u32_as_h2(__shfl_xor_sync(0xffffffffu, h2_as_u32(tm), 4)));
        tm = __hmax2(tm, u32_as_h2(__shfl_xor_sync(0xffffffffu, h2_as_u32(tm), 8)));
        tm = __hmax2(tm, u32_as_h2(__shfl_xor_sync(0xffffffffu, h2_as_u32(tm), 16)));
        const float2 tmf = __half22float2(tm);
        const bool need0 = (2 * t4 < G) && (tmf.x > m0 + 8.f), need1 = (2 * t4 + 1 < G) && (tmf.y > m1 + 8.f);
        if (__any_sync(0xffffffffu, need0 || need1)) {
          const float n0 = need0 ? tmf.x + 0.5f : m0, n1 = need1 ? tmf.y + 0.5f : m1;
          const float f0 = (m0 == -INFINITY) ? 0.f : ex2_approx(m0 - n0), f1 = (m1 == -INFINITY) ? 0.f : ex2_approx(m1 - n1);
          l0 *= f0, l1 *= f1, m0 = n0, m1 = n1;
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) O[mt][0] *= f0, O[mt][1] *= f1, O[mt][2] *= f0, O[mt][3] *= f1;
        }
      }
      const float p0 = ex2_approx(S[0] - m0), p1 = ex2_approx(S[1] - m1), p2 = ex2_approx(S[2] - m0), p3 = ex2_approx(S[3] - m1);
      l0 += p0 + p2, l1 += p1 + p3;
      // ---- values: weights times the per-(row, channel group) scale, one B fragment per group ----
      uint32_t pb[4][2];
      const uint32_t vsw[4] = {fr.vs0.x, fr.vs0.y, fr.vs1.x, fr.vs1.y};
#pragma unroll
      for (int gi = 0; gi < 4; ++gi)
        if (gi < HEAD_DIM / g.v_group) {
          const float sa = __half2float(__ushort_as_half((unsigned short)((gi & 1) ? (vsw[gi >> 1] >> 16) : (vsw[gi >> 1] & 0xFFFFu))));
          const float sb = __half2float(__ushort_as_half((unsigned short)((gi & 1) ? (vsw[2 + (gi >> 1)] >> 16) : (vsw[2 + (gi >> 1)] & 0xFFFFu))));
          pb[gi][0] = movmatrix_trans(h2_as_u32(__floats2half2_rn(p0 * sa, p1 * sa)));
          pb[gi][1] = movmatrix_trans(h2_as_u32(__floats2half2_rn(p2 * sb, p3 * sb)));
        } else {
          pb[gi][0] = pb[gi][1] = 0u;
        }
      const uint32_t vv[4] = {fr.v.x, fr.v.y, fr.v.z, fr.v.w};
#pragma unroll
      for (int jw = 0; jw < 4; ++jw) {
        const uint32_t x0 = vv[jw] & 0x33333333u, x1 = (vv[jw] >> 2) & 0x33333333u;
#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
          const uint32_t s0 = hs ? (x0 >> 16) : x0, s1 = hs ? (x1 >> 16) : x1;
          const uint32_t lo0 = prmt(lut_lo, 0u, s0), hi0 = prmt(lut_hi, 0u, s0), lo1 = prmt(lut_lo, 0u, s1), hi1 = prmt(lut_hi, 0u, s1);
          const int mt = 2 * jw + hs, gi = (16 * mt) / g.v_group;
          mma_f32acc(O[mt][0], O[mt][1], O[mt][2], O[mt][3], prmt(lo0, hi0, 0x5140u), prmt(lo0, hi0, 0x7362u),
                     prmt(lo1, hi1, 0x5140u), prmt(lo1, hi1, 0x7362u), pb[gi][0], pb[gi][1]);
        }
      }
    }
    fr = fn;
    cur = nxt;
  }
  if (cur_bh >= 0) flush(cur_b, cur_h);
}

static int check_rtn_geom(const bmxk_rtn_geom* g, const char* who) {
  BMXK_REQUIRE(g != nullptr, "%s: null geometry", who);
  BMXK_REQUIRE(g->h_kv >= 1 && g->h_kv <= 64 && g->n_q_groups >= 1 && g->n_q_groups <= 8, "%s: h_kv=%d n_q_groups=%d", who,
               g->h_kv, g->n_q_groups);
  BMXK_REQUIRE(g->page == 64 || g->page == 128, "%s: page=%d must be 64 or 128", who, g->page);
  BMXK_REQUIRE(g->k_arm == RTN_TOKEN || g->k_arm == RTN_CHANNEL, "%s: k_arm=%d (0 = rtn_token, 1 = rtn_channel)", who, g->k_arm);
  BMXK_REQUIRE(g->k_group == 32 || g->k_group == 64 || g->k_group == 128, "%s: k_group=%d must be 32, 64 or 128", who, g->k_group);
  BMXK_REQUIRE(g->k_arm == RTN_TOKEN || g->page % g->k_group == 0, "%s: k_group=%d must divide page=%d", who, g->k_group, g->page);
  BMXK_REQUIRE(g->v_group == 32 || g->v_group == 64 || g->v_group == 128, "%s: v_group=%d must be 32, 64 or 128", who, g->v_group);
  BMXK_REQUIRE(g->kbits >= 2 && g->kbits <= 4, "%s: kbits=%d must be in 2..4 (nibble container)", who, g->kbits);
  BMXK_REQUIRE(g->vbits == 2, "%s: vbits=%d (only 2-bit value codes have a kernel)", who, g->vbits);
  return BMXK_OK;
}
static RtnGeom to_rtn(const bmxk_rtn_geom* g) {
  RtnGeom o;
  o.h_kv = g->h_kv, o.n_q_groups = g->n_q_groups, o.page = g->page, o.k_arm = g->k_arm, o.k_group = g->k_group;
  o.v_group = g->v_group, o.kbits = g->kbits, o.vbits = g->vbits;
  return o;
}

}  // namespace bmxk

using namespace bmxk;

extern "C" {

size_t bmxk_rtn_page_block_bytes(const bmxk_rtn_geom* g) { return g ? (size_t)rtn_block_bytes(to_rtn(g)) : 0; }

size_t bmxk_rtn_decode_workspace_bytes(const bmxk_rtn_geom* g, int batch, int max_pages) {
  if (!g || batch <= 0) return 0;
  (void)max_pages;
  return 256 + ((size_t)num_sms() + (size_t)batch * g->h_kv) * g->n_q_groups * PART_STRIDE * sizeof(float);
}

int bmxk_rtn_append(const bmxk_rtn_geom* g, const void* k, const void* v, int src_dtype, int64_t stride_seq,
                    int64_t stride_head, int64_t stride_tok, const int32_t* slots, int n_seq, int n_pages, void* pages,
                    void* stream) {
  int rc = check_rtn_geom(g, "bmxk_rtn_append");
  if (rc) return rc;
  BMXK_REQUIRE(n_seq >= 0 && n_pages >= 0, "bmxk_rtn_append: negative counts");
  if (n_seq == 0 || n_pages == 0) return BMXK_OK;
  BMXK_REQUIRE(k && v && slots && pages, "bmxk_rtn_append: null pointer");
  BMXK_REQUIRE(stride_tok >= HEAD_DIM, "bmxk_rtn_append: stride_tok=%lld < 128", (long long)stride_tok);
  const RtnGeom gg = to_rtn(g);
  const int blocks = n_seq * n_pages * g->h_kv;
  const size_t smem = 2 * (size_t)g->page * HEAD_DIM;
  cudaStream_t s = (cudaStream_t)stream;
  switch (src_dtype) {
    case BMXK_DTYPE_F16:
      rtn_quant_page_kernel<__half><<<blocks, 128, smem, s>>>(gg, (const __half*)k, (const __half*)v, stride_seq, stride_head,
                                                               stride_tok, slots, n_pages, (uint8_t*)pages);
      break;
    case BMXK_DTYPE_BF16:
      rtn_quant_page_kernel<__nv_bfloat16><<<blocks, 128, smem, s>>>(gg, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
                                                                      stride_seq, stride_head, stride_tok, slots, n_pages,
                                                                      (uint8_t*)pages);
      break;
    case BMXK_DTYPE_F32:
      rtn_quant_page_kernel<float><<<blocks, 128, smem, s>>>(gg, (const float*)k, (const float*)v, stride_seq, stride_head,
                                                              stride_tok, slots, n_pages, (uint8_t*)pages);
      break;
    default:
      set_error("bmxk_rtn_append: unknown src_dtype %d", src_dtype);
      return BMXK_ERR_INVALID;
  }
  return check_launch("bmxk_rtn_append");
}

int bmxk_rtn_export(const bmxk_rtn_geom* g, const void* pages, const int32_t* slots, int n, int8_t* k_codes, void* k_scales,
                    int8_t* v_codes, void* v_scales, float* k_deq, float* v_deq, void* stream) {
  int rc = check_rtn_geom(g, "bmxk_rtn_export");
  if (rc) return rc;
  BMXK_REQUIRE(n >= 0, "bmxk_rtn_export: n < 0");
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(pages && slots, "bmxk_rtn_export: null pointer");
  rtn_export_kernel<<<n * g->h_kv, 256, 0, (cudaStream_t)stream>>>(to_rtn(g), (const uint8_t*)pages, slots, k_codes,
                                                                  (__half*)k_scales, v_codes, (__half*)v_scales, k_deq, v_deq);
  return check_launch("bmxk_rtn_export");
}

int bmxk_rtn_decode(const bmxk_rtn_geom* g, const void* q, const void* pages, const int32_t* page_table, int table_stride,
                    const int32_t* n_pages, int batch, int max_pages, const void* k_tail, const void* v_tail,
                    const int32_t* tail_len, int tail_cap, float sm_scale, void* workspace, size_t workspace_bytes, void* out,
                    int out_dtype, float* partial_out, void* stream) {
  int rc = check_rtn_geom(g, "bmxk_rtn_decode");
  if (rc) return rc;
  BMXK_REQUIRE(batch >= 1 && (int64_t)batch * g->h_kv <= MAX_BH, "bmxk_rtn_decode: batch*h_kv out of range");
  BMXK_REQUIRE(max_pages >= 0 && tail_cap >= 0, "bmxk_rtn_decode: negative sizes");
  BMXK_REQUIRE(q && n_pages && workspace, "bmxk_rtn_decode: null pointer");
  BMXK_REQUIRE(max_pages == 0 || (pages && page_table), "bmxk_rtn_decode: null page pool / table");
  BMXK_REQUIRE(tail_cap == 0 || (k_tail && v_tail && tail_len), "bmxk_rtn_decode: null tail");
  BMXK_REQUIRE(out || partial_out, "bmxk_rtn_decode: no output");
  BMXK_REQUIRE(out_dtype == BMXK_DTYPE_F16 || out_dtype == BMXK_DTYPE_F32, "bmxk_rtn_decode: out_dtype=%d", out_dtype);
  BMXK_REQUIRE(workspace_bytes >= bmxk_rtn_decode_workspace_bytes(g, batch, max_pages), "bmxk_rtn_decode: workspace too small");
  BMXK_REQUIRE(((uintptr_t)pages & 15) == 0, "bmxk_rtn_decode: the page pool must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256);
  const int64_t max_tiles = (int64_t)batch * g->h_kv * (((int64_t)max_pages * g->page + TILE_TOKENS - 1) / TILE_TOKENS);
  const int grid = (int)(max_tiles < num_sms() ? (max_tiles < 1 ? 1 : max_tiles) : num_sms());
  const float scale_log2 = sm_scale * 1.4426950408889634f;
  if (max_pages > 0) {
    RtnDecodeParams prm;
    prm.g = to_rtn(g), prm.q = (const __half*)q, prm.pages = (const uint8_t*)pages, prm.page_table = page_table;
    prm.table_stride = table_stride, prm.n_pages = n_pages, prm.batch = batch, prm.scale_log2 = scale_log2, prm.part = part;
    const size_t smem = (size_t)(8 * 8 * HEAD_DIM + 128) * 4 + (size_t)(2 * batch + 1) * 4 + 16;
    static PerDeviceOnce configured;
    if (configured.first()) {
      cudaFuncSetAttribute(rtn_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
      cudaFuncSetAttribute(rtn_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
    }
    BMXK_REQUIRE(smem <= 96 * 1024, "bmxk_rtn_decode: batch too large");
    if (g->page == 128) rtn_decode_kernel<128><<<grid, 256, smem, s>>>(prm);
    else rtn_decode_kernel<64><<<grid, 256, smem, s>>>(prm);
    rc = check_launch("bmxk_rtn_decode");
    if (rc) return rc;
  }
  K2bMergeParams mp;
  mp.g.h_kv = g->h_kv, mp.g.n_q_groups = g->n_q_groups, mp.g.page = g->page, mp.g.rank = 0, mp.g.group = g->k_group;
  mp.g.n_coef_heads = 0, mp.g.kbits = g->kbits, mp.g.vbits = g->vbits, mp.g.layout = 0;
  mp.n_sub = 1;
  mp.q = (const __half*)q, mp.n_pages = n_pages, mp.batch = batch, mp.main_grid = grid, mp.part = part;
  mp.k_tail = (const __half*)k_tail, mp.v_tail = (const __half*)v_tail, mp.tail_len = tail_cap > 0 ? tail_len : nullptr;
  mp.tail_cap = tail_cap, mp.signs = nullptr, mp.scale_log2 = scale_log2, mp.out = out, mp.out_dtype = out_dtype;
  mp.partial_out = partial_out;
  return launch_merge(mp, s, max_pages > 0);
}

}  // extern "C"
