// Paged dequant-prefill for the k2b cache: causal attention of a block of new query positions over the committed
// pages and the fp16 window WITHOUT building dense K / V for the context.
//
// bmx's prefill dequantizes every committed page into dense tensors and calls SDPA with the model's causal mask
// (bmx: src/bmx/cache/chunked_attention.py:320-395, dispatch at :454-476): at 128k tokens that transient is the memory
// peak.  Here one CTA owns 128 / G consecutive query positions of one (sequence, KV head) -- with the G query heads
// that is 128 attention rows, sixteen per warp -- and walks the visible 128-token pages: a page block and its
// coefficient block arrive by bulk copy, are dequantized into shared memory ONCE for all 128 rows
//   K = coef x basis^T (mma.sync) + scale * residual, rotated at the token's absolute position;
//   V = the four fp16 levels of the value table, transposed (channel-major), the token norm folded into the weights
// and feed a flash-attention step (mma.sync m16n8k16, online softmax in base 2, fp32 accumulators in registers).  As in
// the decode kernels the Hadamard rotation of the value codec is linear, so it is undone once per row after the last
// page, in registers; the fp16 window then accumulates into the same rows in the unrotated space.
//
// Layout 1 pools (128-token pages) only.  Causality is by position: key t is visible to the query at position p iff
// t <= p; window slots past tail_len are masked.
#include <atomic>
#include <cstring>

#include "prefill_common.cuh"

namespace bmxk {

namespace {

constexpr int PF_THREADS = 256;
constexpr int KP = 136;  // halves per row of the dequantized K / V tiles: rows start 16 bytes apart modulo 128
constexpr int BP = 40;   // halves per basis row (rank <= 32)


__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

template <int RANK>
__global__ void __launch_bounds__(PF_THREADS, 1) k2b_prefill_kernel(const PrefillParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const K2bGeom g = p.g;
  const int G = g.n_q_groups, PP = 128 / G;  // query positions per CTA
  constexpr int COEF_BYTES = 128 * RANK * 2;
  const int PB = k2b_page_block_bytes(128, g.group);
  const int RAW = COEF_BYTES + PB;
  uint8_t* raw0 = smem;                                               // [2][RAW] coefficient block | page block
  __half* kbuf = reinterpret_cast<__half*>(raw0 + 2 * RAW);           // [128 tokens][KP] rotated keys
  __half* vbuf = kbuf + 128 * KP;                                     // [128 channels][KP] value levels (pages) or [128 tokens][KP] (window)
  __half* bsm = vbuf + 128 * KP;                                      // [128 channels][BP] basis of this head
  uint64_t* bar = reinterpret_cast<uint64_t*>(bsm + 128 * BP);        // [2] raw tile landed
  float* sg = reinterpret_cast<float*>(bar + 2);                      // [128] signs / 128
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  // the latest positions see the most pages: their blocks are scheduled first, so that the last wave is the lightest
  const int b = blockIdx.z, h = blockIdx.y, i0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * PP;
  const int H = g.h_kv * G;

  // ---- set-up: barriers, basis, signs, this warp's query fragments ----
  if (tid == 0) {
    mbar_init(&bar[0], 1), mbar_init(&bar[1], 1);
    fence_barrier_init();
  }
  for (int o = tid; o < 128 * (RANK / 8); o += PF_THREADS) {
    const int c = o / (RANK / 8), i8 = o % (RANK / 8);
    *reinterpret_cast<uint4*>(bsm + c * BP + 8 * i8) = reinterpret_cast<const uint4*>(p.basis16 + ((int64_t)h * HEAD_DIM + c) * RANK)[i8];
  }
  if (tid < 128) sg[tid] = p.signs[tid] * (1.0f / 128.0f);  // signs * fwht / sqrt(d), with the orthonormal fwht = butterflies / sqrt(d)
  // rows of this warp: m = 16 * warp + {gq, gq + 8}; m -> (query head m / PP, position i0 + m % PP)
  const int m0 = 16 * warp + gq, m1 = m0 + 8;
  const int qi0 = m0 / PP, qi1 = m1 / PP, ip0 = i0 + m0 % PP, ip1 = i0 + m1 % PP;
  const bool v0 = ip0 < p.n_q, v1 = ip1 < p.n_q;
  const __half* qr0 = p.q + (((int64_t)b * H + h * G + qi0) * p.n_q + min(ip0, p.n_q - 1)) * HEAD_DIM;
  const __half* qr1 = p.q + (((int64_t)b * H + h * G + qi1) * p.n_q + min(ip1, p.n_q - 1)) * HEAD_DIM;
  uint32_t qa[8][4];  // A fragments of Q for the eight k-steps of 16 channels
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    qa[ks][0] = *reinterpret_cast<const uint32_t*>(qr0 + 16 * ks + 2 * tq);
    qa[ks][1] = *reinterpret_cast<const uint32_t*>(qr1 + 16 * ks + 2 * tq);
    qa[ks][2] = *reinterpret_cast<const uint32_t*>(qr0 + 16 * ks + 8 + 2 * tq);
    qa[ks][3] = *reinterpret_cast<const uint32_t*>(qr1 + 16 * ks + 8 + 2 * tq);
  }
  const int64_t pq0 = p.q_pos0 + ip0, pq1 = p.q_pos0 + ip1;                       // this thread's query positions
  const int64_t pq_max = p.q_pos0 + min(i0 + PP, p.n_q) - 1;                       // last position of the CTA

  const int n_pg = p.n_pages[b];
  // pages whose first token is visible to the CTA's last position
  const int64_t vis = pq_max - p.pos_offset;
  const int n_tiles = (vis < 0) ? 0 : (int)min((int64_t)n_pg, vis / 128 + 1);
  const int tl = p.tail_len ? min(p.tail_len[b], p.tail_cap) : 0;
  const int64_t tail_pos0 = p.pos_offset + (int64_t)n_pg * 128;
  const int n_wtiles = (tl > 0 && pq_max >= tail_pos0) ? (int)((min((int64_t)tl, pq_max - tail_pos0 + 1) + 127) / 128) : 0;

  float o[16][4];  // 16 channel tiles x (row gq: 2 cols, row gq+8: 2 cols)
#pragma unroll
  for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f}, pnrow[2] = {0.f, 0.f};
  fence_proxy_async();
  __syncthreads();

  auto issue_copy = [&](int j) {  // tile j -> raw stage j & 1 (thread 0)
    const int slot = p.page_table[(int64_t)b * p.table_stride + j];
    const int chd = (g.n_coef_heads == 1) ? 0 : h;
    uint8_t* dst = raw0 + (size_t)(j & 1) * RAW;
    mbar_arrive_expect_tx(&bar[j & 1], (uint32_t)RAW);
    bulk_g2s(dst, reinterpret_cast<const uint8_t*>(p.coefs) + ((int64_t)slot * g.n_coef_heads + chd) * COEF_BYTES, COEF_BYTES, &bar[j & 1]);
    bulk_g2s(dst + COEF_BYTES, p.pages + ((int64_t)slot * g.h_kv + h) * PB, PB, &bar[j & 1]);
  };
  if (tid == 0 && n_tiles > 0) issue_copy(0);

  // One flash-attention step of this warp's 16 rows over the 128 keys in kbuf / vbuf.
  //   key_pos0: position of the tile's first key; n_valid: keys of the tile that exist; norms: fp16 per key or nullptr;
  //   v_rows: vbuf holds [token][channel] (window) instead of [channel][token] (pages)
  auto attend_tile = [&](int64_t key_pos0, int n_valid, const __half* norms, bool v_rows) {
    float s[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
      for (int n2 = 0; n2 < 8; ++n2) {
        // four 8x8 blocks: (keys 16 n2 .. +7, ch 16 ks .. +7), (same keys, ch + 8), (keys + 8, ch), (keys + 8, ch + 8)
        uint32_t b0, b1, b2, b3;
        const int key = 16 * n2 + (lane & 7) + ((lane >> 4) << 3), ch = 16 * ks + (((lane >> 3) & 1) << 3);
        ldmatrix_x4(b0, b1, b2, b3, smem_u32(kbuf + key * KP + ch));
        mma_f32acc(s[2 * n2][0], s[2 * n2][1], s[2 * n2][2], s[2 * n2][3], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
        mma_f32acc(s[2 * n2 + 1][0], s[2 * n2 + 1][1], s[2 * n2 + 1][2], s[2 * n2 + 1][3], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
      }
    }
    // scale, mask by position, row maxima
    float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = 8 * n + 2 * tq + (e & 1);
        const int64_t kpos = key_pos0 + key;
        const bool vis_ = key < n_valid && kpos <= ((e < 2) ? pq0 : pq1);
        const float v = vis_ ? s[n][e] * p.scale_log2 : -INFINITY;
        s[n][e] = v;
        tmax[e >> 1] = fmaxf(tmax[e >> 1], v);
      }
    float corr[2], mnew[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
      tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      mnew[r] = fmaxf(mrow[r], tmax[r]);
      corr[r] = (mrow[r] == -INFINITY) ? 0.f : ex2_approx(mrow[r] - mnew[r]);
      mrow[r] = mnew[r];
      lrow[r] *= corr[r], pnrow[r] *= corr[r];
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] *= corr[0], o[n][1] *= corr[0], o[n][2] *= corr[1], o[n][3] *= corr[1];
    // weights (times the key's value norm for packed pages) as A fragments of P V
    uint32_t pa[8][4];
    float lsum[2] = {0.f, 0.f}, pnsum[2] = {0.f, 0.f};
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      float pv[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) pv[e] = (mnew[e >> 1] == -INFINITY) ? 0.f : ex2_approx(s[n][e] - mnew[e >> 1]);
      lsum[0] += pv[0] + pv[1], lsum[1] += pv[2] + pv[3];
      float n0 = 1.f, n1 = 1.f;
      if (norms) {
        const float2 nn = __half22float2(*reinterpret_cast<const __half2*>(norms + 8 * n + 2 * tq));
        n0 = nn.x, n1 = nn.y;
      }
      const __half2 w0 = __floats2half2_rn(pv[0] * n0, pv[1] * n1), w1 = __floats2half2_rn(pv[2] * n0, pv[3] * n1);
      pnsum[0] += __low2float(w0) + __high2float(w0), pnsum[1] += __low2float(w1) + __high2float(w1);
      // C fragment of key tile n -> A fragment of k-step n / 2: (row gq, keys lo), (row gq+8, keys lo), (row gq, keys hi), (row gq+8, keys hi)
      pa[n >> 1][(n & 1) * 2 + 0] = h2_as_u32(w0);
      pa[n >> 1][(n & 1) * 2 + 1] = h2_as_u32(w1);
    }
    lrow[0] += lsum[0], lrow[1] += lsum[1], pnrow[0] += pnsum[0], pnrow[1] += pnsum[1];
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {      // 16 keys per step
#pragma unroll
      for (int n2 = 0; n2 < 8; ++n2) {    // 16 channels per pair of tiles
        uint32_t b0, b1, b2, b3;
        if (!v_rows) {  // vbuf[channel][token]: the "col" operand as stored
          const int ch = 16 * n2 + (lane & 7) + ((lane >> 4) << 3), key = 16 * ks + (((lane >> 3) & 1) << 3);
          ldmatrix_x4(b0, b1, b2, b3, smem_u32(vbuf + ch * KP + key));
        } else {        // vbuf[token][channel]: transposed on the way in
          const int key = 16 * ks + (lane & 7) + (((lane >> 3) & 1) << 3), ch = 16 * n2 + ((lane >> 4) << 3);
          ldmatrix_x4_trans(b0, b1, b2, b3, smem_u32(vbuf + key * KP + ch));
        }
        mma_f32acc(o[2 * n2][0], o[2 * n2][1], o[2 * n2][2], o[2 * n2][3], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], b0, b1);
        mma_f32acc(o[2 * n2 + 1][0], o[2 * n2 + 1][1], o[2 * n2 + 1][2], o[2 * n2 + 1][3], pa[ks][0], pa[ks][1], pa[ks][2], pa[ks][3], b2, b3);
      }
    }
  };

  const __half2 c1032 = __floats2half2_rn(1032.f, 1032.f), c16th = __floats2half2_rn(0.0625f, 0.0625f), cm72 = __floats2half2_rn(-72.f, -72.f);
  bool alive = true;
  for (int j = 0; j < n_tiles && alive; ++j) {
    if (tid == 0 && j + 1 < n_tiles) issue_copy(j + 1);  // its stage was released by the barrier that ended tile j-1
    if (!wait_or_flag(&bar[j & 1], (uint32_t)(j >> 1) & 1u, p.status, 20)) alive = false;
    alive = __syncthreads_and(alive ? 1 : 0) != 0;  // a wait that ran out anywhere ends the CTA as a whole
    if (!alive) break;
    const uint8_t* raw = raw0 + (size_t)(j & 1) * RAW;
    const uint8_t* blk = raw + COEF_BYTES;
    // ---- low-rank part: this warp's 16 tokens x 128 channels, K = RANK ----
    {
      float c[16][4];
#pragma unroll
      for (int n = 0; n < 16; ++n) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;
#pragma unroll
      for (int ks = 0; ks < RANK / 16; ++ks) {
        // coefficient block: 8 x 8 core matrices, (row block, k block) at ((rb * (RANK / 8) + kb) * 64 halves, rows 8 halves apart
        uint32_t a0, a1, a2, a3;
        const int rb = 2 * warp + ((lane >> 3) & 1), kb = 2 * ks + (lane >> 4);
        ldmatrix_x4(a0, a1, a2, a3, smem_u32(reinterpret_cast<const __half*>(raw) + (rb * (RANK / 8) + kb) * 64 + (lane & 7) * 8));
#pragma unroll
        for (int n2 = 0; n2 < 8; ++n2) {
          uint32_t b0, b1, b2, b3;
          const int ch = 16 * n2 + (lane & 7) + ((lane >> 4) << 3), kk = 16 * ks + (((lane >> 3) & 1) << 3);
          ldmatrix_x4(b0, b1, b2, b3, smem_u32(bsm + ch * BP + kk));
          mma_f32acc(c[2 * n2][0], c[2 * n2][1], c[2 * n2][2], c[2 * n2][3], a0, a1, a2, a3, b0, b1);
          mma_f32acc(c[2 * n2 + 1][0], c[2 * n2 + 1][1], c[2 * n2 + 1][2], c[2 * n2 + 1][3], a0, a1, a2, a3, b2, b3);
        }
      }
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        *reinterpret_cast<__half2*>(kbuf + (16 * warp + gq) * KP + 8 * n + 2 * tq) = __floats2half2_rn(c[n][0], c[n][1]);
        *reinterpret_cast<__half2*>(kbuf + (16 * warp + gq + 8) * KP + 8 * n + 2 * tq) = __floats2half2_rn(c[n][2], c[n][3]);
      }
    }
    // ---- value levels: thread = (channel, half of the tokens), transposed into vbuf[channel][token] ----
    {
      const int ch = tid & 127, cc = tid >> 7;
      const uint4 cw = reinterpret_cast<const uint4*>(blk + k2b_off_vcode(128, g.group))[cc * 128 + ch];
      const uint32_t wd[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
      for (int jw = 0; jw < 4; ++jw) {
        const uint32_t wv = wd[jw];
        const uint32_t x0 = wv & 0x33333333u, x1 = (wv >> 2) & 0x33333333u;
        uint32_t outw[8];
#pragma unroll
        for (int hs = 0; hs < 2; ++hs) {
          const uint32_t s0 = hs ? (x0 >> 16) : x0, s1 = hs ? (x1 >> 16) : x1;
          const uint32_t lo0 = prmt(p.lut_lo, 0u, s0), hi0 = prmt(p.lut_hi, 0u, s0);
          const uint32_t lo1 = prmt(p.lut_lo, 0u, s1), hi1 = prmt(p.lut_hi, 0u, s1);
          outw[2 * hs] = prmt(lo0, hi0, 0x5140u), outw[2 * hs + 1] = prmt(lo0, hi0, 0x7362u);          // tokens 4 hs .. 4 hs + 3
          outw[4 + 2 * hs] = prmt(lo1, hi1, 0x5140u), outw[4 + 2 * hs + 1] = prmt(lo1, hi1, 0x7362u);  // tokens 8 + 4 hs ..
        }
        uint4* dst = reinterpret_cast<uint4*>(vbuf + ch * KP + 64 * cc + 16 * jw);
        dst[0] = make_uint4(outw[0], outw[1], outw[2], outw[3]);
        dst[1] = make_uint4(outw[4], outw[5], outw[6], outw[7]);
      }
    }
    __syncthreads();
    // ---- keys: thread = (token, two channel chunks): + scale * residual, rotation at the absolute position ----
    {
      const int row = tid & 127, k0 = 2 * (tid >> 7);
      const int64_t pos = p.pos_offset + (int64_t)j * 128 + row;
      const int grp = row / g.group;
      const __half* ksc = reinterpret_cast<const __half*>(blk + k2b_off_kscale(128)) + grp * 128;
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int k = k0 + kk;
        const uint4 cw = reinterpret_cast<const uint4*>(blk)[k * 128 + row];
        __half* klo = kbuf + row * KP + 16 * k;       // channels 16k .. 16k+15
        __half* khi = klo + 64;                        // channels 64+16k ..
        uint4 lo4[2] = {reinterpret_cast<uint4*>(klo)[0], reinterpret_cast<uint4*>(klo)[1]};
        uint4 hi4[2] = {reinterpret_cast<uint4*>(khi)[0], reinterpret_cast<uint4*>(khi)[1]};
        const uint4 cs4[2] = {reinterpret_cast<const uint4*>(p.rope_cos + pos * HEAD_DIM + 16 * k)[0],
                              reinterpret_cast<const uint4*>(p.rope_cos + pos * HEAD_DIM + 16 * k)[1]};
        const uint4 sn4[2] = {reinterpret_cast<const uint4*>(p.rope_sin + pos * HEAD_DIM + 16 * k)[0],
                              reinterpret_cast<const uint4*>(p.rope_sin + pos * HEAD_DIM + 16 * k)[1]};
        const uint4 scl[2] = {reinterpret_cast<const uint4*>(ksc + 16 * k)[0], reinterpret_cast<const uint4*>(ksc + 16 * k)[1]};
        const uint4 sch[2] = {reinterpret_cast<const uint4*>(ksc + 64 + 16 * k)[0], reinterpret_cast<const uint4*>(ksc + 64 + 16 * k)[1]};
#pragma unroll
        for (int wd = 0; wd < 2; ++wd) {  // word wd: channels 8 wd .. 8 wd + 7 of both halves of the chunk
          const uint32_t wlo = wd ? cw.y : cw.x, whi = wd ? cw.w : cw.z;
          const uint32_t wl8 = wlo >> 8, wh8 = whi >> 8;
          __half2 rl[4], rh[4];
          rl[0] = __hsub2(u32_as_h2(lop3<0x6A>(wlo, 0x000F000Fu, 0x64086408u)), c1032);
          rl[1] = __hfma2(u32_as_h2(lop3<0x6A>(wlo, 0x00F000F0u, 0x64806480u)), c16th, cm72);
          rl[2] = __hsub2(u32_as_h2(lop3<0x6A>(wl8, 0x000F000Fu, 0x64086408u)), c1032);
          rl[3] = __hfma2(u32_as_h2(lop3<0x6A>(wl8, 0x00F000F0u, 0x64806480u)), c16th, cm72);
          rh[0] = __hsub2(u32_as_h2(lop3<0x6A>(whi, 0x000F000Fu, 0x64086408u)), c1032);
          rh[1] = __hfma2(u32_as_h2(lop3<0x6A>(whi, 0x00F000F0u, 0x64806480u)), c16th, cm72);
          rh[2] = __hsub2(u32_as_h2(lop3<0x6A>(wh8, 0x000F000Fu, 0x64086408u)), c1032);
          rh[3] = __hfma2(u32_as_h2(lop3<0x6A>(wh8, 0x00F000F0u, 0x64806480u)), c16th, cm72);
          const uint32_t dl[4] = {lo4[wd].x, lo4[wd].y, lo4[wd].z, lo4[wd].w}, dh[4] = {hi4[wd].x, hi4[wd].y, hi4[wd].z, hi4[wd].w};
          const uint32_t sl[4] = {scl[wd].x, scl[wd].y, scl[wd].z, scl[wd].w}, sh_[4] = {sch[wd].x, sch[wd].y, sch[wd].z, sch[wd].w};
          const uint32_t cc_[4] = {cs4[wd].x, cs4[wd].y, cs4[wd].z, cs4[wd].w}, ss_[4] = {sn4[wd].x, sn4[wd].y, sn4[wd].z, sn4[wd].w};
          uint32_t ol[4], oh[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const __half2 kl = __hfma2(rl[i], u32_as_h2(sl[i]), u32_as_h2(dl[i]));
            const __half2 kh = __hfma2(rh[i], u32_as_h2(sh_[i]), u32_as_h2(dh[i]));
            const __half2 c = u32_as_h2(cc_[i]), sn = u32_as_h2(ss_[i]);
            ol[i] = h2_as_u32(__hfma2(__hneg2(sn), kh, __hmul2(kl, c)));
            oh[i] = h2_as_u32(__hfma2(sn, kl, __hmul2(kh, c)));
          }
          reinterpret_cast<uint4*>(klo)[wd] = make_uint4(ol[0], ol[1], ol[2], ol[3]);
          reinterpret_cast<uint4*>(khi)[wd] = make_uint4(oh[0], oh[1], oh[2], oh[3]);
        }
      }
    }
    __syncthreads();
    attend_tile(p.pos_offset + (int64_t)j * 128, 128, reinterpret_cast<const __half*>(blk + k2b_off_vnorm(128, g.group)), false);
    __syncthreads();  // kbuf / vbuf and this raw stage are free again
  }
  if (!alive) return;

  // ---- leave the rotated space of the value codec: o <- alpha * sum(p n) + beta * o, then signs * fwht(o) / 128 per row.
  //      Column c = 8 n + 2 tq + e: bit 0 is e, bits 1..2 are tq (two shuffles), bits 3..6 are n (in registers). ----
  if (n_tiles > 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {  // the weight sums were kept per thread (its own keys): complete them over the quad
      pnrow[r] += __shfl_xor_sync(0xffffffffu, pnrow[r], 1);
      pnrow[r] += __shfl_xor_sync(0xffffffffu, pnrow[r], 2);
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      o[n][0] = p.lut_alpha * pnrow[0] + p.lut_beta * o[n][0], o[n][1] = p.lut_alpha * pnrow[0] + p.lut_beta * o[n][1];
      o[n][2] = p.lut_alpha * pnrow[1] + p.lut_beta * o[n][2], o[n][3] = p.lut_alpha * pnrow[1] + p.lut_beta * o[n][3];
    }
#pragma unroll
    for (int n = 0; n < 16; ++n) {  // bit 0
      const float a0 = o[n][0] + o[n][1], a1 = o[n][0] - o[n][1], a2 = o[n][2] + o[n][3], a3 = o[n][2] - o[n][3];
      o[n][0] = a0, o[n][1] = a1, o[n][2] = a2, o[n][3] = a3;
    }
#pragma unroll
    for (int mk = 1; mk <= 2; mk <<= 1) {  // bits 1, 2: lanes tq ^ mk
      const bool hi = (tq & mk) != 0;
#pragma unroll
      for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float other = __shfl_xor_sync(0xffffffffu, o[n][e], mk);
          o[n][e] = hi ? (other - o[n][e]) : (o[n][e] + other);
        }
    }
#pragma unroll
    for (int hb = 1; hb < 16; hb <<= 1)  // bits 3..6: tiles n ^ hb
#pragma unroll
      for (int n = 0; n < 16; ++n)
        if (!(n & hb)) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float a = o[n][e], bb = o[n | hb][e];
            o[n][e] = a + bb, o[n | hb][e] = a - bb;
          }
        }
#pragma unroll
    for (int n = 0; n < 16; ++n) {
      const float s0 = sg[8 * n + 2 * tq], s1 = sg[8 * n + 2 * tq + 1];
      o[n][0] *= s0, o[n][1] *= s1, o[n][2] *= s0, o[n][3] *= s1;
    }
  }

  // ---- the fp16 window: keys already rotated, values unrotated ----
  const __half* kt = p.k_tail + ((int64_t)b * g.h_kv + h) * p.tail_cap * HEAD_DIM;
  const __half* vt = p.v_tail + ((int64_t)b * g.h_kv + h) * p.tail_cap * HEAD_DIM;
  for (int wt = 0; wt < n_wtiles; ++wt) {
    const int t0 = wt * 128, nv = min(128, tl - t0);
    for (int oo = tid; oo < 128 * 16; oo += PF_THREADS) {
      const int r = oo >> 4, c8 = oo & 15;
      uint4 kv = make_uint4(0u, 0u, 0u, 0u), vv = make_uint4(0u, 0u, 0u, 0u);
      if (r < nv) {
        kv = reinterpret_cast<const uint4*>(kt + (int64_t)(t0 + r) * HEAD_DIM)[c8];
        vv = reinterpret_cast<const uint4*>(vt + (int64_t)(t0 + r) * HEAD_DIM)[c8];
      }
      *reinterpret_cast<uint4*>(kbuf + r * KP + 8 * c8) = kv;
      *reinterpret_cast<uint4*>(vbuf + r * KP + 8 * c8) = vv;
    }
    __syncthreads();
    attend_tile(tail_pos0 + t0, nv, nullptr, true);
    __syncthreads();
  }

  // ---- normalise and store ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 1);
    lrow[r] += __shfl_xor_sync(0xffffffffu, lrow[r], 2);
  }
  const float inv0 = 1.f / lrow[0], inv1 = 1.f / lrow[1];
  __half* or0 = p.out + (((int64_t)b * H + h * G + qi0) * p.n_q + ip0) * HEAD_DIM;
  __half* or1 = p.out + (((int64_t)b * H + h * G + qi1) * p.n_q + ip1) * HEAD_DIM;
#pragma unroll
  for (int n = 0; n < 16; ++n) {
    if (v0) *reinterpret_cast<__half2*>(or0 + 8 * n + 2 * tq) = __floats2half2_rn(o[n][0] * inv0, o[n][1] * inv0);
    if (v1) *reinterpret_cast<__half2*>(or1 + 8 * n + 2 * tq) = __floats2half2_rn(o[n][2] * inv1, o[n][3] * inv1);
  }
}

size_t prefill_smem_bytes(int rank, int group) {
  return (size_t)2 * (128 * rank * 2 + k2b_page_block_bytes(128, group)) + (size_t)2 * 128 * KP * 2 + (size_t)128 * BP * 2 + 16 + 128 * 4 + 128;
}

}  // namespace

}  // namespace bmxk

using namespace bmxk;

// 0: the tcgen05 kernel where its alignment needs are met, else the mma.sync kernel; 1: always the mma.sync kernel
static std::atomic<int> g_prefill_kernel{0};

extern "C" {

int bmxk_k2b_prefill_select(int kernel) {
  BMXK_REQUIRE(kernel == 0 || kernel == 1, "bmxk_k2b_prefill_select: kernel=%d (0: tcgen05 where it applies, 1: mma.sync)", kernel);
  g_prefill_kernel.store(kernel, std::memory_order_relaxed);
  return BMXK_OK;
}

size_t bmxk_k2b_prefill_workspace_bytes(const bmxk_k2b_geom* g, int n_q, int batch, int n_split) {
  if (!g || n_q < 1 || batch < 1 || n_split <= 1) return 0;
  return (size_t)batch * g->h_kv * g->n_q_groups * n_q * n_split * PF_PART_STRIDE * sizeof(float);
}

static int prefill_impl(const bmxk_k2b_geom* g, const void* q, int n_q, int64_t q_pos0, const void* pages, const void* coefs,
                        const void* basis_f16, const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch,
                        const void* rope_cos, const void* rope_sin, int64_t pos_offset, const void* k_tail, const void* v_tail,
                        const int32_t* tail_len, int tail_cap, const uint32_t* v_lut, const float* signs, float sm_scale,
                        int32_t* status, void* out, int n_split, void* workspace, size_t workspace_bytes, void* stream);

int bmxk_k2b_prefill(const bmxk_k2b_geom* g, const void* q, int n_q, int64_t q_pos0, const void* pages, const void* coefs,
                     const void* basis_f16, const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch,
                     const void* rope_cos, const void* rope_sin, int64_t pos_offset, const void* k_tail, const void* v_tail,
                     const int32_t* tail_len, int tail_cap, const uint32_t* v_lut, const float* signs, float sm_scale,
                     int32_t* status, void* out, void* stream) {
  return prefill_impl(g, q, n_q, q_pos0, pages, coefs, basis_f16, page_table, table_stride, n_pages, batch, rope_cos, rope_sin, pos_offset,
                      k_tail, v_tail, tail_len, tail_cap, v_lut, signs, sm_scale, status, out, 1, nullptr, 0, stream);
}

int bmxk_k2b_prefill_split(const bmxk_k2b_geom* g, const void* q, int n_q, int64_t q_pos0, const void* pages, const void* coefs,
                           const void* basis_f16, const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch,
                           const void* rope_cos, const void* rope_sin, int64_t pos_offset, const void* k_tail, const void* v_tail,
                           const int32_t* tail_len, int tail_cap, const uint32_t* v_lut, const float* signs, float sm_scale,
                           int32_t* status, void* out, int n_split, void* workspace, size_t workspace_bytes, void* stream) {
  return prefill_impl(g, q, n_q, q_pos0, pages, coefs, basis_f16, page_table, table_stride, n_pages, batch, rope_cos, rope_sin, pos_offset,
                      k_tail, v_tail, tail_len, tail_cap, v_lut, signs, sm_scale, status, out, n_split, workspace, workspace_bytes, stream);
}

}  // extern "C"

static int prefill_impl(const bmxk_k2b_geom* g, const void* q, int n_q, int64_t q_pos0, const void* pages, const void* coefs,
                        const void* basis_f16, const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch,
                        const void* rope_cos, const void* rope_sin, int64_t pos_offset, const void* k_tail, const void* v_tail,
                        const int32_t* tail_len, int tail_cap, const uint32_t* v_lut, const float* signs, float sm_scale,
                        int32_t* status, void* out, int n_split, void* workspace, size_t workspace_bytes, void* stream) {
  BMXK_REQUIRE(g != nullptr, "bmxk_k2b_prefill: null geometry");
  BMXK_REQUIRE(g->layout == 1 && g->page == 128, "bmxk_k2b_prefill: layout=%d page=%d (row-order pools of 128-token pages only)", g->layout,
               g->page);
  BMXK_REQUIRE(g->rank == 16 || g->rank == 32, "bmxk_k2b_prefill: rank=%d must be 16 or 32", g->rank);
  BMXK_REQUIRE(g->group == 32 || g->group == 64 || g->group == 128, "bmxk_k2b_prefill: group=%d must be 32, 64 or 128", g->group);
  BMXK_REQUIRE(g->n_q_groups == 1 || g->n_q_groups == 2 || g->n_q_groups == 4 || g->n_q_groups == 8,
               "bmxk_k2b_prefill: n_q_groups=%d must be 1, 2, 4 or 8", g->n_q_groups);
  BMXK_REQUIRE(g->h_kv >= 1 && (g->n_coef_heads == 1 || g->n_coef_heads == g->h_kv), "bmxk_k2b_prefill: h_kv=%d n_coef_heads=%d", g->h_kv,
               g->n_coef_heads);
  BMXK_REQUIRE(g->vbits == 2, "bmxk_k2b_prefill: vbits=%d (only 2)", g->vbits);
  BMXK_REQUIRE(batch >= 1 && batch <= 65535 && g->h_kv <= 65535 && n_q >= 1, "bmxk_k2b_prefill: batch=%d n_q=%d", batch, n_q);
  BMXK_REQUIRE(q && n_pages && v_lut && signs && status && out, "bmxk_k2b_prefill: null pointer");
  BMXK_REQUIRE(pages && coefs && basis_f16 && page_table && rope_cos && rope_sin, "bmxk_k2b_prefill: null page pool / tables");
  BMXK_REQUIRE(tail_cap == 0 || (k_tail && v_tail && tail_len), "bmxk_k2b_prefill: null window");
  BMXK_REQUIRE(((uintptr_t)pages & 15) == 0 && ((uintptr_t)coefs & 15) == 0 && ((uintptr_t)basis_f16 & 15) == 0 &&
                   ((uintptr_t)rope_cos & 15) == 0 && ((uintptr_t)rope_sin & 15) == 0 && ((uintptr_t)q & 3) == 0 && ((uintptr_t)out & 3) == 0 &&
                   (tail_cap == 0 || ((((uintptr_t)k_tail | (uintptr_t)v_tail) & 15) == 0)),
               "bmxk_k2b_prefill: misaligned buffer");
  PrefillParams prm;
  prm.g.h_kv = g->h_kv, prm.g.n_q_groups = g->n_q_groups, prm.g.page = g->page, prm.g.rank = g->rank, prm.g.group = g->group;
  prm.g.n_coef_heads = g->n_coef_heads, prm.g.kbits = g->kbits, prm.g.vbits = g->vbits, prm.g.layout = g->layout;
  prm.q = (const __half*)q, prm.n_q = n_q, prm.q_pos0 = q_pos0, prm.pages = (const uint8_t*)pages, prm.coefs = (const __half*)coefs;
  prm.basis16 = (const __half*)basis_f16, prm.page_table = page_table, prm.table_stride = table_stride, prm.n_pages = n_pages;
  prm.rope_cos = (const __half*)rope_cos, prm.rope_sin = (const __half*)rope_sin, prm.pos_offset = pos_offset;
  prm.k_tail = (const __half*)k_tail, prm.v_tail = (const __half*)v_tail, prm.tail_len = tail_cap > 0 ? tail_len : nullptr, prm.tail_cap = tail_cap;
  prm.lut_lo = v_lut[0], prm.lut_hi = v_lut[1];
  memcpy(&prm.lut_alpha, &v_lut[2], 4);
  memcpy(&prm.lut_beta, &v_lut[3], 4);
  prm.signs = signs, prm.scale_log2 = sm_scale * 1.4426950408889634f, prm.out = (__half*)out, prm.status = status;
  const size_t smem = prefill_smem_bytes(g->rank, g->group);
  const int pp = 128 / g->n_q_groups;
  const dim3 grid((unsigned)((n_q + pp - 1) / pp), (unsigned)g->h_kv, (unsigned)batch);
  cudaStream_t s = (cudaStream_t)stream;
  const bool aligned16 = ((uintptr_t)q & 15) == 0 && ((uintptr_t)out & 15) == 0;
  const bool t5 = g_prefill_kernel.load(std::memory_order_relaxed) == 0 && aligned16;
  BMXK_REQUIRE(n_split >= 1 && n_split <= 64, "bmxk_k2b_prefill_split: n_split=%d must be in 1..64", n_split);
  if (!t5) n_split = 1;  // the split is the tcgen05 kernel's; the mma.sync kernel walks every page of a block in one CTA
  prm.n_split = n_split, prm.part = (float*)workspace;
  if (n_split > 1) {
    const size_t need = bmxk_k2b_prefill_workspace_bytes(g, n_q, batch, n_split);
    BMXK_REQUIRE(workspace && workspace_bytes >= need && ((uintptr_t)workspace & 15) == 0,
                 "bmxk_k2b_prefill_split: workspace of %zu bytes needed (16-byte aligned), %zu given", need, workspace_bytes);
    BMXK_REQUIRE((int64_t)grid.x * n_split <= 0x7fffffff && (int64_t)batch * g->h_kv * g->n_q_groups * n_q <= 0x7fffffff,
                 "bmxk_k2b_prefill_split: n_q=%d batch=%d n_split=%d too large", n_q, batch, n_split);
    return launch_prefill_t5(prm, dim3(grid.x * (unsigned)n_split, grid.y, grid.z), s);
  }
  if (t5) return launch_prefill_t5(prm, grid, s);
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e1 = cudaFuncSetAttribute(k2b_prefill_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    cudaError_t e2 = cudaFuncSetAttribute(k2b_prefill_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e1 != cudaSuccess || e2 != cudaSuccess) {
      configured.retract();
      set_error("bmxk_k2b_prefill: cudaFuncSetAttribute: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
      return BMXK_ERR_CUDA;
    }
  }
  if (g->rank == 32) k2b_prefill_kernel<32><<<grid, PF_THREADS, smem, s>>>(prm);
  else k2b_prefill_kernel<16><<<grid, PF_THREADS, smem, s>>>(prm);
  return check_launch("bmxk_k2b_prefill");
}


