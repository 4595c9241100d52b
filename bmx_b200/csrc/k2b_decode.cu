// k2b split-KV decode for sm_100a: a persistent, warp-specialised kernel that streams packed pages
// HBM -> shared memory with 1-D bulk async copies (one copy-issuing warp, an mbarrier ring) and has
// eight consumer warps dequantize in registers and feed mma.sync, plus the small kernel that merges
// the per-CTA partial states, attends over the fp16 recent window and undoes the value rotation.
//
// Work unit: a "tile" of 128 consecutive tokens of one (sequence, KV head).  All tiles of all
// (sequence, head) pairs form one flat list that is cut into equal contiguous ranges, one per CTA
// (grid = number of SMs), so every SM streams the same number of bytes whatever the batch and the
// context lengths are.  A CTA emits one partial (max, sum, accumulator) per (sequence, head) range
// it touches; the merge kernel combines them.
//
// Consumer warp w owns token rows 16w..16w+15 of every tile.  Per tile it
//   1. loads its low-rank coefficients as mma A fragments (ldmatrix) and computes
//        K_pre = coef x basis^T + residual      (mma m16n8k16, fp16 accumulate; the residual,
//        nibble -> half2 by one LOP3 + one exact fix-up, times its fp16 scale, is the C operand)
//   2. rotates K_pre by the token's offset INSIDE the tile (cos/sin of those 2 offsets live in
//        registers for the whole kernel); the tile's base rotation is applied to q instead,
//        once per tile, by the producer warp:  q . R(t0+o) k  =  (R(-t0) q) . (R(o) k)
//   3. scores S = K x q_rot^T (mma, fp32 accumulate) -- the K accumulators are, in register order,
//        the A operand, so nothing moves;  online softmax in base 2 with a lazy rescale; the
//        weights are transposed into the B operand of step 4 with movmatrix
//   4. values: 2-bit codes -> fp16 codebook levels with byte-permute lookups, straight into A
//        fragments; O^T += V^T x (p * norm) (mma).  The 128-point Hadamard and the signs are
//        applied once per (head, query) in the merge kernel, since they are linear in V.
#include <cmath>
#include <cstring>
#include <mutex>

#include "decode_common.cuh"

namespace bmxk {

constexpr int DEC_CONSUMER_WARPS = 8;
constexpr int DEC_THREADS = (DEC_CONSUMER_WARPS + 4) * 32;  // + one producer warpgroup (one warp of it works)
template <int RANK, int PAGE>
__global__ void __launch_bounds__(DEC_THREADS, 1) k2b_decode_kernel(const K2bDecodeParams p) {
  constexpr int KS = RANK / 16;               // k-steps of the low-rank contraction
  constexpr int PAGES_PER_TILE = TILE_TOKENS / PAGE;
  constexpr int WR_PER_PAGE = PAGE / 16;
  constexpr int COEF_TILE_BYTES = TILE_TOKENS * RANK * 2;
  constexpr int COEF_PAGE_BYTES = PAGE * RANK * 2;
  constexpr int QROT_BYTES = 8 * 4 * 8 * 8;   // [query row 0..7][t][k-step][2 regs] uint32

  extern __shared__ __align__(128) uint8_t smem[];
  const K2bGeom g = p.g;
  const int G = g.n_q_groups;
  const int PB = k2b_page_block_bytes(PAGE, g.group);
  const int STAGE_BYTES = COEF_TILE_BYTES + PAGES_PER_TILE * PB + QROT_BYTES;
  const int n_stages = p.n_stages;

  uint8_t* stage0 = smem;
  float* red = reinterpret_cast<float*>(smem + (size_t)n_stages * STAGE_BYTES);  // [8 warps][8 q][128] + m/l/pn
  float* red_m = red + DEC_CONSUMER_WARPS * 8 * HEAD_DIM;                         // [8][8]
  float* red_l = red_m + 64;
  float* red_pn = red_l + 64;
  float* q_sm = red_pn + 64;                                                      // [8][128] producer's copy of q
  uint64_t* full = reinterpret_cast<uint64_t*>(q_sm + 8 * HEAD_DIM);
  uint64_t* empty = full + 16;
  int* cum = reinterpret_cast<int*>(empty + 16);                                  // [batch + 1]
  int* npg_sm = cum + p.batch + 1;                                                // [batch] page counts

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int gq = lane >> 2, t4 = lane & 3;

  asm volatile("griddepcontrol.launch_dependents;");  // the merge kernel is this kernel's programmatic dependent (see launch_merge)
  if (warp == 0) fill_cum(cum, p.n_pages, p.batch, g.h_kv, PAGE, lane);
  for (int i = tid; i < p.batch; i += DEC_THREADS) npg_sm[i] = p.n_pages[i];
  // query rows beyond the group size stay zero in every stage (their scores are never read)
  for (int st_ = 0; st_ < n_stages; ++st_) {
    uint32_t* qr0 = reinterpret_cast<uint32_t*>(stage0 + (size_t)st_ * STAGE_BYTES + COEF_TILE_BYTES + PAGES_PER_TILE * PB);
    for (int i = tid; i < QROT_BYTES / 4; i += DEC_THREADS) qr0[i] = 0u;
  }
  if (tid == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(&full[s], 2);  // the copy warp (with the byte count) and the query-rotation warp
      mbar_init(&empty[s], DEC_CONSUMER_WARPS);
    }
    fence_barrier_init();
  }
  __syncthreads();

  const int total = cum[p.batch];
  const int per_cta = (total + gridDim.x - 1) / gridDim.x;
  const int f_begin = min(total, (int)blockIdx.x * per_cta);
  const int f_end = min(total, f_begin + per_cta);
  if (f_begin >= f_end) return;

  TileCursor cur;
  cur.init(cum, npg_sm, f_begin, PAGE);

  if (warp >= DEC_CONSUMER_WARPS) {
    // ===================== producer warpgroup =====================
    // Hands most of its registers to the consumers.  Its first warp only issues the bulk copies of each
    // tile; the other three take the tiles in turn and prepare the tile's rotated queries.  Two arrivals
    // complete a stage: the copy warp's (with the byte count) and the rotating warp's.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    int s = 0;
    uint32_t ph = 1;  // parity to wait for on empty[s]: a fresh barrier passes parity 1
    if (warp == DEC_CONSUMER_WARPS) {
      for (int f = f_begin; f < f_end; ++f, cur.next(npg_sm, g.h_kv, PAGE, p.batch)) {
        if (!wait_or_flag(&empty[s], ph, p.status, 1)) return;
        if (lane == 0) {
          const int b = cur.b, h = cur.h, j = cur.j;
          uint8_t* st = stage0 + (size_t)s * STAGE_BYTES;
          const int pg0 = j * PAGES_PER_TILE;
          const int npg = min(PAGES_PER_TILE, npg_sm[b] - pg0);
          const int chd = (g.n_coef_heads == 1) ? 0 : h;
          mbar_arrive_expect_tx(&full[s], (uint32_t)(npg * (COEF_PAGE_BYTES + PB)));
          for (int k = 0; k < npg; ++k) {
            const int slot = p.page_table[(int64_t)b * p.table_stride + pg0 + k];
            bulk_g2s(st + k * COEF_PAGE_BYTES,
                     reinterpret_cast<const uint8_t*>(p.coefs) + ((int64_t)slot * g.n_coef_heads + chd) * COEF_PAGE_BYTES,
                     COEF_PAGE_BYTES, &full[s]);
            bulk_g2s(st + COEF_TILE_BYTES + k * PB, p.pages + ((int64_t)slot * g.h_kv + h) * PB, PB, &full[s]);
          }
        }
        if (++s == n_stages) s = 0, ph ^= 1;
      }
      return;
    }
    // ---- query rotation warps: warp r of 3 takes tiles r, r+3, ... of the CTA's range ----
    const int rw = warp - DEC_CONSUMER_WARPS - 1;
    int it = 0;
    for (int f = f_begin; f < f_end; ++f, ++it, cur.next(npg_sm, g.h_kv, PAGE, p.batch)) {
      if (it % 3 == rw) {
        const int b = cur.b, h = cur.h, j = cur.j;
        // everything this tile needs from global memory is requested before the stage is waited for
        const int64_t t0 = p.pos_offset + (int64_t)j * TILE_TOKENS;
        const __half* qsrc = p.q + ((int64_t)b * g.h_kv + h) * G * HEAD_DIM;
        float cs[2], sn[2], x1[2][8], x2[2][8];
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int c = lane + 32 * jj;  // rotary pair (c, c + 64)
          cs[jj] = __half2float(p.rope_cos[t0 * HEAD_DIM + c]);
          sn[jj] = __half2float(p.rope_sin[t0 * HEAD_DIM + c]);
#pragma unroll
          for (int qi = 0; qi < 8; ++qi) {
            x1[jj][qi] = (qi < G) ? __half2float(qsrc[qi * HEAD_DIM + c]) : 0.f;
            x2[jj][qi] = (qi < G) ? __half2float(qsrc[qi * HEAD_DIM + c + 64]) : 0.f;
          }
        }
        if (!wait_or_flag(&empty[s], ph, p.status, 3)) return;
        __half* qr = reinterpret_cast<__half*>(stage0 + (size_t)s * STAGE_BYTES + COEF_TILE_BYTES + PAGES_PER_TILE * PB);
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          const int c = lane + 32 * jj;
          // channel ch -> k-step ch/16, register (ch%16)/8, t = (ch%8)/2, e = ch%2
          const int ks1 = c >> 4, r1 = (c >> 3) & 1, tt = (c & 7) >> 1, e = c & 1, ks2 = ks1 + 4;
#pragma unroll
          for (int qi = 0; qi < 8; ++qi)
            if (qi < G) {
              const float a = x1[jj][qi] * p.scale_log2, bb = x2[jj][qi] * p.scale_log2;
              const float y1 = a * cs[jj] + bb * sn[jj], y2 = bb * cs[jj] - a * sn[jj];
              // B fragment of k-step ks: word ((ks/2)*32 + 4*qi + tt)*4 + (ks%2)*2 + r1
              qr[((((ks1 >> 1) * 32 + qi * 4 + tt) * 4 + (ks1 & 1) * 2 + r1) * 2) + e] = __float2half_rn(y1);
              qr[((((ks2 >> 1) * 32 + qi * 4 + tt) * 4 + (ks2 & 1) * 2 + r1) * 2) + e] = __float2half_rn(y2);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&full[s]);
      }
      if (++s == n_stages) s = 0, ph ^= 1;
    }
    return;
  }

  // ===================== consumer warps =====================
  asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
  // loop-invariant rotation of the two token rows this lane owns (offsets inside the tile)
  uint32_t cosr[2][8], sinr[2][8], nsinr[2][8];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int dlt = 16 * warp + 8 * c + gq;
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      cosr[c][n] = *reinterpret_cast<const uint32_t*>(p.rope_cos + (int64_t)dlt * HEAD_DIM + 8 * n + 2 * t4);
      sinr[c][n] = *reinterpret_cast<const uint32_t*>(p.rope_sin + (int64_t)dlt * HEAD_DIM + 8 * n + 2 * t4);
      nsinr[c][n] = sinr[c][n] ^ 0x80008000u;
    }
  }
  uint32_t Bb[16][KS][2];
  float O[8][4];
  // this lane owns queries 2t and 2t+1; columns beyond the group size keep a finite maximum so that
  // their (unused) values stay finite
  float m0 = (2 * t4 < G) ? -INFINITY : 0.f, m1 = (2 * t4 + 1 < G) ? -INFINITY : 0.f;
  float l0 = 0.f, l1 = 0.f, pn0 = 0.f, pn1 = 0.f;
  int cur_bh = -1, cur_b = 0, cur_h = 0;
  const int sub_page = warp / WR_PER_PAGE, wr = warp % WR_PER_PAGE;
  const int grp = (16 * wr) / g.group;
  const __half2 c1032 = __floats2half2_rn(1032.f, 1032.f);
  const __half2 c16th = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 cm72 = __floats2half2_rn(-72.f, -72.f);

  auto flush = [&](int b_, int h_) {
    // sums over this warp's tokens (the 8 lanes that share t), then over the 8 warps through shared memory
#pragma unroll
    for (int m = 4; m <= 16; m <<= 1) {
      l0 += __shfl_xor_sync(0xffffffffu, l0, m), l1 += __shfl_xor_sync(0xffffffffu, l1, m);
      pn0 += __shfl_xor_sync(0xffffffffu, pn0, m), pn1 += __shfl_xor_sync(0xffffffffu, pn1, m);
    }
    if (gq == 0) {
      red_m[warp * 8 + 2 * t4] = m0, red_m[warp * 8 + 2 * t4 + 1] = m1;
      red_l[warp * 8 + 2 * t4] = l0, red_l[warp * 8 + 2 * t4 + 1] = l1;
      red_pn[warp * 8 + 2 * t4] = pn0, red_pn[warp * 8 + 2 * t4 + 1] = pn1;
    }
#pragma unroll
    for (int mt = 0; mt < 8; ++mt) {
      float* o = red + (warp * 8) * HEAD_DIM;
      o[(2 * t4) * HEAD_DIM + 16 * mt + gq] = O[mt][0];
      o[(2 * t4 + 1) * HEAD_DIM + 16 * mt + gq] = O[mt][1];
      o[(2 * t4) * HEAD_DIM + 16 * mt + gq + 8] = O[mt][2];
      o[(2 * t4 + 1) * HEAD_DIM + 16 * mt + gq + 8] = O[mt][3];
    }
    asm volatile("bar.sync 1, %0;" ::"n"(DEC_CONSUMER_WARPS * 32));
    float* dst = p.part + ((int64_t)(blockIdx.x + b_ * g.h_kv + h_) * G) * PART_STRIDE;
    for (int o = tid; o < G * HEAD_DIM; o += DEC_CONSUMER_WARPS * 32) {
      const int qi = o / HEAD_DIM, ch = o % HEAD_DIM;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < DEC_CONSUMER_WARPS; ++w) M = fmaxf(M, red_m[w * 8 + qi]);
      float acc = 0.f, l = 0.f, pn = 0.f;
#pragma unroll
      for (int w = 0; w < DEC_CONSUMER_WARPS; ++w) {
        const float mw = red_m[w * 8 + qi];
        const float f = (mw == -INFINITY) ? 0.f : ex2_approx(mw - M);
        acc += red[(w * 8 + qi) * HEAD_DIM + ch] * f;
        l += red_l[w * 8 + qi] * f;
        pn += red_pn[w * 8 + qi] * f;
      }
      dst[qi * PART_STRIDE + 2 + ch] = p.lut_alpha * pn + p.lut_beta * acc;
      if (ch == 0) {
        dst[qi * PART_STRIDE + 0] = M;
        dst[qi * PART_STRIDE + 1] = l;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(DEC_CONSUMER_WARPS * 32));
  };

  int s = 0;
  uint32_t ph = 0;
  bool dead = false;
  for (int f = f_begin; f < f_end; ++f, cur.next(npg_sm, g.h_kv, PAGE, p.batch)) {
    const int b = cur.b, h = cur.h, j = cur.j;
    const int bh = b * g.h_kv + h;
    if (bh != cur_bh) {
      if (cur_bh >= 0) flush(cur_b, cur_h);
      cur_bh = bh, cur_b = b, cur_h = h;
      m0 = (2 * t4 < G) ? -INFINITY : 0.f, m1 = (2 * t4 + 1 < G) ? -INFINITY : 0.f;
      l0 = l1 = pn0 = pn1 = 0.f;
#pragma unroll
      for (int mt = 0; mt < 8; ++mt) O[mt][0] = O[mt][1] = O[mt][2] = O[mt][3] = 0.f;
#pragma unroll
      for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const __half* bp = p.basis16 + ((int64_t)h * HEAD_DIM + 8 * n + gq) * RANK + 16 * ks + 2 * t4;
          Bb[n][ks][0] = *reinterpret_cast<const uint32_t*>(bp);
          Bb[n][ks][1] = *reinterpret_cast<const uint32_t*>(bp + 8);
        }
    }
    // After a wait has given up this warp stops computing but keeps walking the loop, so that it still
    // meets the other consumer warps at every named barrier.
    if (!dead && !wait_or_flag(&full[s], ph, p.status, 2)) dead = true;
    const int valid_pages = (PAGES_PER_TILE == 1) ? 1 : min(PAGES_PER_TILE, npg_sm[b] - j * PAGES_PER_TILE);
    if (!dead && sub_page < valid_pages) {
      const uint8_t* st = stage0 + (size_t)s * STAGE_BYTES;
      const uint8_t* blk = st + COEF_TILE_BYTES + sub_page * PB;
      // ---- values: 2-bit codes -> fp16 levels, directly as the A fragments of O^T += V^T P.  The two warps that
      //      share a scheduler do this ALU-bound step at opposite ends of the key work (FMA and tensor bound),
      //      so that the pipes overlap ----
      uint32_t VA[8][4];
      auto unpack_v = [&]() {
        const uint4 vw = *reinterpret_cast<const uint4*>(blk + k2b_off_vcode(PAGE, g.group) + (wr * 32 + lane) * 16);
        const uint32_t vv[4] = {vw.x, vw.y, vw.z, vw.w};
#pragma unroll
        for (int jw = 0; jw < 4; ++jw) {
          const uint32_t x0 = vv[jw] & 0x33333333u, x1 = (vv[jw] >> 2) & 0x33333333u;
#pragma unroll
          for (int hs = 0; hs < 2; ++hs) {
            const uint32_t s0 = hs ? (x0 >> 16) : x0, s1 = hs ? (x1 >> 16) : x1;
            const uint32_t lo0 = prmt(p.lut_lo, 0u, s0), hi0 = prmt(p.lut_hi, 0u, s0);
            const uint32_t lo1 = prmt(p.lut_lo, 0u, s1), hi1 = prmt(p.lut_hi, 0u, s1);
            const int mt = 2 * jw + hs;
            VA[mt][0] = prmt(lo0, hi0, 0x5140u), VA[mt][1] = prmt(lo0, hi0, 0x7362u);
            VA[mt][2] = prmt(lo1, hi1, 0x5140u), VA[mt][3] = prmt(lo1, hi1, 0x7362u);
          }
        }
      };
      const bool v_first = (warp >> 2) & 1;
      if (v_first) unpack_v();
      // ---- low-rank coefficients as A fragments ----
      uint32_t A[KS][4];
      {
        const int mi = lane >> 3, rin = lane & 7;
        const int R = 16 * warp + (mi & 1) * 8 + rin;
        const int sw = (RANK == 32) ? ((R >> 1) & 3) : ((R >> 2) & 1);
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
          const int chunk = ks * 2 + (mi >> 1);
          ldmatrix_x4(A[ks][0], A[ks][1], A[ks][2], A[ks][3], smem_u32(st + (R * RANK + ((chunk ^ sw) << 3)) * 2));
        }
      }
      // ---- residual -> C operand ----
      uint32_t acc[16][2];
      {
        const uint4 w0 = *reinterpret_cast<const uint4*>(blk + ((wr * 2 + 0) * 32 + lane) * 16);
        const uint4 w1 = *reinterpret_cast<const uint4*>(blk + ((wr * 2 + 1) * 32 + lane) * 16);
        const uint4* scp = reinterpret_cast<const uint4*>(blk + k2b_off_kscale(PAGE) + (grp * 128 + t4 * 8) * 2);
        uint32_t sc[16];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint4 v = scp[4 * k];
          sc[4 * k] = v.x, sc[4 * k + 1] = v.y, sc[4 * k + 2] = v.z, sc[4 * k + 3] = v.w;
        }
        const uint32_t ww[2][4] = {{w0.x, w0.y, w0.z, w0.w}, {w1.x, w1.y, w1.z, w1.w}};
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int qd = 0; qd < 4; ++qd) {
            const uint32_t wlo = ww[c][qd], whi = ww[c][qd] >> 8;
            // (w & mask) ^ magic : nibble^8 under a 1024 (or 1024 + 16 x) exponent
            const __half2 h0 = u32_as_h2(lop3<0x6A>(wlo, 0x000F000Fu, 0x64086408u));
            const __half2 h1 = u32_as_h2(lop3<0x6A>(wlo, 0x00F000F0u, 0x64806480u));
            const __half2 h2 = u32_as_h2(lop3<0x6A>(whi, 0x000F000Fu, 0x64086408u));
            const __half2 h3 = u32_as_h2(lop3<0x6A>(whi, 0x00F000F0u, 0x64806480u));
            const __half2 k0 = __hsub2(h0, c1032), k1 = __hfma2(h1, c16th, cm72);
            const __half2 k2 = __hsub2(h2, c1032), k3 = __hfma2(h3, c16th, cm72);
            acc[4 * qd + 0][c] = h2_as_u32(__hmul2(k0, u32_as_h2(sc[4 * qd + 0])));
            acc[4 * qd + 1][c] = h2_as_u32(__hmul2(k1, u32_as_h2(sc[4 * qd + 1])));
            acc[4 * qd + 2][c] = h2_as_u32(__hmul2(k2, u32_as_h2(sc[4 * qd + 2])));
            acc[4 * qd + 3][c] = h2_as_u32(__hmul2(k3, u32_as_h2(sc[4 * qd + 3])));
          }
      }
      // ---- K_pre = coef x basis^T + residual ----
#pragma unroll
      for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int ks = 0; ks < KS; ++ks)
          mma_f16acc(acc[n][0], acc[n][1], A[ks][0], A[ks][1], A[ks][2], A[ks][3], Bb[n][ks][0], Bb[n][ks][1]);
      // ---- rotate by the offset inside the tile ----
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int n = 0; n < 8; ++n) {
          const __half2 lo = u32_as_h2(acc[n][c]), hi = u32_as_h2(acc[n + 8][c]);
          const __half2 cs = u32_as_h2(cosr[c][n]), sn = u32_as_h2(sinr[c][n]), nsn = u32_as_h2(nsinr[c][n]);
          const __half2 lo2 = __hfma2(lo, cs, __hmul2(hi, nsn));
          const __half2 hi2 = __hfma2(hi, cs, __hmul2(lo, sn));
          acc[n][c] = h2_as_u32(lo2);
          acc[n + 8][c] = h2_as_u32(hi2);
        }
      // ---- scores: rows = this warp's 16 tokens, columns = queries.  The K accumulators of n-tiles
      //      2ks, 2ks+1 are, in register order, exactly the A fragment of k-step ks ----
      float S[4] = {0.f, 0.f, 0.f, 0.f};  // (token g; q 2t, 2t+1), (token g+8; q 2t, 2t+1)
      float S2[4] = {0.f, 0.f, 0.f, 0.f};  // second accumulator: halves the dependent mma chain
      {
        const uint4* qp = reinterpret_cast<const uint4*>(st + COEF_TILE_BYTES + PAGES_PER_TILE * PB) + lane;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const uint4 v = qp[32 * k4];  // B fragments of k-steps 2*k4 and 2*k4+1
          mma_f32acc(S[0], S[1], S[2], S[3], acc[4 * k4][0], acc[4 * k4][1], acc[4 * k4 + 1][0], acc[4 * k4 + 1][1], v.x, v.y);
          mma_f32acc(S2[0], S2[1], S2[2], S2[3], acc[4 * k4 + 2][0], acc[4 * k4 + 2][1], acc[4 * k4 + 3][0], acc[4 * k4 + 3][1], v.z, v.w);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) S[i] += S2[i];
      }
      if (!v_first) unpack_v();
      // ---- online softmax, base 2; this lane owns queries 2t and 2t+1.  The running maximum only
      //      moves when a tile exceeds it by more than 2^8 (the sums stay far from overflow) ----
      {
        __half2 tm = __floats2half2_rn(fmaxf(S[0], S[2]), fmaxf(S[1], S[3]));
        tm = __hmax2(tm, u32_as_h2(__shfl_xor_sync(0xffffffffu, h2_as_u32(tm), 4)));
        tm = __hmax2(tm, u32_as_h2(__shfl_xor_sync(0xffffffffu, h2_as_u32(tm), 8)));
        tm = __hmax2(tm, u32_as_h2(__shfl_xor_sync(0xffffffffu, h2_as_u32(tm), 16)));
        const float2 tmf = __half22float2(tm);
        // fp16 rounds the maximum by at most 2^-11 relative; add a margin so that exp2 stays <= 2^9
        const bool need0 = (2 * t4 < G) && (tmf.x > m0 + 8.f), need1 = (2 * t4 + 1 < G) && (tmf.y > m1 + 8.f);
        if (__any_sync(0xffffffffu, need0 || need1)) {
          const float n0 = need0 ? tmf.x + 0.5f : m0, n1 = need1 ? tmf.y + 0.5f : m1;
          const float f0 = (m0 == -INFINITY) ? 0.f : ex2_approx(m0 - n0), f1 = (m1 == -INFINITY) ? 0.f : ex2_approx(m1 - n1);
          l0 *= f0, l1 *= f1, pn0 *= f0, pn1 *= f1, m0 = n0, m1 = n1;
#pragma unroll
          for (int mt = 0; mt < 8; ++mt) O[mt][0] *= f0, O[mt][1] *= f1, O[mt][2] *= f0, O[mt][3] *= f1;
        }
      }
      uint32_t pb0, pb1;
      {
        const float p0 = ex2_approx(S[0] - m0), p1 = ex2_approx(S[1] - m1);
        const float p2 = ex2_approx(S[2] - m0), p3 = ex2_approx(S[3] - m1);
        l0 += p0 + p2, l1 += p1 + p3;
        const __half* vn = reinterpret_cast<const __half*>(blk + k2b_off_vnorm(PAGE, g.group)) + 16 * wr + gq;
        const float na = __half2float(vn[0]), nb = __half2float(vn[8]);
        const float w0 = p0 * na, w1 = p1 * na, w2 = p2 * nb, w3 = p3 * nb;
        pn0 += w0 + w2, pn1 += w1 + w3;
        // (token g; q 2t, 2t+1) -> transpose -> (q g; tokens 2t, 2t+1): the B fragment of O^T += V^T P
        pb0 = movmatrix_trans(h2_as_u32(__floats2half2_rn(w0, w1)));
        pb1 = movmatrix_trans(h2_as_u32(__floats2half2_rn(w2, w3)));
      }
#pragma unroll
      for (int mt = 0; mt < 8; ++mt)
        mma_f32acc(O[mt][0], O[mt][1], O[mt][2], O[mt][3], VA[mt][0], VA[mt][1], VA[mt][2], VA[mt][3], pb0, pb1);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);
    if (++s == n_stages) s = 0, ph ^= 1;
  }
  if (cur_bh >= 0) flush(cur_b, cur_h);
}

// ---------------------------------------------------------------------------------------------
// Merge: one block of 256 threads per (sequence, KV head, query head).
//   1. attention over the fp16 recent window (keys already RoPE'd), as one more partial state
//      (bmx: src/bmx/cache/triton_dequant_attention.py:324-360)
//   2. the page-streaming kernel's partial records of this (sequence, head), folded by an online
//      softmax over records (bmx: :409-461; maxima are in log2 units on both sides)
//   3. the inverse value rotation of the packed part: signs * fwht(acc) / sqrt(128)
// The kernel is bound by the latency of its dependent global loads, not by bytes: it is laid out so that one
// (sequence, head, query) costs two load round trips before the grid dependency (window keys, window values)
// and one after it (all partial records of a thread in flight together).
// ---------------------------------------------------------------------------------------------
constexpr int MERGE_THREADS = 256;

__global__ void __launch_bounds__(MERGE_THREADS, 2) k2b_merge_kernel(const K2bMergeParams p) {
  extern __shared__ __align__(16) float msm[];
  const K2bGeom g = p.g;
  const int G = g.n_q_groups;
  const int cap4 = (p.tail_cap + 3) & ~3;
  float* sc = msm;             // [tail_cap] window scores, then weights
  float* qs = sc + cap4;       // [128] scaled query
  float* red = qs + HEAD_DIM;  // [16][128] window accumulators per token group; later [2][128] record halves
  float* atl = red + 16 * HEAD_DIM;  // [128] window accumulator
  float* sm = atl + HEAD_DIM;  // [32]: warp maxima [0..7], warp sums [8..15], record states [16..19]
  int* si = reinterpret_cast<int*>(sm + 32);  // tiles before this sequence, tiles in all
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int qi = blockIdx.x % G, bh = blockIdx.x / G, b = bh / g.h_kv, h = bh % g.h_kv;

  if (warp == 0) {
    int pre = 0, tot = 0;
    for (int i = lane; i < p.batch; i += 32) {
      const int t = tiles_of(p.n_pages[i], g.page) * g.h_kv;
      tot += t;
      if (i < b) pre += t;
    }
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) pre += __shfl_xor_sync(0xffffffffu, pre, m), tot += __shfl_xor_sync(0xffffffffu, tot, m);
    if (lane == 0) si[0] = pre, si[1] = tot;
  }
  if (tid < HEAD_DIM) qs[tid] = __half2float(p.q[((int64_t)bh * G + qi) * HEAD_DIM + tid]) * p.scale_log2;
  __syncthreads();

  // ---- window scores: eight lanes per token (16 channels each: 8l..8l+7 and 64+8l..), 32 tokens per pass ----
  const int tl = p.tail_len ? min(p.tail_len[b], p.tail_cap) : 0;
  const __half* kt = p.k_tail + (int64_t)bh * p.tail_cap * HEAD_DIM;
  const __half* vt = p.v_tail + (int64_t)bh * p.tail_cap * HEAD_DIM;
  float mx = -INFINITY;
  {
    const int l8 = tid & 7, tp = tid >> 3;
    float qr[16];
#pragma unroll
    for (int k = 0; k < 8; ++k) qr[k] = qs[8 * l8 + k], qr[8 + k] = qs[64 + 8 * l8 + k];
    for (int t0 = 0; t0 < tl; t0 += 256) {
      uint4 ka[8], kb[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {  // all loads of the chunk in flight together
        const int t = t0 + 32 * i + tp;
        const uint4* row = reinterpret_cast<const uint4*>(kt + (int64_t)min(t, tl - 1) * HEAD_DIM);
        ka[i] = row[l8], kb[i] = row[8 + l8];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int t = t0 + 32 * i + tp;
        const uint32_t w[8] = {ka[i].x, ka[i].y, ka[i].z, ka[i].w, kb[i].x, kb[i].y, kb[i].z, kb[i].w};
        float d = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float2 f = __half22float2(u32_as_h2(w[k]));
          d = fmaf(f.x, qr[2 * k], d), d = fmaf(f.y, qr[2 * k + 1], d);
        }
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        if (t < tl) {
          mx = fmaxf(mx, d);
          if (l8 == 0) sc[t] = d;
        }
      }
    }
  }
  // ---- window values: thread = (token group of 16, channel octet); the first 256 tokens' loads are issued before
  //      the softmax reductions so that they travel meanwhile ----
  const int c8 = tid & 15, tg = tid >> 4;
  uint4 vv[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int t = tg + 16 * i;
    vv[i] = (t < tl) ? reinterpret_cast<const uint4*>(vt + (int64_t)t * HEAD_DIM)[c8] : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
  if (lane == 0) sm[warp] = mx;
  __syncthreads();
  float m_w = sm[0];
#pragma unroll
  for (int w = 1; w < MERGE_THREADS / 32; ++w) m_w = fmaxf(m_w, sm[w]);
  float lsum = 0.f;
  for (int t = tid; t < tl; t += MERGE_THREADS) {
    const float e = ex2_approx(sc[t] - m_w);
    sc[t] = e, lsum += e;
  }
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, m);
  if (lane == 0) sm[8 + warp] = lsum;
  __syncthreads();
  float l_w = 0.f;
#pragma unroll
  for (int w = 0; w < MERGE_THREADS / 32; ++w) l_w += sm[8 + w];
  {
    float a[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) a[k] = 0.f;
    for (int t0 = 0; t0 < tl; t0 += 256) {
      if (t0 > 0) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const int t = t0 + tg + 16 * i;
          vv[i] = (t < tl) ? reinterpret_cast<const uint4*>(vt + (int64_t)t * HEAD_DIM)[c8] : make_uint4(0u, 0u, 0u, 0u);
        }
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int t = t0 + tg + 16 * i;
        const float wgt = (t < tl) ? sc[t] : 0.f;
        const uint32_t w[4] = {vv[i].x, vv[i].y, vv[i].z, vv[i].w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __half22float2(u32_as_h2(w[k]));
          a[2 * k] = fmaf(wgt, f.x, a[2 * k]), a[2 * k + 1] = fmaf(wgt, f.y, a[2 * k + 1]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) red[tg * HEAD_DIM + 8 * c8 + k] = a[k];
  }
  __syncthreads();
  if (tid < HEAD_DIM) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) s += red[k * HEAD_DIM + tid];
    atl[tid] = s;
  }
  // Everything above reads only what earlier steps' kernels wrote.  When this kernel was launched as a programmatic
  // dependent of the page-streaming kernel, that kernel's partial states are complete and visible from here on
  // (a plain launch passes straight through).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  __syncthreads();  // `red` is reused below

  // ---- partial records of the page-streaming kernel.  Record r of this (sequence, head): sub-record r / n_cta of
  //      CTA cta0 + r % n_cta.  Thread = (record parity, channel): an online softmax over its records ----
  const int total = si[1];
  const int per_cta = max(1, (total + p.main_grid - 1) / p.main_grid);
  const int tiles_b = tiles_of(p.n_pages[b], g.page);
  const int T0 = si[0] + h * tiles_b, T1 = T0 + tiles_b;
  const int cta0 = T0 / per_cta, cta1 = (tiles_b > 0) ? (T1 - 1) / per_cta : cta0 - 1;
  const int sub_slots = p.main_grid + p.batch * g.h_kv;
  const int n_cta = max(0, cta1 - cta0 + 1), n_rec = n_cta * p.n_sub;
  auto rec_ptr = [&](int r) {
    const int sb = r / n_cta, c = cta0 + (r - sb * n_cta);
    return p.part + ((int64_t)(sb * sub_slots + c + bh) * G + qi) * PART_STRIDE;
  };
  {
    const int ch = tid & 127, half = tid >> 7;
    float M = -INFINITY, L = 0.f, A = 0.f;
    for (int r0 = half; r0 < n_rec; r0 += 8) {
      float m_[4], l_[4], a_[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = r0 + 2 * j;
        if (r < n_rec) {
          const float* ps = rec_ptr(r);
          m_[j] = ps[0], l_[j] = ps[1], a_[j] = ps[2 + ch];
        } else {
          m_[j] = -INFINITY, l_[j] = 0.f, a_[j] = 0.f;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float Mn = fmaxf(M, m_[j]);
        const float fo = (M == -INFINITY) ? 0.f : ex2_approx(M - Mn);
        const float fn = (m_[j] == -INFINITY) ? 0.f : ex2_approx(m_[j] - Mn);
        L = L * fo + l_[j] * fn, A = A * fo + a_[j] * fn, M = Mn;
      }
    }
    red[half * HEAD_DIM + ch] = A;
    if (ch == 0) sm[16 + 2 * half] = M, sm[17 + 2 * half] = L;
  }
  __syncthreads();
  if (warp == 0) {
    const float M0 = sm[16], L0 = sm[17], M1 = sm[18], L1 = sm[19];
    const float Mp = fmaxf(M0, M1);
    const float f0 = (M0 == -INFINITY) ? 0.f : ex2_approx(M0 - Mp), f1 = (M1 == -INFINITY) ? 0.f : ex2_approx(M1 - Mp);
    const float Lp = L0 * f0 + L1 * f1;
    float x[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) x[k] = red[4 * lane + k] * f0 + red[HEAD_DIM + 4 * lane + k] * f1;
    if (p.signs != nullptr) {  // undo the value rotation (codecs without one pass signs == nullptr)
      fwht128_warp(x, lane);
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] = x[k] * p.signs[4 * lane + k] * 0.08838834764831845f;
    }
    const float mw = (tl > 0) ? m_w : -INFINITY;
    const float Mf = fmaxf(Mp, mw);
    const float fp = (Mp == -INFINITY) ? 0.f : ex2_approx(Mp - Mf), fw = (mw == -INFINITY) ? 0.f : ex2_approx(mw - Mf);
    const float l = Lp * fp + ((tl > 0) ? l_w : 0.f) * fw;
    const int64_t row = (int64_t)bh * G + qi;
    float val[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) val[k] = x[k] * fp + atl[4 * lane + k] * fw;
    if (p.partial_out) {
      float* po = p.partial_out + row * PART_STRIDE;
#pragma unroll
      for (int k = 0; k < 4; ++k) po[2 + 4 * lane + k] = val[k];
      if (lane == 0) po[0] = Mf, po[1] = l;
    } else if (p.out_dtype == BMXK_DTYPE_F32) {
      *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + row * HEAD_DIM + 4 * lane) =
          make_float4(val[0] / l, val[1] / l, val[2] / l, val[3] / l);
    } else {
      const __half2 h01 = __floats2half2_rn(val[0] / l, val[1] / l), h23 = __floats2half2_rn(val[2] / l, val[3] / l);
      *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(p.out) + row * HEAD_DIM + 4 * lane) = make_uint2(h2_as_u32(h01), h2_as_u32(h23));
    }
  }
}

// Merge of whole partial states across ranks or splits: parts (n_parts, rows, 130).
__global__ void merge_partials_kernel(const float* __restrict__ parts, int n_parts, int rows, void* out, int out_dtype) {
  const int row = blockIdx.x, ch = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < n_parts; ++s) M = fmaxf(M, parts[((int64_t)s * rows + row) * PART_STRIDE]);
  float l = 0.f, a = 0.f;
  for (int s = 0; s < n_parts; ++s) {
    const float* ps = parts + ((int64_t)s * rows + row) * PART_STRIDE;
    const float f = (ps[0] == -INFINITY) ? 0.f : ex2_approx(ps[0] - M);
    l += ps[1] * f;
    a += ps[2 + ch] * f;
  }
  const float r = a / l;
  if (out_dtype == BMXK_DTYPE_F32)
    reinterpret_cast<float*>(out)[(int64_t)row * HEAD_DIM + ch] = r;
  else
    reinterpret_cast<__half*>(out)[(int64_t)row * HEAD_DIM + ch] = __float2half_rn(r);
}

// Self-test of the bounded wait every decode kernel uses: one warp waits on an mbarrier on which nothing ever arrives.
// The wait must give up after `limit` cycles, record (block, site) in the status word and return, so that the
// kernel ends and the context stays usable.
__global__ void bounded_wait_selftest_kernel(int32_t* status, long long limit, int site) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  __syncthreads();
  const bool ok = wait_or_flag(&bar, 0, status, site, limit);
  if (threadIdx.x == 0) status[3] = ok ? 1 : 2;  // 2: the wait gave up, as it must
}

static int g_num_sms[MAX_DEVICES] = {};
int num_sms() {
  const int dev = current_device();
  int n = g_num_sms[dev];
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_num_sms[dev] = n;
  }
  return n;
}

int launch_merge(const K2bMergeParams& mp, cudaStream_t s, bool after_main) {
  const int G = mp.g.n_q_groups;
  const size_t msmem = ((size_t)((mp.tail_cap + 3) & ~3) + (1 + 16 + 1) * HEAD_DIM + 32 + 4) * sizeof(float);
  BMXK_REQUIRE(msmem <= 48 * 1024, "decode: tail_cap=%d too large for the merge kernel", mp.tail_cap);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(mp.batch * mp.g.h_kv * G)), cfg.blockDim = dim3(MERGE_THREADS), cfg.dynamicSmemBytes = msmem, cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = after_main ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, k2b_merge_kernel, mp);
  if (e != cudaSuccess) {
    set_error("decode(merge): %s", cudaGetErrorString(e));
    return BMXK_ERR_CUDA;
  }
  return check_launch("decode(merge)");
}

static size_t decode_stage_bytes(const bmxk_k2b_geom* g) {
  return (size_t)TILE_TOKENS * g->rank * 2 + (size_t)(TILE_TOKENS / g->page) * k2b_page_block_bytes(g->page, g->group) + 8 * 4 * 8 * 8;
}
static size_t decode_fixed_smem(int batch) {
  return (size_t)(DEC_CONSUMER_WARPS * 8 * HEAD_DIM + 3 * 64 + 8 * HEAD_DIM) * 4 + 32 * 8 + (size_t)(2 * batch + 1) * 4 + 16;
}

template <int RANK, int PAGE>
static int launch_decode(const K2bDecodeParams& prm, int grid, size_t smem, cudaStream_t s) {
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(k2b_decode_kernel<RANK, PAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
    if (e != cudaSuccess) {
      configured.retract();
      set_error("bmxk_k2b_decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return BMXK_ERR_CUDA;
    }
  }
  k2b_decode_kernel<RANK, PAGE><<<grid, DEC_THREADS, smem, s>>>(prm);
  return check_launch("bmxk_k2b_decode");
}

}  // namespace bmxk

// Built-in scratch of bmxk_k2b_decode_static: one copy per GPU that loads the library, held until the
// process exits.  Zero-initialised when the module is loaded.
static __device__ __align__(256) unsigned char g_static_scratch[BMXK_STATIC_SCRATCH_BYTES];
constexpr int kMaxStaticDevices = 64;
static void* g_static_ptr[kMaxStaticDevices] = {};
static std::mutex g_static_mu;

using namespace bmxk;

extern "C" {

size_t bmxk_k2b_decode_workspace_bytes(const bmxk_k2b_geom* g, int batch, int max_pages) {
  if (!g || batch <= 0) return 0;
  (void)max_pages;
  const size_t slots = ((size_t)num_sms() + (size_t)batch * g->h_kv) * (g->layout == 1 ? 2 : 1);
  return 256 + slots * g->n_q_groups * PART_STRIDE * sizeof(float);
}

int bmxk_k2b_decode(const bmxk_k2b_geom* g, const void* q, const void* pages, const void* coefs, const void* basis_f16,
                    const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch, int max_pages,
                    const void* rope_cos, const void* rope_sin, int64_t pos_offset, const void* k_tail,
                    const void* v_tail, const int32_t* tail_len, int tail_cap, const uint32_t* v_lut, const float* signs,
                    float sm_scale, void* workspace, size_t workspace_bytes, void* out, int out_dtype, float* partial_out,
                    int phases, void* stream) {
  BMXK_REQUIRE(g != nullptr, "bmxk_k2b_decode: null geometry");
  BMXK_REQUIRE(phases >= 1 && phases <= 3, "bmxk_k2b_decode: phases=%d must be 1, 2 or 3", phases);
  BMXK_REQUIRE(g->h_kv >= 1 && g->n_q_groups >= 1 && g->n_q_groups <= 8, "bmxk_k2b_decode: h_kv=%d n_q_groups=%d", g->h_kv,
               g->n_q_groups);
  BMXK_REQUIRE(g->page == 64 || g->page == 128, "bmxk_k2b_decode: page=%d must be 64 or 128", g->page);
  BMXK_REQUIRE(g->rank == 16 || g->rank == 32, "bmxk_k2b_decode: rank=%d must be 16 or 32", g->rank);
  BMXK_REQUIRE((g->group == 32 || g->group == 64 || g->group == 128) && g->page % g->group == 0,
               "bmxk_k2b_decode: group=%d must be 32/64/128 and divide page", g->group);
  BMXK_REQUIRE(g->n_coef_heads == 1 || g->n_coef_heads == g->h_kv, "bmxk_k2b_decode: n_coef_heads=%d", g->n_coef_heads);
  BMXK_REQUIRE(g->vbits == 2, "bmxk_k2b_decode: vbits=%d (only 2)", g->vbits);
  BMXK_REQUIRE(g->layout == 0 || (g->layout == 1 && g->page == 128), "bmxk_k2b_decode: layout=%d must be 0, or 1 with page=128",
               g->layout);
  BMXK_REQUIRE(batch >= 1 && (int64_t)batch * g->h_kv <= MAX_BH, "bmxk_k2b_decode: batch*h_kv=%lld out of range",
               (long long)batch * g->h_kv);
  BMXK_REQUIRE(max_pages >= 0 && tail_cap >= 0, "bmxk_k2b_decode: negative sizes");
  BMXK_REQUIRE(q && n_pages && v_lut && signs && workspace, "bmxk_k2b_decode: null pointer");
  BMXK_REQUIRE(max_pages == 0 || (pages && coefs && basis_f16 && page_table && rope_cos && rope_sin),
               "bmxk_k2b_decode: null page pool / tables");
  BMXK_REQUIRE(tail_cap == 0 || (k_tail && v_tail && tail_len), "bmxk_k2b_decode: null tail");
  BMXK_REQUIRE(out || partial_out, "bmxk_k2b_decode: no output");
  BMXK_REQUIRE(out_dtype == BMXK_DTYPE_F16 || out_dtype == BMXK_DTYPE_F32, "bmxk_k2b_decode: out_dtype=%d", out_dtype);
  BMXK_REQUIRE(workspace_bytes >= bmxk_k2b_decode_workspace_bytes(g, batch, max_pages), "bmxk_k2b_decode: workspace too small");
  BMXK_REQUIRE(((uintptr_t)pages & 15) == 0 && ((uintptr_t)coefs & 15) == 0, "bmxk_k2b_decode: pools must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;

  int32_t* status = reinterpret_cast<int32_t*>(workspace);
  float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256);
  const int64_t max_tiles = (int64_t)batch * g->h_kv * (((int64_t)max_pages * g->page + TILE_TOKENS - 1) / TILE_TOKENS);
  const int grid = (int)(max_tiles < num_sms() ? (max_tiles < 1 ? 1 : max_tiles) : num_sms());
  const float scale_log2 = sm_scale * 1.4426950408889634f;
  float alpha, beta;
  memcpy(&alpha, &v_lut[2], 4);
  memcpy(&beta, &v_lut[3], 4);

  if (max_pages > 0 && (phases & 1)) {
    K2bDecodeParams prm;
    prm.g.h_kv = g->h_kv, prm.g.n_q_groups = g->n_q_groups, prm.g.page = g->page, prm.g.rank = g->rank;
    prm.g.group = g->group, prm.g.n_coef_heads = g->n_coef_heads, prm.g.kbits = g->kbits, prm.g.vbits = g->vbits;
    prm.g.layout = g->layout;
    prm.q = (const __half*)q, prm.pages = (const uint8_t*)pages, prm.coefs = (const __half*)coefs;
    prm.basis16 = (const __half*)basis_f16, prm.page_table = page_table, prm.table_stride = table_stride;
    prm.n_pages = n_pages, prm.batch = batch, prm.rope_cos = (const __half*)rope_cos, prm.rope_sin = (const __half*)rope_sin;
    prm.pos_offset = pos_offset, prm.lut_lo = v_lut[0], prm.lut_hi = v_lut[1], prm.lut_alpha = alpha, prm.lut_beta = beta;
    prm.scale_log2 = scale_log2, prm.part = part, prm.status = status;
    if (g->layout == 1) {
      prm.n_stages = 0;
      const int rc5 = launch_decode_t5(prm, grid, s);
      if (rc5) return rc5;
    } else {
    const size_t stage = decode_stage_bytes(g), fixed = decode_fixed_smem(batch);
    int n_stages = (int)((220 * 1024 - fixed) / stage);
    if (n_stages > 8) n_stages = 8;
    BMXK_REQUIRE(n_stages >= 2, "bmxk_k2b_decode: shared memory too small for 2 stages");
    prm.n_stages = n_stages;
    const size_t smem = fixed + (size_t)n_stages * stage;
    int rc;
    if (g->rank == 32 && g->page == 128) rc = launch_decode<32, 128>(prm, grid, smem, s);
    else if (g->rank == 16 && g->page == 128) rc = launch_decode<16, 128>(prm, grid, smem, s);
    else if (g->rank == 32 && g->page == 64) rc = launch_decode<32, 64>(prm, grid, smem, s);
    else rc = launch_decode<16, 64>(prm, grid, smem, s);
    if (rc) return rc;
    }
  }
  if (!(phases & 2)) return BMXK_OK;
  K2bMergeParams mp;
  mp.g.h_kv = g->h_kv, mp.g.n_q_groups = g->n_q_groups, mp.g.page = g->page, mp.g.rank = g->rank, mp.g.group = g->group;
  mp.g.n_coef_heads = g->n_coef_heads, mp.g.kbits = g->kbits, mp.g.vbits = g->vbits, mp.g.layout = g->layout;
  mp.n_sub = (g->layout == 1) ? 2 : 1;  // the tcgen05 kernel keeps one state per tile parity
  mp.q = (const __half*)q, mp.n_pages = n_pages, mp.batch = batch, mp.main_grid = grid, mp.part = part;
  mp.k_tail = (const __half*)k_tail, mp.v_tail = (const __half*)v_tail, mp.tail_len = tail_cap > 0 ? tail_len : nullptr;
  mp.tail_cap = tail_cap, mp.signs = signs, mp.scale_log2 = scale_log2, mp.out = out, mp.out_dtype = out_dtype;
  mp.partial_out = partial_out;
  return launch_merge(mp, s, max_pages > 0 && (phases & 1));
}

int bmxk_k2b_decode_static(const bmxk_k2b_geom* g, const void* q, const void* pages, const void* coefs,
                           const void* basis_f16, const int32_t* page_table, int table_stride, const int32_t* n_pages,
                           int batch, int max_pages, const void* rope_cos, const void* rope_sin, int64_t pos_offset,
                           const void* k_tail, const void* v_tail, const int32_t* tail_len, int tail_cap,
                           const uint32_t* v_lut, const float* signs, float sm_scale, void* out, int out_dtype,
                           void* stream) {
  BMXK_REQUIRE(g != nullptr && batch >= 1, "bmxk_k2b_decode_static: null geometry or empty batch");
  const size_t need = bmxk_k2b_decode_workspace_bytes(g, batch, max_pages);
  BMXK_REQUIRE(need <= (size_t)BMXK_STATIC_SCRATCH_BYTES,
               "bmxk_k2b_decode_static: this call needs %zu bytes of scratch but the built-in scratch holds %d "
               "(batch*h_kv=%d, n_q_groups=%d); use bmxk_k2b_decode with a caller-owned workspace",
               need, BMXK_STATIC_SCRATCH_BYTES, batch * g->h_kv, g->n_q_groups);
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxStaticDevices) {
    set_error("bmxk_k2b_decode_static: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
    return BMXK_ERR_CUDA;
  }
  void* scratch = nullptr;
  {
    // First call on this device: resolve the device address of the built-in array.  The array's name
    // is only a host-side handle; what a kernel needs is the address cudaGetSymbolAddress returns for
    // the device that is current now.
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
      void* ptr = nullptr;
      e = cudaGetSymbolAddress(&ptr, g_static_scratch);
      if (e != cudaSuccess || ptr == nullptr) {
        set_error("bmxk_k2b_decode_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        return BMXK_ERR_CUDA;
      }
      g_static_ptr[dev] = ptr;
    }
    scratch = g_static_ptr[dev];
  }
  // The scratch keeps whatever the previous call left.  Partial states are fully rewritten by every
  // call; the status word at its start must read zero before the kernels run, so clear it in stream order.
  e = cudaMemsetAsync(scratch, 0, 256, (cudaStream_t)stream);
  if (e != cudaSuccess) {
    set_error("bmxk_k2b_decode_static: cudaMemsetAsync: %s", cudaGetErrorString(e));
    return BMXK_ERR_CUDA;
  }
  return bmxk_k2b_decode(g, q, pages, coefs, basis_f16, page_table, table_stride, n_pages, batch, max_pages, rope_cos,
                         rope_sin, pos_offset, k_tail, v_tail, tail_len, tail_cap, v_lut, signs, sm_scale, scratch,
                         (size_t)BMXK_STATIC_SCRATCH_BYTES, out, out_dtype, nullptr, 3, stream);
}

int bmxk_k2b_decode_static_status(void* stream) {
  const int dev = current_device();
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_mu);
    scratch = g_static_ptr[dev];
  }
  if (scratch == nullptr) return BMXK_OK;  // no call of bmxk_k2b_decode_static on this device yet: nothing to report
  return bmxk_check_workspace_status(scratch, stream);
}

int bmxk_selftest_bounded_wait(int32_t* status, int64_t limit_cycles, void* stream) {
  BMXK_REQUIRE(status != nullptr, "bmxk_selftest_bounded_wait: null status word");
  BMXK_REQUIRE(limit_cycles >= 1000 && limit_cycles <= 200000000LL,
               "bmxk_selftest_bounded_wait: limit of %lld cycles outside [1e3, 2e8] (this test must end within a fraction of a second)",
               (long long)limit_cycles);
  bounded_wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (long long)limit_cycles, 77);
  return check_launch("bmxk_selftest_bounded_wait");
}

int bmxk_k2b_make_v_lut(const float* codebook, uint32_t* out_lut) {
  BMXK_REQUIRE(codebook && out_lut, "bmxk_k2b_make_v_lut: null pointer");
  const double cb[4] = {codebook[0], codebook[1], codebook[2], codebook[3]};
  BMXK_REQUIRE(cb[0] < cb[1] && cb[1] < cb[2] && cb[2] < cb[3] && cb[0] < 0 && cb[3] > 0,
               "bmxk_k2b_make_v_lut: codebook must ascend through zero");
  // Search fp16 pairs (h0, h3) over two binades around the outer levels; each pair fixes the affine
  // map through levels 0 and 3, and the inner levels take the nearest fp16.  Keep the pair whose
  // worst inner error is smallest, with |alpha| small so that sum(P*h) carries no large offset.
  auto f16 = [](double x) { return (double)__half2float(__float2half_rn((float)x)); };
  auto bits16 = [](double x) { __half h = __float2half_rn((float)x); uint16_t u; memcpy(&u, &h, 2); return u; };
  double best = 1e30, bh[4] = {0, 0, 0, 0}, balpha = 0, bbeta = 1;
  for (int i3 = 0; i3 < 2048; ++i3) {
    uint16_t u3 = (uint16_t)(bits16(cb[3] * 0.5) + i3);
    __half hh3; memcpy(&hh3, &u3, 2);
    const double h3 = __half2float(hh3);
    const double h0c = h3 * cb[0] / cb[3];
    const uint16_t u0c = bits16(h0c);
    for (int d0 = -24; d0 <= 24; ++d0) {
      uint16_t u0 = (uint16_t)(u0c + d0);
      __half hh0; memcpy(&hh0, &u0, 2);
      const double h0 = __half2float(hh0);
      if (!(h0 < 0) || !(h3 > 0)) continue;
      const double beta = (cb[3] - cb[0]) / (h3 - h0), alpha = cb[0] - beta * h0;
      if (fabs(alpha) > 0.02) continue;
      const double h1 = f16((cb[1] - alpha) / beta), h2 = f16((cb[2] - alpha) / beta);
      const double e1 = fabs(alpha + beta * h1 - cb[1]), e2 = fabs(alpha + beta * h2 - cb[2]);
      const double e = e1 > e2 ? e1 : e2;
      if (e < best) best = e, bh[0] = h0, bh[1] = h1, bh[2] = h2, bh[3] = h3, balpha = alpha, bbeta = beta;
    }
  }
  BMXK_REQUIRE(best < 1e-3, "bmxk_k2b_make_v_lut: no fp16 table found");
  // Remove the mean residual under the Gaussian bin probabilities, so that the leftover per-level
  // error does not add up over many tokens.
  double mid[3] = {(cb[0] + cb[1]) / 2, (cb[1] + cb[2]) / 2, (cb[2] + cb[3]) / 2};
  auto Phi = [](double x) { return 0.5 * erfc(-x / sqrt(2.0)); };
  const double P[4] = {Phi(mid[0]), Phi(mid[1]) - Phi(mid[0]), Phi(mid[2]) - Phi(mid[1]), 1.0 - Phi(mid[2])};
  double bias = 0;
  for (int i = 0; i < 4; ++i) bias += P[i] * (balpha + bbeta * bh[i] - cb[i]);
  balpha -= bias;
  uint32_t lo = 0, hi = 0;
  for (int i = 0; i < 4; ++i) {
    const uint16_t u = bits16(bh[i]);
    lo |= (uint32_t)(u & 0xFF) << (8 * i);
    hi |= (uint32_t)(u >> 8) << (8 * i);
  }
  const float fa = (float)balpha, fb = (float)bbeta;
  out_lut[0] = lo, out_lut[1] = hi;
  memcpy(&out_lut[2], &fa, 4);
  memcpy(&out_lut[3], &fb, 4);
  return BMXK_OK;
}

int bmxk_merge_partials(const float* parts, int n_parts, int rows, void* out, int out_dtype, void* stream) {
  BMXK_REQUIRE(parts && out && n_parts >= 1 && rows >= 1, "bmxk_merge_partials: bad arguments");
  BMXK_REQUIRE(out_dtype == BMXK_DTYPE_F16 || out_dtype == BMXK_DTYPE_F32, "bmxk_merge_partials: out_dtype=%d", out_dtype);
  merge_partials_kernel<<<rows, HEAD_DIM, 0, (cudaStream_t)stream>>>(parts, n_parts, rows, out, out_dtype);
  return check_launch("bmxk_merge_partials");
}

int bmxk_check_workspace_status(const void* workspace, void* stream) {
  BMXK_REQUIRE(workspace != nullptr, "bmxk_check_workspace_status: null workspace");
  int32_t st[4] = {0, 0, 0, 0};
  cudaError_t e = cudaMemcpyAsync(st, workspace, sizeof(st), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) {
    set_error("bmxk_check_workspace_status: %s", cudaGetErrorString(e));
    return BMXK_ERR_CUDA;
  }
  if (st[0] == 2) {
    set_error("window append: a sequence's fp16 window was full (a flush was skipped); nothing was written");
    return BMXK_ERR_DEVICE;
  }
  if (st[0] != 0) {
    set_error("decode kernel: a bounded wait ran out in block %d (site %d)", st[1], st[2]);
    return BMXK_ERR_DEVICE;
  }
  return BMXK_OK;
}

}  // extern "C"
