// Paged dequant-prefill for the k2b cache on the sm_100a tensor-core path (tcgen05.mma + tensor memory).
//
// Same job and same grid as the mma.sync kernel of k2b_prefill.cu: one CTA owns 128 / G consecutive query positions
// of one (sequence, KV head) -- 128 attention rows with the G query heads -- and walks the visible 128-token pages and
// then the fp16 window.  Here the three contractions of a tile are tcgen05.mma instructions issued by three warps, the
// attention rows live on the 128 lanes of tensor memory (one softmax thread per row: no reduction across threads),
// and the dequantization of tile n+1 runs in its own warps while tile n is multiplied and normalised:
//
//   U1  K_low[128 tok x 128 ch]  = coef (smem, straight from the bulk copy) x basis^T (smem), fp16 accumulators
//   key warps (8; thread = token, two chunks of 16 + 16 channels):
//                                  K = K_low + scale * residual, rotated at the token's absolute position
//                                  -> shared memory, as the B operand of U2 (double-buffered by tile parity).
//                                  Two more "channels" carry log2(value norm) / scale as an fp16 pair (high part,
//                                  remainder) against two ones in Q, so that the scores arrive with the norm in the
//                                  exponent and the weights leave the softmax as p * norm with ONE rounding to fp16
//   U2  S[128 rows x 64 tok]     = Q (smem) x K^T over 144 channels, fp32, once per half of the tile: the two halves
//                                  have their own score and weight columns, so U2 of one half runs while the other
//                                  half is in the softmax
//   softmax warps (4; thread = row): one pass per half with the running maximum (base 2); only when a score exceeds it
//                                  by more than 8 is the accumulator rescaled and the half redone;
//                                  weights -> tensor memory as fp16 (A operand of U3)
//   value warps (8; thread = channel, warp = 64 tokens): 2-bit codes -> the four fp16 levels of the value table
//                                  -> shared memory as the B operand of U3.  Rows 128 / 129 of that operand hold
//                                  1 / norm as an fp16 pair and row 130 ones: the same contraction returns the sum
//                                  of the weights p (to 2^-22, from the rounded weights the numerator uses) and the
//                                  sum of p * norm (the affine term of the level table)
//   U3  O[128 rows x 144]       += P (TMEM) x V^T over the 64 tokens of the half, fp32
//
// The Hadamard rotation of the value codec is linear: it is undone once per row, in place in tensor memory, after
// the last page and before the first window tile (whose values are not rotated).  Window tiles take the same route
// with the key / value warps copying the fp16 window into the operand buffers (norm 1).
//
// Few query rows against a long context leave most SMs idle and one CTA with the whole page walk: with n_split > 1 the
// visible pages of a block are shared out over n_split CTAs, each writes a partial record per row (accumulators after
// the rotation is undone, running maximum, sum of weights) and a small kernel merges them.
//
// Every wait is bounded and reports through the status words; nothing here waits on another CTA.
#include "prefill_common.cuh"
#include "tc5.cuh"

namespace bmxk {

namespace {

constexpr int P5_THREADS = 768;  // warps 0-7 key, 8-11 softmax, 12 copies + U1, 13 U2, 14 U3 (15 idle), 16-23 value
constexpr int P5_STAGES = 3;
// Registers per thread after each group of four warps resizes itself; the pool is what the launch handed out.
constexpr int P5_REG_LAUNCH = 80, P5_REG_KEY = 112, P5_REG_SOFTMAX = 112, P5_REG_SERVICE = 48, P5_REG_VALUE = 48;
static_assert(8 * P5_REG_KEY + 4 * P5_REG_SOFTMAX + 4 * P5_REG_SERVICE + 8 * P5_REG_VALUE <= 24 * P5_REG_LAUNCH,
              "register split exceeds the CTA's pool");
// A [128 rows][144 K] fp16 operand in the unswizzled K-major form: 8-row x 16-byte core matrices, the 18 core matrices
// of one row group 128 bytes apart along K, row groups 2304 bytes apart.  K index 128 / 129: the norm pair (see above).
constexpr int OP_SBO = 18 * 128;
constexpr int OP_BYTES = 16 * OP_SBO;
constexpr int VROWS = 144;  // rows of the U3 operand: 128 channels, 1/norm (two rows), ones, 13 rows of zeros; K = 128 tokens
constexpr int V_SBO = 16 * 128;
constexpr int VOP_BYTES = (VROWS / 8) * V_SBO;
constexpr float MIN_NORM = 9.765625e-4f;  // 2^-10: a zero value vector keeps a weight the fp16 pair can carry
// TMEM columns: scores (64 per half of a tile), weights (fp16 pairs, 32 per half), output accumulator (128 channels, sum of p in two parts, sum of p x norm, 13 unused), K_low
constexpr uint32_t TM_S = 0, TM_P = 128, TM_O = 192, TM_KL = 336, TM_COLS = 512;

struct P5Smem {
  uint64_t full[P5_STAGES];          // raw tile landed (bulk copies)
  uint64_t low, sdone[2][2], odone[2];  // completion of U1, of U2 [half][tile parity] and of U3 [half] (tcgen05.commit)
  uint32_t tmem_base;
  // Arrivals, never reset: key warps (8 per tile, counted per tile parity: a key warp may be two tiles ahead of another
  // one, never two tiles of the same parity), value warps (8), scores read (4 per half tile), weights written (4 per half tile)
  // klcnt: key warps that hold K_low of the tile in registers (U1 of the next tile may start)
  int kcnt[2], klcnt[2], vcnt, scnt, pcnt;
};

// Per-role wait / work cycle counters of CTA (0, 0, 0), compiled in with -DP5_PROF only: written behind the status words
// (words 16 .. 71, in units of 16 cycles), so the status buffer of such a build must hold 72 words.
#ifdef P5_PROF
#define PROF_DECL(n) long long prof_acc[n] = {}; long long prof_t = clock64();
#define PROF_ADD(i) { const long long prof_n = clock64(); prof_acc[i] += prof_n - prof_t; prof_t = prof_n; }
#define PROF_OUT(base, n) if (lane == 0 && (warp & 3) == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) { for (int i_ = 0; i_ < n; ++i_) p.status[base + i_] = (int32_t)(prof_acc[i_] >> 4); }
#else
#define PROF_DECL(n)
#define PROF_ADD(i)
#define PROF_OUT(base, n)
#endif

__device__ __forceinline__ bool elect_one_p5() {
  uint32_t pred;
  asm volatile("{\n .reg .pred P;\n elect.sync _|P, 0xffffffff;\n selp.u32 %0, 1, 0, P;\n}\n" : "=r"(pred));
  return pred != 0;
}

// The bounded wait with one answer for the whole warp: what follows a wait is warp-wide (tcgen05.ld / st), so a warp
// leaves its loop together or not at all.
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity, int32_t* status, int where) {
  return __all_sync(0xffffffffu, wait_or_flag(bar, parity, status, where) ? 1 : 0) != 0;
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

}  // namespace

template <int RANK>
__global__ void __launch_bounds__(P5_THREADS, 1) k2b_prefill_t5_kernel(const PrefillParams p) {
  constexpr int KS = RANK / 16;
  constexpr int COEF_BYTES = 128 * RANK * 2;
  constexpr uint32_t AB_SBO = RANK * 16;  // bytes between 8-row groups of the coef / basis operands
  extern __shared__ __align__(128) uint8_t smem[];
  const K2bGeom g = p.g;
  const int G = g.n_q_groups, PP = 128 / G;  // query positions per CTA
  const int PB = k2b_page_block_bytes(128, g.group);
  const int STAGE_BYTES = COEF_BYTES + PB;

  uint8_t* stage0 = smem;                                  // [P5_STAGES][coefficient block | page block]
  uint8_t* qop = stage0 + P5_STAGES * STAGE_BYTES;         // A of U2
  uint8_t* kop0 = qop + OP_BYTES;                          // [2] B of U2
  uint8_t* vop = kop0 + 2 * OP_BYTES;                      // B of U3
  uint8_t* bop = vop + VOP_BYTES;                          // B of U1: this head's basis
  float* sg = reinterpret_cast<float*>(bop + COEF_BYTES);  // [128] signs / 128
  P5Smem* sh = reinterpret_cast<P5Smem*>(sg + 128);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // the latest positions see the most pages: their blocks are scheduled first, so that the last wave is the lightest
  // (blockIdx.x = position block * n_split + share: the shares of a block run side by side)
  const int n_split = p.n_split, share = (int)blockIdx.x % n_split, n_blocks = (int)gridDim.x / n_split;
  const int b = blockIdx.z, h = blockIdx.y, i0 = (n_blocks - 1 - (int)blockIdx.x / n_split) * PP;
  const int H = g.h_kv * G;

  const int64_t pq_min = p.q_pos0 + i0;                                // first query position of the CTA
  const int64_t pq_max = p.q_pos0 + min(i0 + PP, p.n_q) - 1;           // last one
  const int n_pg = p.n_pages[b];
  const int64_t vis = pq_max - p.pos_offset;
  const int NPv = (vis < 0) ? 0 : (int)min((int64_t)n_pg, vis / 128 + 1);  // pages whose first token the last position sees
  // this CTA's share of them: pages T0 .. T0 + NP - 1; the window goes with the last share
  const int per_share = (NPv + n_split - 1) / n_split;
  const int T0 = min(NPv, share * per_share), NP = min(NPv, T0 + per_share) - T0;
  const int tl = p.tail_len ? min(p.tail_len[b], p.tail_cap) : 0;
  const int64_t tail_pos0 = p.pos_offset + (int64_t)n_pg * 128;
  const int NW = (share == n_split - 1 && tl > 0 && pq_max >= tail_pos0) ? (int)((min((int64_t)tl, pq_max - tail_pos0 + 1) + 127) / 128) : 0;
  const int NT = NP + NW;
  const int64_t page_pos0 = p.pos_offset + (int64_t)T0 * 128;  // position of the first key of this share

  // ---- prologue: barriers, tensor memory, the operands that do not change (Q, basis, constant rows of V') ----
  if (tid == 0) {
    for (int s = 0; s < P5_STAGES; ++s) mbar_init(&sh->full[s], 1);
    mbar_init(&sh->low, 1);
    for (int e = 0; e < 2; ++e) mbar_init(&sh->sdone[0][e], 1), mbar_init(&sh->sdone[1][e], 1), mbar_init(&sh->odone[e], 1);
    sh->kcnt[0] = sh->kcnt[1] = sh->klcnt[0] = sh->klcnt[1] = sh->vcnt = sh->scnt = sh->pcnt = 0;
    fence_barrier_init();
  }
  if (warp == 12) {
    tc5::alloc(smem_u32(&sh->tmem_base), TM_COLS);
    tc5::relinquish();
  }
  for (int o = tid; o < 128 * 18; o += P5_THREADS) {  // row m = (query head m / PP, position i0 + m % PP)
    const int m = o / 18, c8 = o % 18;
    const int qi = m / PP, ip = min(i0 + m % PP, p.n_q - 1);
    uint4 v = make_uint4(c8 == 16 ? 0x3C003C00u : 0u, 0u, 0u, 0u);  // K index 128, 129: ones against the norm pair
    if (c8 < 16) v = reinterpret_cast<const uint4*>(p.q + (((int64_t)b * H + h * G + qi) * p.n_q + ip) * HEAD_DIM)[c8];
    *reinterpret_cast<uint4*>(qop + (m >> 3) * OP_SBO + c8 * 128 + (m & 7) * 16) = v;
    if (c8 == 17) {  // K index 136 .. 143 of both key buffers: zero for good
      *reinterpret_cast<uint4*>(kop0 + (m >> 3) * OP_SBO + 17 * 128 + (m & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
      *reinterpret_cast<uint4*>(kop0 + OP_BYTES + (m >> 3) * OP_SBO + 17 * 128 + (m & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
    }
  }
  {
    uint4* bd = reinterpret_cast<uint4*>(bop);
    const uint4* bs = reinterpret_cast<const uint4*>(p.basis16 + (int64_t)h * HEAD_DIM * RANK);
    for (int o = tid; o < 128 * (RANK / 8); o += P5_THREADS) {
      const int c = o / (RANK / 8), i8 = o % (RANK / 8);
      bd[((c >> 3) * (RANK / 8) + i8) * 8 + (c & 7)] = bs[o];
    }
  }
  for (int o = tid; o < 16 * 16; o += P5_THREADS) {  // rows 128 .. 143: 1/norm pair (rewritten per tile), ones, zeros
    const int r = 128 + (o >> 4), i = o & 15;
    const uint32_t w = (r == 130) ? 0x3C003C00u : 0u;
    *reinterpret_cast<uint4*>(vop + (r >> 3) * V_SBO + i * 128 + (r & 7) * 16) = make_uint4(w, w, w, w);
  }
  if (tid < 128) sg[tid] = p.signs[tid] * (1.0f / 128.0f);  // signs * fwht / sqrt(d), with the orthonormal fwht = butterflies / sqrt(d)
  fence_proxy_async();
  tc5::fence_before();
  __syncthreads();
  tc5::fence_after();
  const uint32_t tmem = sh->tmem_base;

  if (warp < 8) {
    // ===================== key warps: 32 token rows x two chunks of 16 + 16 channels =====================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(P5_REG_KEY));
    const int wq = warp & 3, k0 = 2 * (warp >> 2), row = 32 * wq + lane;
    const uint32_t tk = tmem + TM_KL + ((uint32_t)(32 * wq) << 16);
    const int grp = row / g.group;
    const __half2 c1032 = __floats2half2_rn(1032.f, 1032.f);
    const __half2 c16th = __floats2half2_rn(0.0625f, 0.0625f);
    const __half2 cm72 = __floats2half2_rn(-72.f, -72.f);
    const __half* kt = p.k_tail + ((int64_t)b * g.h_kv + h) * p.tail_cap * HEAD_DIM;
    const float inv_scale = 1.0f / p.scale_log2;
    // cos / sin of this token's rotary pairs 16k .. 16k+15 for both chunks, fetched one tile ahead: the registers of a
    // chunk are reloaded for the next tile as soon as the chunk is done, so the loads have a whole tile to land
    uint4 cs4[2][2], sn4[2][2];
    auto load_rope = [&](int n, int kk) {
      const int64_t pos = page_pos0 + (int64_t)n * 128 + row;
      const uint4* pc = reinterpret_cast<const uint4*>(p.rope_cos + pos * HEAD_DIM + 16 * (k0 + kk));
      const uint4* ps = reinterpret_cast<const uint4*>(p.rope_sin + pos * HEAD_DIM + 16 * (k0 + kk));
      cs4[kk][0] = pc[0], cs4[kk][1] = pc[1], sn4[kk][0] = ps[0], sn4[kk][1] = ps[1];
    };
    if (NP > 0) load_rope(0, 0), load_rope(0, 1);
    int s = 0;
    uint32_t fp = 0;
    PROF_DECL(6)
    for (int n = 0; n < NT; ++n) {
      const int e = n & 1;
      uint8_t* krow = kop0 + (size_t)e * OP_BYTES + (row >> 3) * OP_SBO + (row & 7) * 16;
      // the buffer still feeds U2 of tile n-2
      if (n >= 2 && !(warp_wait(&sh->sdone[0][e], (uint32_t)((n - 2) >> 1) & 1u, p.status, 41) &&
                      warp_wait(&sh->sdone[1][e], (uint32_t)((n - 2) >> 1) & 1u, p.status, 41))) break;
      PROF_ADD(0)
      if (n < NP) {
        const uint8_t* blk = stage0 + (size_t)s * STAGE_BYTES + COEF_BYTES;
        if (!warp_wait(&sh->full[s], fp, p.status, 42)) break;
        PROF_ADD(1)
        if (!warp_wait(&sh->low, (uint32_t)n & 1u, p.status, 43)) break;
        PROF_ADD(2)
        tc5::fence_after();
        uint32_t dl[2][8], dh[2][8];
        // all of this thread's K_low (both chunks) in one round trip; U1 of the next tile may then overwrite it
        tc5::ld16_pack(tk + 16 * k0, dl[0]);
        tc5::ld16_pack(tk + 64 + 16 * k0, dh[0]);
        tc5::ld16_pack(tk + 16 * k0 + 16, dl[1]);
        tc5::ld16_pack(tk + 64 + 16 * k0 + 16, dh[1]);
        if (k0 == 0) {  // K index 128, 129 of this token: log2(norm) / scale as high part + remainder
          const float nj = fmaxf(__half2float(reinterpret_cast<const __half*>(blk + k2b_off_vnorm(128, g.group))[row]), MIN_NORM);
          const float x = __log2f(nj) * inv_scale;
          const __half xh = __float2half_rn(x), xl = __float2half_rn(x - __half2float(xh));
          *reinterpret_cast<uint4*>(krow + 16 * 128) = make_uint4(h2_as_u32(__halves2half2(xh, xl)), 0u, 0u, 0u);
        }
        const uint4* ksc4 = reinterpret_cast<const uint4*>(blk + k2b_off_kscale(128)) + grp * 16;
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int k = k0 + kk;
          uint32_t out[16];
          const uint4 cw = reinterpret_cast<const uint4*>(blk)[k * 128 + row];
          const uint4 scl[2] = {ksc4[2 * k], ksc4[2 * k + 1]}, sch[2] = {ksc4[8 + 2 * k], ksc4[9 + 2 * k]};
          if (kk == 0) {
            tc5::wait_ld();
            PROF_ADD(3)
            tc5::fence_before();
            __syncwarp();
            if (lane == 0) smem_add_release(&sh->klcnt[e], 1);
          }
#pragma unroll
          for (int wd = 0; wd < 2; ++wd) {
            const uint32_t wlo = wd ? cw.y : cw.x, whi = wd ? cw.w : cw.z;
            const uint32_t sl[4] = {scl[wd].x, scl[wd].y, scl[wd].z, scl[wd].w}, sh_[4] = {sch[wd].x, sch[wd].y, sch[wd].z, sch[wd].w};
            const uint32_t cc_[4] = {cs4[kk][wd].x, cs4[kk][wd].y, cs4[kk][wd].z, cs4[kk][wd].w};
            const uint32_t ss_[4] = {sn4[kk][wd].x, sn4[kk][wd].y, sn4[kk][wd].z, sn4[kk][wd].w};
            __half2 rl[4], rh[4];
            {
              const uint32_t wl8 = wlo >> 8, wh8 = whi >> 8;
              rl[0] = __hsub2(u32_as_h2(lop3<0x6A>(wlo, 0x000F000Fu, 0x64086408u)), c1032);
              rl[1] = __hfma2(u32_as_h2(lop3<0x6A>(wlo, 0x00F000F0u, 0x64806480u)), c16th, cm72);
              rl[2] = __hsub2(u32_as_h2(lop3<0x6A>(wl8, 0x000F000Fu, 0x64086408u)), c1032);
              rl[3] = __hfma2(u32_as_h2(lop3<0x6A>(wl8, 0x00F000F0u, 0x64806480u)), c16th, cm72);
              rh[0] = __hsub2(u32_as_h2(lop3<0x6A>(whi, 0x000F000Fu, 0x64086408u)), c1032);
              rh[1] = __hfma2(u32_as_h2(lop3<0x6A>(whi, 0x00F000F0u, 0x64806480u)), c16th, cm72);
              rh[2] = __hsub2(u32_as_h2(lop3<0x6A>(wh8, 0x000F000Fu, 0x64086408u)), c1032);
              rh[3] = __hfma2(u32_as_h2(lop3<0x6A>(wh8, 0x00F000F0u, 0x64806480u)), c16th, cm72);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const __half2 klo = __hfma2(rl[i], u32_as_h2(sl[i]), u32_as_h2(dl[kk][4 * wd + i]));
              const __half2 khi = __hfma2(rh[i], u32_as_h2(sh_[i]), u32_as_h2(dh[kk][4 * wd + i]));
              const __half2 c = u32_as_h2(cc_[i]), sn = u32_as_h2(ss_[i]);
              out[4 * wd + i] = h2_as_u32(__hfma2(__hneg2(sn), khi, __hmul2(klo, c)));
              out[8 + 4 * wd + i] = h2_as_u32(__hfma2(sn, klo, __hmul2(khi, c)));
            }
          }
          if (n + 1 < NP) load_rope(n + 1, kk);
          // channels 16k .. 16k+15 are 16-byte chunks 2k, 2k+1 of the row; channels 64+16k .. are chunks 8+2k, 9+2k
          *reinterpret_cast<uint4*>(krow + (2 * k) * 128) = make_uint4(out[0], out[1], out[2], out[3]);
          *reinterpret_cast<uint4*>(krow + (2 * k + 1) * 128) = make_uint4(out[4], out[5], out[6], out[7]);
          *reinterpret_cast<uint4*>(krow + (8 + 2 * k) * 128) = make_uint4(out[8], out[9], out[10], out[11]);
          *reinterpret_cast<uint4*>(krow + (9 + 2 * k) * 128) = make_uint4(out[12], out[13], out[14], out[15]);
        }
        if (++s == P5_STAGES) s = 0, fp ^= 1u;
      } else {
        // window tile: the keys are stored rotated; rows past the window's length are zero; norm 1
        const int t0 = (n - NP) * 128;
        const bool valid = t0 + row < tl;
        const uint4* src = reinterpret_cast<const uint4*>(kt + (int64_t)(t0 + row) * HEAD_DIM);
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
          const int k = k0 + kk;
          const int cks[4] = {2 * k, 2 * k + 1, 8 + 2 * k, 9 + 2 * k};
#pragma unroll
          for (int i = 0; i < 4; ++i) *reinterpret_cast<uint4*>(krow + cks[i] * 128) = valid ? src[cks[i]] : make_uint4(0u, 0u, 0u, 0u);
        }
        if (k0 == 0) *reinterpret_cast<uint4*>(krow + 16 * 128) = make_uint4(0u, 0u, 0u, 0u);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) smem_add_release(&sh->kcnt[e], 1);
      PROF_ADD(4)
    }
    PROF_OUT(16, 6)
  } else if (warp >= 16) {
    // ===================== value warps: thread = channel, warp = one half (64 tokens) of the tile =====================
    // (levels as stored in the table: the norm is in the weights)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(P5_REG_VALUE));
    const int wq = warp & 3, cc = (warp - 16) >> 2, ch = 32 * wq + lane;
    uint8_t* vrow = vop + (ch >> 3) * V_SBO + (ch & 7) * 16;
    __half* vinv = reinterpret_cast<__half*>(vop + 16 * V_SBO + (ch >> 3) * 128) + (ch & 7);  // rows 128 / 129, token = ch (warps 16 - 19)
    const __half* vt = p.v_tail + ((int64_t)b * g.h_kv + h) * p.tail_cap * HEAD_DIM;
    int s = 0;
    uint32_t fp = 0;
    PROF_DECL(4)
    for (int n = 0; n < NT; ++n) {
      // the buffer still feeds U3 of tile n-1
      if (n >= 1 && !(warp_wait(&sh->odone[0], (uint32_t)(n - 1) & 1u, p.status, 44) && warp_wait(&sh->odone[1], (uint32_t)(n - 1) & 1u, p.status, 44))) break;
      PROF_ADD(0)
      if (n < NP) {
        if (!warp_wait(&sh->full[s], fp, p.status, 45)) break;
        PROF_ADD(1)
        const uint8_t* blk = stage0 + (size_t)s * STAGE_BYTES + COEF_BYTES;
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
          *reinterpret_cast<uint4*>(vrow + (8 * cc + 2 * jw) * 128) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
          *reinterpret_cast<uint4*>(vrow + (8 * cc + 2 * jw + 1) * 128) = make_uint4(outw[4], outw[5], outw[6], outw[7]);
        }
        if (cc == 0) {  // rows 128 / 129, token = ch: 1 / norm as high part + remainder
          const float nj = fmaxf(__half2float(reinterpret_cast<const __half*>(blk + k2b_off_vnorm(128, g.group))[ch]), MIN_NORM);
          const float r = 1.0f / nj;
          const __half rh = __float2half_rn(r);
          vinv[0] = rh, vinv[8] = __float2half_rn(r - __half2float(rh));
        }
        if (++s == P5_STAGES) s = 0, fp ^= 1u;
      } else {
        // window tile: values as stored, transposed; tokens past the window's length are zero
        const int t0 = (n - NP) * 128;
#pragma unroll 1
        for (int i = 0; i < 8; ++i) {
          uint32_t w4[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int ta = t0 + 64 * cc + 8 * i + 2 * j;
            const __half a = (ta < tl) ? vt[(int64_t)ta * HEAD_DIM + ch] : __float2half_rn(0.f);
            const __half c = (ta + 1 < tl) ? vt[(int64_t)(ta + 1) * HEAD_DIM + ch] : __float2half_rn(0.f);
            w4[j] = h2_as_u32(__halves2half2(a, c));
          }
          *reinterpret_cast<uint4*>(vrow + (8 * cc + i) * 128) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
        }
        if (cc == 0) vinv[0] = __float2half_rn(1.f), vinv[8] = __float2half_rn(0.f);
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) smem_add_release(&sh->vcnt, 1);
      PROF_ADD(2)
    }
    PROF_OUT(32, 4)
  } else if (warp < 12) {
    // ===================== softmax warps: thread = attention row = TMEM lane =====================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(P5_REG_SOFTMAX));
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t tl_ = tmem + ((uint32_t)(32 * wq) << 16);
    const int qi = row / PP, ip = i0 + row % PP;
    const int64_t pq = p.q_pos0 + ip;
    float m = -1e30f;
    bool alive = true;

    // O <- signs * fwht(alpha * sum(p n) + beta * O) / 128, in place (columns 0 .. 127 of the accumulator)
    auto unrotate = [&]() {
      uint32_t r4[4];
      tc5::ld4(tl_ + TM_O + 128, r4);
      tc5::wait_ld();
      const float add = p.lut_alpha * __uint_as_float(r4[2]);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {  // index bits 0 .. 4: inside each chunk of 32 columns
        uint32_t r[32];
        tc5::ld32(tl_ + TM_O + 32 * c, r);
        tc5::wait_ld();
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = fmaf(p.lut_beta, __uint_as_float(r[i]), add);
#pragma unroll
        for (int hb = 1; hb < 32; hb <<= 1)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (!(i & hb)) {
              const float a = v[i], bb = v[i | hb];
              v[i] = a + bb, v[i | hb] = a - bb;
            }
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(v[i]);
        tc5::st32(tl_ + TM_O + 32 * c, r);
      }
      tc5::wait_st();
#pragma unroll 1
      for (int j0 = 0; j0 < 32; j0 += 8) {  // index bits 5, 6: across the four chunks
        uint32_t a0[8], a1[8], a2[8], a3[8];
        tc5::ld8(tl_ + TM_O + j0, a0);
        tc5::ld8(tl_ + TM_O + 32 + j0, a1);
        tc5::ld8(tl_ + TM_O + 64 + j0, a2);
        tc5::ld8(tl_ + TM_O + 96 + j0, a3);
        tc5::wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float x0 = __uint_as_float(a0[i]), x1 = __uint_as_float(a1[i]), x2 = __uint_as_float(a2[i]), x3 = __uint_as_float(a3[i]);
          const float y0 = x0 + x1, y1 = x0 - x1, y2 = x2 + x3, y3 = x2 - x3;
          a0[i] = __float_as_uint((y0 + y2) * sg[j0 + i]);
          a1[i] = __float_as_uint((y1 + y3) * sg[32 + j0 + i]);
          a2[i] = __float_as_uint((y0 - y2) * sg[64 + j0 + i]);
          a3[i] = __float_as_uint((y1 - y3) * sg[96 + j0 + i]);
        }
        tc5::st8(tl_ + TM_O + j0, a0);
        tc5::st8(tl_ + TM_O + 32 + j0, a1);
        tc5::st8(tl_ + TM_O + 64 + j0, a2);
        tc5::st8(tl_ + TM_O + 96 + j0, a3);
      }
      tc5::wait_st();
    };
    // 32 scores (token columns col0 .. of the half tile) -> weights with the running maximum -> 16 columns of fp16
    // pairs; returns the maximum of the visible scores together with `acc`
    auto weights32 = [&](const uint32_t (&r)[32], uint32_t tp, int col0, bool masked, int jl, float negm, float acc) {
      uint32_t pk[16];
      if (masked) {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const bool v0 = col0 + 2 * i < jl, v1 = col0 + 2 * i + 1 < jl;
          const float s0 = __uint_as_float(r[2 * i]), s1 = __uint_as_float(r[2 * i + 1]);
          acc = fmaxf(acc, fmaxf(v0 ? s0 : -INFINITY, v1 ? s1 : -INFINITY));
          pk[i] = pack_h2(v0 ? ex2_approx(fmaf(s0, p.scale_log2, negm)) : 0.f, v1 ? ex2_approx(fmaf(s1, p.scale_log2, negm)) : 0.f);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float s0 = __uint_as_float(r[2 * i]), s1 = __uint_as_float(r[2 * i + 1]);
          acc = fmaxf(acc, fmaxf(s0, s1));
          pk[i] = pack_h2(ex2_approx(fmaf(s0, p.scale_log2, negm)), ex2_approx(fmaf(s1, p.scale_log2, negm)));
        }
      }
      tc5::st16(tp + (col0 >> 1), pk);
      return acc;
    };

    // keys of the current half visible to this row / to the CTA's first row: position - first key position + 1
    int64_t rel = pq - page_pos0 + 1, rel_min = pq_min - page_pos0 + 1;
    PROF_DECL(8)
    for (int u = 0; u < 2 * NT && alive; ++u) {  // half tile u = (tile n, half hf): tokens 64 hf .. 64 hf + 63
      const int n = u >> 1, hf = u & 1, e = n & 1;
      if (u == 2 * NP) rel = pq - tail_pos0 + 1, rel_min = pq_min - tail_pos0 + 1;  // the window's first token follows the last page
      const int n_valid = (n < NP) ? 64 : max(0, min(64, tl - (n - NP) * 128 - 64 * hf));
      const bool masked = (rel_min < 64) || (n_valid < 64);                               // the same for the whole CTA
      const int jl = (int)max((int64_t)0, min((int64_t)n_valid, rel));                    // keys [0, jl) of the half are visible to this row
      rel -= 64, rel_min -= 64;
      const uint32_t tS = tl_ + TM_S + 64 * hf, tP = tl_ + TM_P + 32 * hf;
      if (u == 2 * NP && NP > 0) {  // first window tile after pages: leave the rotated space of the value codec
        if (!(warp_wait(&sh->odone[0], (uint32_t)(n - 1) & 1u, p.status, 46) && warp_wait(&sh->odone[1], (uint32_t)(n - 1) & 1u, p.status, 46))) {
          alive = false;
          break;
        }
        tc5::fence_after();
        unrotate();
      }
      PROF_ADD(0)
      if (!warp_wait(&sh->sdone[hf][e], (uint32_t)(n >> 1) & 1u, p.status, 47)) { alive = false; break; }
      PROF_ADD(1)
      // the weight columns of this half still feed U3 of the previous tile's same half
      if (n >= 1 && !warp_wait(&sh->odone[hf], (uint32_t)(n - 1) & 1u, p.status, 48)) { alive = false; break; }
      tc5::fence_after();
      PROF_ADD(2)
      for (int attempt = 0; attempt < 2; ++attempt) {
        uint32_t ra[32], rb[32];
        const float negm = -m;
        tc5::ld32(tS, ra);
        tc5::ld32(tS + 32, rb);
        tc5::wait_ld();
        float tmax = weights32(ra, tP, 0, masked, jl, negm, -INFINITY);
        tmax = weights32(rb, tP, 32, masked, jl, negm, tmax);
        // Lazy maximum: as long as no score exceeds the running maximum by more than 8 (weights below 2^8) the weights
        // just written stand.  Otherwise the whole warp (TMEM access is warp-wide) rescales its rows of the accumulator
        // once every earlier U3 has finished, and goes through the half again with the new maximum.
        const float ts = tmax * p.scale_log2;
        const bool need = ts > m + 8.f;
        if (!__any_sync(0xffffffffu, need)) break;
        if (u > 0) {  // the U3 just before this half: the other half of this tile, or of the previous one
          const bool ok = hf ? warp_wait(&sh->odone[0], (uint32_t)n & 1u, p.status, 50) : warp_wait(&sh->odone[1], (uint32_t)(n - 1) & 1u, p.status, 50);
          if (!ok) { alive = false; break; }
          tc5::fence_after();
        }
        const float f = need ? ex2_approx(m - ts) : 1.f;
        if (need) m = ts;
        if (u > 0) {
          uint32_t r4[4];
          tc5::ld4(tl_ + TM_O + 128, r4);
          tc5::wait_ld();
#pragma unroll
          for (int i = 0; i < 4; ++i) r4[i] = __float_as_uint(__uint_as_float(r4[i]) * f);
          tc5::st4(tl_ + TM_O + 128, r4);
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t r[32];
            tc5::ld32(tl_ + TM_O + 32 * c, r);
            tc5::wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * f);
            tc5::st32(tl_ + TM_O + 32 * c, r);
          }
        }
      }
      if (!alive) break;
      PROF_ADD(3)
      // every score of the half has been read: U2 of the next tile's same half may overwrite them
      tc5::fence_before();
      __syncwarp();
      if (lane == 0) smem_add_release(&sh->scnt, 1);
      tc5::wait_st();
      tc5::fence_before();
      __syncwarp();
      if (lane == 0) smem_add_release(&sh->pcnt, 1);
      PROF_ADD(4)
    }
    PROF_OUT(48, 8)

    // ---- the last U3, the rotation if no window tile undid it, normalise and store ----
    if (alive && NT > 0 && !(warp_wait(&sh->odone[0], (uint32_t)(NT - 1) & 1u, p.status, 49) && warp_wait(&sh->odone[1], (uint32_t)(NT - 1) & 1u, p.status, 49)))
      alive = false;
    if (alive) {
      float inv = 0.f;
      if (NT > 0) {
        tc5::fence_after();
        if (NW == 0) unrotate();
        uint32_t r4[4];
        tc5::ld4(tl_ + TM_O + 128, r4);
        tc5::wait_ld();
        const float l = __uint_as_float(r4[0]) + __uint_as_float(r4[1]);
        inv = (l > 0.f) ? 1.f / l : 0.f;
      }
      const int64_t grow = ((int64_t)b * H + h * G + qi) * p.n_q + ip;  // row of q / out
      if (n_split > 1) {  // partial record of this share: unnormalised accumulators, running maximum, sum of weights
        float* rec = p.part + (grow * n_split + share) * PF_PART_STRIDE;
        float lsum = 0.f;
        if (NT > 0) {
          uint32_t r4[4];
          tc5::ld4(tl_ + TM_O + 128, r4);
          tc5::wait_ld();
          lsum = __uint_as_float(r4[0]) + __uint_as_float(r4[1]);
        }
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t r[32];
          if (NT > 0) {
            tc5::ld32(tl_ + TM_O + 32 * c, r);
            tc5::wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = 0u;
          }
          if (ip < p.n_q) {
#pragma unroll
            for (int j = 0; j < 8; ++j) reinterpret_cast<uint4*>(rec + 32 * c)[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          }
        }
        if (ip < p.n_q) *reinterpret_cast<float4*>(rec + 128) = make_float4(m, lsum, 0.f, 0.f);
      } else {
      uint4* dst = reinterpret_cast<uint4*>(p.out + grow * HEAD_DIM);
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        if (NT > 0) {
          tc5::ld32(tl_ + TM_O + 32 * c, r);
          tc5::wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (ip < p.n_q) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t w4[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
              w4[i] = pack_h2(__uint_as_float(r[8 * j + 2 * i]) * inv, __uint_as_float(r[8 * j + 2 * i + 1]) * inv);
            dst[4 * c + j] = make_uint4(w4[0], w4[1], w4[2], w4[3]);
          }
        }
      }
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(P5_REG_SERVICE));
    // ===================== service warps: 12 copies + U1, 13 U2, 14 U3 (15 idle) =====================
    // Tile n:  copy -> full[n % 3];  A: U1 -> low;  per half hf:  B: U2 -> sdone[hf][n & 1];  C: U3 -> odone[hf].
    // A(n) needs the copy landed and K_low of tile n-1 read by every key warp; B(n, hf) the keys of tile n and the
    // scores of the same half of tile n-1 read; C(n, hf) the weights of the half and the values of tile n; copy(n) the
    // raw stage of tile n-3 consumed by the key and value warps.  A thread gets an MMA out every 100 - 200 cycles, far
    // less than the tensor pipe takes: the three contractions are issued by three warps, each polling only the counters
    // its own action needs.  A whole warp walks its state machine, one elected lane issues.
    const bool el = elect_one_p5();
    long long t_last = clock64();
    uint32_t idle = 0;
    bool ok = true;
    // bounded polling: gives up (and says where) once nothing has moved for the wait limit, or another wait gave up
    auto stalled = [&](bool progressed, int where) {
      if (progressed) {
        idle = 0;
      } else if ((++idle & 255u) == 0u) {
        if (idle == 256u) t_last = clock64();
        if (clock64() - t_last > WAIT_LIMIT_CYCLES || *reinterpret_cast<volatile int32_t*>(p.status) != 0) {
          if (el && atomicCAS(p.status, 0, 1) == 0) p.status[1] = blockIdx.x, p.status[2] = where;
          return true;
        }
      }
      return false;
    };
    if (warp == 12) {
      constexpr uint32_t ID_U1 = tc5::idesc_f16_f16(128, 128);
      const uint64_t d_stage = tc5::smem_desc(smem_u32(stage0), 128, AB_SBO), d_b = tc5::smem_desc(smem_u32(bop), 128, AB_SBO);
      const int chd = (g.n_coef_heads == 1) ? 0 : h;
      const int32_t* table = p.page_table + (int64_t)b * p.table_stride + T0;
      int nP = 0, nA = 0, sP = 0, sA = 0;
      uint32_t phA = 0;
      int slot = (NP > 0) ? table[0] : 0;  // page slot of the next copy, fetched one copy ahead
      while (ok && nA < NP) {
        bool progressed = false;
        const int kc0 = smem_load_acquire(&sh->kcnt[0]), kc1 = smem_load_acquire(&sh->kcnt[1]), vc = smem_load_acquire(&sh->vcnt);
        const int kl0 = smem_load_acquire(&sh->klcnt[0]), kl1 = smem_load_acquire(&sh->klcnt[1]);
        auto kdone = [&](int t) { return t < 0 || ((t & 1) ? kc1 : kc0) >= 8 * ((t >> 1) + 1); };   // every key warp is through tile t
        auto kldone = [&](int t) { return t < 0 || ((t & 1) ? kl1 : kl0) >= 8 * ((t >> 1) + 1); };  // ... holds K_low of tile t in registers
        // ---- A ----
        if (nA < nP && kldone(nA - 1) && mbar_test_wait(&sh->full[sA], phA)) {
          tc5::fence_after();
          const uint64_t da = d_stage + (uint64_t)(sA * (STAGE_BYTES >> 4));
          if (el) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) tc5::mma_ss(tmem + TM_KL, da + 16 * ks, d_b + 16 * ks, ID_U1, ks > 0);
            tc5::commit(smem_u32(&sh->low));
          }
          __syncwarp();
          ++nA;
          if (++sA == P5_STAGES) sA = 0, phA ^= 1u;
          progressed = true;
        }
        // ---- copy ----
        if (nP < NP && (nP < P5_STAGES || (kdone(nP - P5_STAGES) && vc >= 8 * (nP - P5_STAGES + 1)))) {
          uint8_t* st = stage0 + (size_t)sP * STAGE_BYTES;
          if (el) {
            mbar_arrive_expect_tx(&sh->full[sP], (uint32_t)STAGE_BYTES);
            bulk_g2s(st, reinterpret_cast<const uint8_t*>(p.coefs) + ((int64_t)slot * g.n_coef_heads + chd) * COEF_BYTES, COEF_BYTES,
                     &sh->full[sP]);
            bulk_g2s(st + COEF_BYTES, p.pages + ((int64_t)slot * g.h_kv + h) * PB, PB, &sh->full[sP]);
          }
          __syncwarp();
          ++nP;
          if (++sP == P5_STAGES) sP = 0;
          if (nP < NP) slot = table[nP];
          progressed = true;
        }
        if (stalled(progressed, 40)) ok = false;
      }
    } else if (warp == 13) {
      constexpr uint32_t ID_U2 = tc5::idesc_f16_f32(128, 64);
      const uint64_t d_q = tc5::smem_desc(smem_u32(qop), 128, OP_SBO), d_k = tc5::smem_desc(smem_u32(kop0), 128, OP_SBO);
      int uB = 0;  // half tiles issued
      while (ok && uB < 2 * NT) {
        const int n = uB >> 1, hf = uB & 1;
        const int kc = smem_load_acquire(&sh->kcnt[n & 1]), sc = smem_load_acquire(&sh->scnt);
        bool progressed = false;
        if (kc >= 8 * ((n >> 1) + 1) && sc >= 4 * (uB - 1)) {
          tc5::fence_after();
          const uint64_t db = d_k + (uint64_t)((n & 1) * (OP_BYTES >> 4) + hf * (8 * OP_SBO >> 4));  // token rows 64 hf ..
          if (el) {
#pragma unroll
            for (int ks = 0; ks < 9; ++ks) tc5::mma_ss(tmem + TM_S + 64 * hf, d_q + 16 * ks, db + 16 * ks, ID_U2, ks > 0);  // 144 channels
            tc5::commit(smem_u32(&sh->sdone[hf][n & 1]));
          }
          __syncwarp();
          ++uB;
          progressed = true;
        }
        if (stalled(progressed, 51)) ok = false;
      }
    } else if (warp == 14) {
      constexpr uint32_t ID_U3 = tc5::idesc_f16_f32(128, VROWS);
      const uint64_t d_v = tc5::smem_desc(smem_u32(vop), 128, V_SBO);
      int uC = 0;
      while (ok && uC < 2 * NT) {
        const int hf = uC & 1;
        const int pc = smem_load_acquire(&sh->pcnt), vc = smem_load_acquire(&sh->vcnt);
        bool progressed = false;
        if (pc >= 4 * (uC + 1) && vc >= 8 * ((uC >> 1) + 1)) {
          tc5::fence_after();
          if (el) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)  // 64 tokens of the half: weight columns 32 hf .., token chunks 8 hf ..
              tc5::mma_ts(tmem + TM_O, tmem + TM_P + 32 * hf + 8 * ks, d_v + 64 * hf + 16 * ks, ID_U3, (uC > 0 || ks > 0) ? 1u : 0u);
            tc5::commit(smem_u32(&sh->odone[hf]));
          }
          __syncwarp();
          ++uC;
          progressed = true;
        }
        if (stalled(progressed, 52)) ok = false;
      }
    }
  }

  // ---- epilogue: every role ends here; the tensor memory goes back before the CTA leaves ----
  tc5::fence_before();
  __syncthreads();
  if (warp == 12) {
    tc5::fence_after();
    tc5::dealloc(tmem, TM_COLS);
  }
}

static size_t p5_smem_bytes(int rank, int group) {
  return (size_t)P5_STAGES * ((size_t)128 * rank * 2 + k2b_page_block_bytes(128, group)) + 3 * (size_t)OP_BYTES + VOP_BYTES +
         (size_t)128 * rank * 2 + 128 * 4 + sizeof(P5Smem) + 128;
}

template <int RANK>
static int launch_p5(const PrefillParams& prm, dim3 grid, size_t smem, cudaStream_t s) {
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(k2b_prefill_t5_kernel<RANK>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      configured.retract();
      set_error("bmxk_k2b_prefill: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return BMXK_ERR_CUDA;
    }
  }
  k2b_prefill_t5_kernel<RANK><<<grid, P5_THREADS, smem, s>>>(prm);
  return check_launch("bmxk_k2b_prefill(tcgen05)");
}

// out[row] = sum_s 2^(m_s - M) O_s / sum_s 2^(m_s - M) l_s over the n_split partial records of the row; one block of 128
// threads (one per channel) per row.
__global__ void __launch_bounds__(128) prefill_merge_kernel(const float* __restrict__ part, int n_split, __half* __restrict__ out) {
  const int64_t row = blockIdx.x;
  const float* rec = part + row * n_split * PF_PART_STRIDE;
  float M = -INFINITY;
  for (int s = 0; s < n_split; ++s) M = fmaxf(M, rec[s * PF_PART_STRIDE + 128]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < n_split; ++s) {
    const float w = ex2_approx(rec[s * PF_PART_STRIDE + 128] - M);
    acc = fmaf(w, rec[s * PF_PART_STRIDE + threadIdx.x], acc);
    l = fmaf(w, rec[s * PF_PART_STRIDE + 129], l);
  }
  out[row * HEAD_DIM + threadIdx.x] = __float2half_rn(l > 0.f ? acc / l : 0.f);
}

int launch_prefill_t5(const PrefillParams& prm, dim3 grid, cudaStream_t s) {
  const size_t smem = p5_smem_bytes(prm.g.rank, prm.g.group);
  BMXK_REQUIRE(smem <= 227 * 1024, "bmxk_k2b_prefill: rank=%d group=%d needs %zu bytes of shared memory", prm.g.rank, prm.g.group, smem);
  const int rc = prm.g.rank == 32 ? launch_p5<32>(prm, grid, smem, s) : launch_p5<16>(prm, grid, smem, s);
  if (rc != BMXK_OK || prm.n_split <= 1) return rc;
  const int64_t rows = (int64_t)grid.z * prm.g.h_kv * prm.g.n_q_groups * prm.n_q;
  prefill_merge_kernel<<<(unsigned)rows, 128, 0, s>>>(prm.part, prm.n_split, prm.out);
  return check_launch("bmxk_k2b_prefill(merge)");
}

}  // namespace bmxk
