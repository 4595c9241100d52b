// k2b split-KV decode on the sm_100a tensor-core path (tcgen05.mma + tensor memory) for pools in
// layout 1 (row order, page = 128 tokens = one tile).
//
// One persistent CTA per SM walks an equal share of the flat tile list, as the mma.sync kernel does.
// The three contractions of a tile run as tcgen05.mma instructions issued by one warp, with their
// accumulators and two of their A operands in tensor memory; the per-element work is spread over 24
// warps in which a thread owns one token (keys, softmax) or one channel (values):
//
//   U1  K_low[128 tok x 128 ch]   = coef[128 x rank] (smem, straight from the bulk copy) x basis^T (smem),
//                                   fp16 accumulators
//   key warps (8; warp = 32 tokens x two chunks of 16 + 16 channels):
//                                   K = K_low + scale * residual   (nibble -> half2 by LOP3 + exact fix-up),
//                                   rotated by the token's offset inside the tile (its cos/sin stay in
//                                   registers), written back into the same TMEM columns as the A operand of U2
//   U2  S[128 tok x 16]            = K_rot (TMEM) x q_rot^T (smem; the tile's base rotation is applied to q)
//   softmax warps (two sets of 4; set e takes the tiles of parity e and owns that parity's running
//                                   (max, sum) and output accumulator): online softmax in base 2 with a lazy
//                                   rescale; p * norm -> smem (B of U3)
//   value warps (8; thread = channel, warp = 64 tokens): 2-bit codes -> fp16 levels by byte-permute lookups
//                                   -> TMEM (A of U3)
//   U3  O_e^T[128 ch x 16]        += V_lev^T (TMEM) x P (smem), fp32
//
// The K, S, V and P buffers are double-buffered by tile parity, so the key warps start tile n+1 while U2
// and the softmax of tile n are still under way.  Service warps: one thread issues the bulk copies, two
// warps rotate q (and lay out the basis operand when the head changes), one warp issues every
// tcgen05.mma.  That warp shares its scheduler with compute warps, so what it executes between "operand
// complete" and "MMA issued" is kept minimal: the compute warps arrive on plain counters in shared memory,
// which it reads with independent loads (an mbarrier test costs ~70 cycles and tests do not overlap), and
// per-tile facts it would have to derive (basis buffer, first tile of a range) are left for it in shared
// memory by the rotation warps.  The two parities end as two partial records per (CTA, range).
#include "decode_common.cuh"
#include "tc5.cuh"

namespace bmxk {

namespace {

constexpr int T5_THREADS = 896;   // warps 0-7 key, 8-15 softmax (two sets), 16-23 value (two halves), 24 copy, 25 issue, 26-27 query rotation
constexpr int T5_STAGES = 7;
// Registers per thread after each role resizes itself.  setmaxnreg.inc blocks (without a time limit) until the
// CTA's pool has room, and the pool is what the launch handed out: 72 registers x 896 threads = 28 warps x 72.
constexpr int REG_LAUNCH = 72, REG_KEY = 112, REG_SOFTMAX = 56, REG_VALUE = 56, REG_SERVICE = 56;
static_assert(8 * REG_KEY + 8 * REG_SOFTMAX + 8 * REG_VALUE + 4 * REG_SERVICE <= 28 * REG_LAUNCH, "register split exceeds the CTA's pool");
constexpr int T5_QB_BYTES = 4096;  // B operand of U2 / U3: 16 rows x 128 fp16, K-major core matrices
// TMEM columns: K_low / K_rot of buffer b at 128*b; value levels at 256 + 64*b; scores at 384 + 16*b; output of tile parity e at 416 + 16*e
constexpr uint32_t TM_KD = 0, TM_V = 256, TM_S = 384, TM_O = 416, TM_COLS = 512;

struct T5Smem {
  uint64_t full[T5_STAGES], empty[T5_STAGES];
  uint64_t low[2], sdone[2], odone[2];   // completion of U1 / U2 / U3 on buffer b (tcgen05.commit)
  uint32_t tmem_base;
  volatile int released;   // tiles whose stage has been handed back
  int bcnt, ccnt;                          // U2 / U3 issued so far, each written by its issuing warp for the other
  int kcnt[2], pcnt[2], vcnt[2];           // arrivals of key (8 per tile) / softmax (4) / value (4) warps on buffer b, never reset
  volatile int slot_ring[16];              // page slot of tile n at n % 16, fetched by the rotation warps ahead of the copy
  int slot_seq[2];                         // rotation warp r has published the slots of its tiles below this index
  volatile int bsel[T5_STAGES], first[T5_STAGES];  // per stage: basis buffer of the tile, and whether it starts a range
  float wmax[2][4][8];
  __align__(16) int flag[2][4];
  float red[2][4][16];
};

// Walks the CTA's tile range; `seg` counts the (sequence, head) ranges met so far.
struct Walker {
  TileCursor cur;
  int it, seg, bh;
  __device__ __forceinline__ void init(const int* cum, const int* npg, int f_begin, int h_kv) {
    cur.init(cum, npg, f_begin, 128);
    it = 0, seg = 0, bh = cur.b * h_kv + cur.h;
  }
  __device__ __forceinline__ void advance(const int* npg, int h_kv, int batch) {
    cur.next(npg, h_kv, 128, batch);
    ++it;
    const int nb = cur.b * h_kv + cur.h;
    if (nb != bh) bh = nb, ++seg;
  }
};

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred P;\n elect.sync _|P, 0xffffffff;\n selp.u32 %0, 1, 0, P;\n}\n" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void named_bar(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

}  // namespace

template <int RANK, int GQ>
__global__ void __launch_bounds__(T5_THREADS, 1) k2b_decode_t5_kernel(const K2bDecodeParams p) {
  constexpr int KS = RANK / 16;
  constexpr int COEF_BYTES = 128 * RANK * 2;
  constexpr uint32_t AB_SBO = RANK * 16;  // bytes between 8-row groups of the coef / basis operands
  extern __shared__ __align__(128) uint8_t smem[];
  const K2bGeom g = p.g;
  const int G = g.n_q_groups;
  const int PB = k2b_page_block_bytes(128, g.group);
  const int STAGE_BYTES = COEF_BYTES + PB;

  uint8_t* stage0 = smem;
  uint8_t* qb0 = stage0 + T5_STAGES * STAGE_BYTES;       // [stage][4096] rotated queries
  uint8_t* bbuf0 = qb0 + T5_STAGES * T5_QB_BYTES;        // [2][COEF_BYTES] basis operand per range parity
  uint8_t* pbuf0 = bbuf0 + 2 * COEF_BYTES;               // [2][4096] softmax weights per tile parity
  T5Smem* sh = reinterpret_cast<T5Smem*>(pbuf0 + 2 * T5_QB_BYTES);
  int* cum = reinterpret_cast<int*>(sh + 1);
  int* npg_sm = cum + p.batch + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // the merge kernel is launched as this kernel's programmatic dependent: let its blocks become resident as soon as
  // SMs free up (it waits for this grid's completion itself before it reads the partial states)
  asm volatile("griddepcontrol.launch_dependents;");
  if (warp == 0) fill_cum(cum, p.n_pages, p.batch, g.h_kv, 128, lane);
  for (int i = tid; i < p.batch; i += T5_THREADS) npg_sm[i] = p.n_pages[i];
  __syncthreads();
  const int total = cum[p.batch];
  const int per_cta = (total + gridDim.x - 1) / gridDim.x;
  const int f_begin = min(total, (int)blockIdx.x * per_cta);
  const int f_end = min(total, f_begin + per_cta);
  const int n_tiles = f_end - f_begin;
  if (n_tiles <= 0) return;

  // ---- prologue: zeroed operand rows, barriers, tensor memory ----
  for (int i = tid; i < (T5_STAGES + 2) * T5_QB_BYTES / 16; i += T5_THREADS) {
    uint8_t* base = (i < T5_STAGES * T5_QB_BYTES / 16) ? qb0 + (size_t)i * 16 : pbuf0 + ((size_t)i - T5_STAGES * T5_QB_BYTES / 16) * 16;
    *reinterpret_cast<uint4*>(base) = make_uint4(0u, 0u, 0u, 0u);
  }
  if (tid == 0) {
    for (int s = 0; s < T5_STAGES; ++s) mbar_init(&sh->full[s], 2), mbar_init(&sh->empty[s], 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->low[b], 1), mbar_init(&sh->sdone[b], 1), mbar_init(&sh->odone[b], 1);
    }
    sh->released = 0, sh->bcnt = 0, sh->ccnt = 0, sh->slot_seq[0] = sh->slot_seq[1] = 0;
    for (int b = 0; b < 2; ++b) sh->kcnt[b] = sh->pcnt[b] = sh->vcnt[b] = 0;
    fence_barrier_init();
  }
  if (warp == 25) {
    tc5::alloc(smem_u32(&sh->tmem_base), TM_COLS);
    tc5::relinquish();
  }
  fence_proxy_async();
  tc5::fence_before();
  __syncthreads();
  tc5::fence_after();
  const uint32_t tmem = sh->tmem_base;

  Walker w;
  w.init(cum, npg_sm, f_begin, g.h_kv);

  // Registers move from the softmax, value and service warps to the key warps: each group of four warps
  // resizes itself first thing in its branch.
  if (warp < 8) {
    // ===================== key warps: 32 token rows x two chunks of 16 + 16 channels =====================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REG_KEY));
    const int wq = warp & 3, k0 = 2 * (warp >> 2), row = 32 * wq + lane;
    const uint32_t tk = tmem + TM_KD + ((uint32_t)(32 * wq) << 16);
    const int grp = row / g.group;
    const __half2 c1032 = __floats2half2_rn(1032.f, 1032.f);
    const __half2 c16th = __floats2half2_rn(0.0625f, 0.0625f);
    const __half2 cm72 = __floats2half2_rn(-72.f, -72.f);
    // rotation by this token's offset inside the tile, for rotary pairs 16k .. 16k+15 of both chunks
    uint32_t cs_[2][8], sn_[2][8];
#pragma unroll
    for (int kk = 0; kk < 2; ++kk)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        cs_[kk][i] = *reinterpret_cast<const uint32_t*>(p.rope_cos + (int64_t)row * HEAD_DIM + 16 * (k0 + kk) + 2 * i);
        sn_[kk][i] = *reinterpret_cast<const uint32_t*>(p.rope_sin + (int64_t)row * HEAD_DIM + 16 * (k0 + kk) + 2 * i);
      }
    int s = 0;
    uint32_t fp = 0;
    for (int n = 0; n < n_tiles; ++n) {
      const int b = n & 1;
      const uint32_t par = (uint32_t)(n >> 1) & 1u;
      const uint8_t* blk = stage0 + (size_t)s * STAGE_BYTES + COEF_BYTES;
      if (!wait_or_flag(&sh->full[s], fp, p.status, 2)) break;
      if (!wait_or_flag(&sh->low[b], par, p.status, 6)) break;
      tc5::fence_after();
      uint32_t dl[2][8], dh[2][8];
      // a warp's TMEM loads complete one after the other, so the second chunk's are issued only after the first
      // chunk's have landed and travel while the first chunk is computed
      tc5::ld16_pack(tk + 128 * b + 16 * k0, dl[0]);
      tc5::ld16_pack(tk + 128 * b + 64 + 16 * k0, dh[0]);
      const uint4* ksc4 = reinterpret_cast<const uint4*>(blk + k2b_off_kscale(128)) + grp * 16;
#pragma unroll
      for (int kk = 0; kk < 2; ++kk) {
        const int k = k0 + kk;
        uint32_t out[16];
        const uint4 cw = reinterpret_cast<const uint4*>(blk)[k * 128 + row];
        const uint4 scl[2] = {ksc4[2 * k], ksc4[2 * k + 1]}, sch[2] = {ksc4[8 + 2 * k], ksc4[9 + 2 * k]};
        tc5::wait_ld();
        if (kk == 0) {
          tc5::ld16_pack(tk + 128 * b + 16 * k0 + 16, dl[1]);
          tc5::ld16_pack(tk + 128 * b + 64 + 16 * k0 + 16, dh[1]);
        }
#pragma unroll
        for (int wd = 0; wd < 2; ++wd) {
          const uint32_t wlo = wd ? cw.y : cw.x, whi = wd ? cw.w : cw.z;
          const uint32_t sl[4] = {scl[wd].x, scl[wd].y, scl[wd].z, scl[wd].w}, sh_[4] = {sch[wd].x, sch[wd].y, sch[wd].z, sch[wd].w};
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
            const __half2 c = u32_as_h2(cs_[kk][4 * wd + i]), sn = u32_as_h2(sn_[kk][4 * wd + i]);
            out[4 * wd + i] = h2_as_u32(__hfma2(__hneg2(sn), khi, __hmul2(klo, c)));
            out[8 + 4 * wd + i] = h2_as_u32(__hfma2(sn, klo, __hmul2(khi, c)));
          }
        }
        tc5::st16(tk + 128 * b + 16 * k, out);
      }
      tc5::wait_st();
      tc5::fence_before();
      __syncwarp();
      if (lane == 0) smem_add_release(&sh->kcnt[b], 1);
      if (++s == T5_STAGES) s = 0, fp ^= 1u;
    }
  } else if (warp >= 16 && warp < 24) {
    // ===================== value warps: thread = channel, warp = one half (64 tokens) of the tile =====================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REG_VALUE));
    const int wq = warp & 3, cc = (warp - 16) >> 2, ch = 32 * wq + lane;
    const uint32_t tv = tmem + TM_V + ((uint32_t)(32 * wq) << 16);
    int s = 0;
    uint32_t fp = 0;
    for (int n = 0; n < n_tiles; ++n) {
      const int b = n & 1;
      if (!wait_or_flag(&sh->full[s], fp, p.status, 10)) break;
      // the columns still feed U3 of tile n-2
      if (n >= 2 && !wait_or_flag(&sh->odone[b], (uint32_t)((n - 2) >> 1) & 1u, p.status, 11)) break;
      tc5::fence_after();
      const uint4* vc = reinterpret_cast<const uint4*>(stage0 + (size_t)s * STAGE_BYTES + COEF_BYTES + k2b_off_vcode(128, g.group));
      {
        const uint4 cw = vc[cc * 128 + ch];
        const uint32_t wd[4] = {cw.x, cw.y, cw.z, cw.w};
#pragma unroll
        for (int jp = 0; jp < 2; ++jp) {
          uint32_t out[16];
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const uint32_t wv = wd[2 * jp + jj];
            const uint32_t x0 = wv & 0x33333333u, x1 = (wv >> 2) & 0x33333333u;
#pragma unroll
            for (int hs = 0; hs < 2; ++hs) {
              const uint32_t s0 = hs ? (x0 >> 16) : x0, s1 = hs ? (x1 >> 16) : x1;
              const uint32_t lo0 = prmt(p.lut_lo, 0u, s0), hi0 = prmt(p.lut_hi, 0u, s0);
              const uint32_t lo1 = prmt(p.lut_lo, 0u, s1), hi1 = prmt(p.lut_hi, 0u, s1);
              out[8 * jj + 2 * hs] = prmt(lo0, hi0, 0x5140u), out[8 * jj + 2 * hs + 1] = prmt(lo0, hi0, 0x7362u);
              out[8 * jj + 4 + 2 * hs] = prmt(lo1, hi1, 0x5140u), out[8 * jj + 4 + 2 * hs + 1] = prmt(lo1, hi1, 0x7362u);
            }
          }
          tc5::st16(tv + 64 * b + 32 * cc + 16 * jp, out);
        }
      }
      tc5::wait_st();
      tc5::fence_before();
      __syncwarp();
      if (lane == 0) smem_add_release(&sh->vcnt[b], 1);
      if (++s == T5_STAGES) s = 0, fp ^= 1u;
    }
  } else if (warp < 16) {
    // ===================== softmax warps: thread = token row =====================
    // Two sets of four warps; set e takes the tiles of parity e and owns the running (max, sum) and the output
    // accumulator of that parity, so each set has two tile periods per tile.  Each set writes its own partial
    // record per (sequence, head) range.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REG_SOFTMAX));
    const int e = (warp - 8) >> 2, wq = warp & 3, row = 32 * wq + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * wq) << 16);
    float m[GQ], l[GQ], pn[GQ];
#pragma unroll
    for (int qi = 0; qi < GQ; ++qi) m[qi] = -INFINITY, l[qi] = 0.f, pn[qi] = 0.f;
    int cur_seg = -1, cur_b = 0, cur_h = 0, last_n = -1;
    bool had = false, alive = true;
    const int64_t sub_slots = (int64_t)gridDim.x + (int64_t)p.batch * g.h_kv;

    // Writes this set's partial record of the range that just ended (an empty one if the set had no tile in it).
    auto flush = [&](int b_, int h_) {
      float acc[GQ];
#pragma unroll
      for (int qi = 0; qi < GQ; ++qi) acc[qi] = 0.f;
      if (had && alive && !wait_or_flag(&sh->odone[e], (uint32_t)(last_n >> 1) & 1u, p.status, 9)) alive = false;
      if (had && alive) {
        tc5::fence_after();
        uint32_t r[GQ];
        if constexpr (GQ == 4) tc5::ld4(tl + TM_O + 16 * e, r); else tc5::ld8(tl + TM_O + 16 * e, r);
        tc5::wait_ld();
#pragma unroll
        for (int qi = 0; qi < GQ; ++qi) acc[qi] = __uint_as_float(r[qi]);
        tc5::fence_before();
      }
#pragma unroll
      for (int qi = 0; qi < GQ; ++qi) {
        float a = l[qi], b2 = pn[qi];
#pragma unroll
        for (int mk = 16; mk >= 1; mk >>= 1) a += __shfl_xor_sync(0xffffffffu, a, mk), b2 += __shfl_xor_sync(0xffffffffu, b2, mk);
        if (lane == 0) sh->red[e][wq][qi] = a, sh->red[e][wq][GQ + qi] = b2;
      }
      named_bar(1 + e, 128);
      float* dst = p.part + ((e * sub_slots + blockIdx.x + (int64_t)b_ * g.h_kv + h_) * G) * PART_STRIDE;
#pragma unroll
      for (int qi = 0; qi < GQ; ++qi)
        if (qi < G) {
          const float L = sh->red[e][0][qi] + sh->red[e][1][qi] + sh->red[e][2][qi] + sh->red[e][3][qi];
          const float P = sh->red[e][0][GQ + qi] + sh->red[e][1][GQ + qi] + sh->red[e][2][GQ + qi] + sh->red[e][3][GQ + qi];
          dst[qi * PART_STRIDE + 2 + row] = had ? p.lut_alpha * P + p.lut_beta * acc[qi] : 0.f;
          if (row == 0) dst[qi * PART_STRIDE] = had ? m[qi] : -INFINITY, dst[qi * PART_STRIDE + 1] = had ? L : 0.f;
        }
      named_bar(1 + e, 128);
    };

    for (; w.it < n_tiles; w.advance(npg_sm, g.h_kv, p.batch)) {
      const int n = w.it;
      if (w.seg != cur_seg) {
        if (cur_seg >= 0) flush(cur_b, cur_h);
        cur_seg = w.seg, cur_b = w.cur.b, cur_h = w.cur.h, had = false;
#pragma unroll
        for (int qi = 0; qi < GQ; ++qi) m[qi] = -INFINITY, l[qi] = 0.f, pn[qi] = 0.f;
      }
      if ((n & 1) != e) continue;
      const int s = n % T5_STAGES;
      const uint32_t fp = (uint32_t)(n / T5_STAGES) & 1u, par = (uint32_t)(n >> 1) & 1u;
      const uint8_t* blk = stage0 + (size_t)s * STAGE_BYTES + COEF_BYTES;
      float sv[GQ];
#pragma unroll
      for (int qi = 0; qi < GQ; ++qi) sv[qi] = -INFINITY;
      if (alive && !wait_or_flag(&sh->full[s], fp, p.status, 12)) alive = false;
      if (alive && !wait_or_flag(&sh->sdone[e], par, p.status, 7)) alive = false;
      if (alive) {
        tc5::fence_after();
        uint32_t r[GQ];
        if constexpr (GQ == 4) tc5::ld4(tl + TM_S + 16 * e, r); else tc5::ld8(tl + TM_S + 16 * e, r);
        tc5::wait_ld();
#pragma unroll
        for (int qi = 0; qi < GQ; ++qi) sv[qi] = __uint_as_float(r[qi]);
      }
      // Lazy maximum: as long as no score of the tile exceeds the running maximum by more than 8 (weights
      // below 2^8), nothing is reduced; the four warps only exchange one flag each.
      bool need = false;
#pragma unroll
      for (int qi = 0; qi < GQ; ++qi) need |= (qi < G) && (sv[qi] > m[qi] + 8.f);
      const bool wneed = __any_sync(0xffffffffu, need);
      if (lane == 0) sh->flag[e][wq] = wneed ? 1 : 0;
      named_bar(1 + e, 128);
      const int4 fl = *reinterpret_cast<const int4*>(sh->flag[e]);
      const bool resc = (fl.x | fl.y | fl.z | fl.w) != 0;
      // the weight buffer and the accumulator of this parity still belong to U3 of tile n-2
      if (alive && n >= 2 && !wait_or_flag(&sh->odone[e], (uint32_t)((n - 2) >> 1) & 1u, p.status, 8)) alive = false;
      if (resc) {
        float mnew[GQ];
#pragma unroll
        for (int qi = 0; qi < GQ; ++qi) {
          float v = sv[qi];
#pragma unroll
          for (int mk = 16; mk >= 1; mk >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, mk));
          if (lane == 0) sh->wmax[e][wq][qi] = v;
        }
        named_bar(1 + e, 128);
#pragma unroll
        for (int qi = 0; qi < GQ; ++qi) {
          const float tm = fmaxf(fmaxf(sh->wmax[e][0][qi], sh->wmax[e][1][qi]), fmaxf(sh->wmax[e][2][qi], sh->wmax[e][3][qi]));
          mnew[qi] = (qi < G && tm > m[qi] + 8.f) ? tm : m[qi];
        }
        named_bar(1 + e, 128);  // the flags and maxima may be rewritten by the next tile only after everyone has read them
        if (alive) {
          float f[GQ];
#pragma unroll
          for (int qi = 0; qi < GQ; ++qi) {
            f[qi] = (m[qi] == -INFINITY) ? 0.f : ex2_approx(m[qi] - mnew[qi]);
            l[qi] *= f[qi], pn[qi] *= f[qi], m[qi] = mnew[qi];
          }
          if (had) {  // this thread's TMEM lane is channel `row` of the accumulator
            tc5::fence_after();
            uint32_t r[GQ];
            if constexpr (GQ == 4) tc5::ld4(tl + TM_O + 16 * e, r); else tc5::ld8(tl + TM_O + 16 * e, r);
            tc5::wait_ld();
#pragma unroll
            for (int qi = 0; qi < GQ; ++qi) r[qi] = __float_as_uint(__uint_as_float(r[qi]) * f[qi]);
            if constexpr (GQ == 4) tc5::st4(tl + TM_O + 16 * e, r); else tc5::st8(tl + TM_O + 16 * e, r);
            tc5::wait_st();
          }
        }
      }
      if (alive) {
        const float norm = __half2float(reinterpret_cast<const __half*>(blk + k2b_off_vnorm(128, g.group))[row]);
        __half* pb = reinterpret_cast<__half*>(pbuf0 + (size_t)e * T5_QB_BYTES) + (row >> 3) * 64 + (row & 7);
#pragma unroll
        for (int qi = 0; qi < GQ; qi += 2) {
          const float p0 = ex2_approx(sv[qi] - m[qi]), p1 = ex2_approx(sv[qi + 1] - m[qi + 1]);
          const __half2 hw = __floats2half2_rn(p0 * norm, p1 * norm);
          if (qi < G) l[qi] += p0, pn[qi] += __low2float(hw), pb[qi * 8] = __low2half(hw);
          if (qi + 1 < G) l[qi + 1] += p1, pn[qi + 1] += __high2float(hw), pb[(qi + 1) * 8] = __high2half(hw);
        }
        fence_proxy_async();
        tc5::fence_before();
        __syncwarp();
        if (lane == 0) smem_add_release(&sh->pcnt[e], 1);
      }
      had = true, last_n = n;
    }
    flush(cur_b, cur_h);
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REG_SERVICE));  // the four service warps, as one group
    if (warp == 24) {
      // ===================== copy + U3 warp =====================
      // Two jobs polled in turn: (1) the bulk copies of the next tile as soon as its stage is free (the page's
      // slot index comes from the rotation warps through shared memory); (2) C(n): once the softmax weights and the value levels of tile n
      // are in place, U3 -> odone[n & 1], and the stage is handed back.  U3 is issued here and not by the U1 / U2
      // warp because three issues per tile are more than one warp gets through in a tile period.
      constexpr uint32_t ID_N16 = tc5::idesc_f16_f32(128, 16);
      const bool el = elect_one();
      const uint64_t d_pb = tc5::smem_desc(smem_u32(pbuf0), 128, 2048);
      // Stage indices, barrier phases and arrival thresholds are carried from action to action (no division in the
      // polling loop): what runs between "operands complete" and "MMA issued" is what a tile waits for.
      int nC = 0, nP = 0, sC = 0, sP = 0, need_p = 4, need_v = 8;   // arrivals that complete tile nC on its parity's counters
      uint32_t phP = 1;                                             // parity to test on empty[sP]: a fresh barrier passes 1
      long long t_last = clock64();
      uint32_t idle = 0;
      bool ok = true;
      while (ok && nC < n_tiles) {
        bool progressed = false;
        const int pc = smem_load_acquire(&sh->pcnt[nC & 1]);
        const int vc = smem_load_acquire(&sh->vcnt[nC & 1]);
        const int bdone = smem_load_acquire(&sh->bcnt);
        if (nC < bdone && pc >= need_p && vc >= need_v) {
          tc5::fence_after();
          const int s = sC, b = nC & 1;
          const uint32_t keep = sh->first[s] ? 0u : 1u;  // the first tile of its parity in a range starts a new accumulator
          const uint64_t db = d_pb + (uint64_t)(b * (T5_QB_BYTES >> 4));
          ++nC;
          if (b) need_p += 4, need_v += 8;  // the next tile of parity 0 needs one more round of arrivals
          if (++sC == T5_STAGES) sC = 0;
          if (el) {
            tc5::mma_ts(tmem + TM_O + 16 * b, tmem + TM_V + 64 * b, db, ID_N16, keep);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks) tc5::mma_ts(tmem + TM_O + 16 * b, tmem + TM_V + 64 * b + 8 * ks, db + 16 * ks, ID_N16, 1u);
            tc5::commit(smem_u32(&sh->odone[b]));
            mbar_arrive(&sh->empty[s]);
            smem_add_release(&sh->ccnt, 1);
            sh->released = nC;
          }
          __syncwarp();
          progressed = true;
        }
        if (nP < n_tiles && smem_load_acquire(&sh->slot_seq[nP & 1]) > nP && mbar_test_wait(&sh->empty[sP], phP)) {
          const int s = sP, h = w.cur.h, slot = sh->slot_ring[nP & 15];
          uint8_t* st = stage0 + (size_t)s * STAGE_BYTES;
          const int chd = (g.n_coef_heads == 1) ? 0 : h;
          if (el) {
            mbar_arrive_expect_tx(&sh->full[s], (uint32_t)(COEF_BYTES + PB));
            bulk_g2s(st, reinterpret_cast<const uint8_t*>(p.coefs) + ((int64_t)slot * g.n_coef_heads + chd) * COEF_BYTES, COEF_BYTES,
                     &sh->full[s]);
            bulk_g2s(st + COEF_BYTES, p.pages + ((int64_t)slot * g.h_kv + h) * PB, PB, &sh->full[s]);
          }
          __syncwarp();
          ++nP;
          if (++sP == T5_STAGES) sP = 0, phP ^= 1u;
          if (nP < n_tiles) w.advance(npg_sm, g.h_kv, p.batch);
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if ((++idle & 255u) == 0u) {
          if (idle == 256u) t_last = clock64();
          if (clock64() - t_last > 4000000000LL || *reinterpret_cast<volatile int32_t*>(p.status) != 0) {
            if (el && atomicCAS(p.status, 0, 1) == 0) p.status[1] = blockIdx.x, p.status[2] = 1;
            ok = false;
          }
        }
      }
    } else if (warp >= 26) {
      // ===================== query rotation warps: tiles of parity rw =====================
      // q_rot = R(-t0) q * scale, written as the B operand of U2 in the K order the key warps produce:
      // position 32k + e holds channel 16k + e (e < 16) or 64 + 16k + (e - 16).  The warp that meets the
      // first tile of a (sequence, head) range also lays out that head's basis as the B operand of U1.
      const int rw = warp - 26;
      int s = 0;
      uint32_t ph = 1;
      int prev_seg = -1, first_cur = 0, first_prev = 0;  // first tile of the current / previous range
      bool alive = true;
      for (; w.it < n_tiles && alive; w.advance(npg_sm, g.h_kv, p.batch)) {
        const bool new_seg = (w.seg != prev_seg);
        if (new_seg) first_prev = first_cur, first_cur = w.it, prev_seg = w.seg;
        if ((w.it & 1) == rw) {
          const int b = w.cur.b, h = w.cur.h, j = w.cur.j;
          const int64_t t0 = p.pos_offset + (int64_t)j * TILE_TOKENS;
          const __half* qsrc = p.q + ((int64_t)b * g.h_kv + h) * G * HEAD_DIM;
          // the page-table entry of this tile, for the copy warp: a global load there would sit in front of every
          // release it does, so it is fetched here, where loads are prefetched anyway
          const int slot = p.page_table[(int64_t)b * p.table_stride + j];
          float cs[2], sn[2], x1[2][GQ], x2[2][GQ];
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const int c = lane + 32 * jj;  // rotary pair (c, c + 64)
            cs[jj] = __half2float(p.rope_cos[t0 * HEAD_DIM + c]);
            sn[jj] = __half2float(p.rope_sin[t0 * HEAD_DIM + c]);
#pragma unroll
            for (int qi = 0; qi < GQ; ++qi) {
              x1[jj][qi] = (qi < G) ? __half2float(qsrc[qi * HEAD_DIM + c]) : 0.f;
              x2[jj][qi] = (qi < G) ? __half2float(qsrc[qi * HEAD_DIM + c + 64]) : 0.f;
            }
          }
          if (lane == 0) {
            sh->slot_ring[w.it & 15] = slot;
            asm volatile("st.release.cta.shared::cta.u32 [%0], %1;" ::"r"(smem_u32(&sh->slot_seq[rw])), "r"(w.it + 1) : "memory");
          }
          if (!wait_or_flag(&sh->empty[s], ph, p.status, 3)) { alive = false; break; }
          __half* qr = reinterpret_cast<__half*>(qb0 + (size_t)s * T5_QB_BYTES);
#pragma unroll
          for (int jj = 0; jj < 2; ++jj) {
            const int c = lane + 32 * jj;
            const int k1 = 32 * (c >> 4) + (c & 15), k2 = k1 + 16;
#pragma unroll
            for (int qi = 0; qi < GQ; ++qi)
              if (qi < G) {
                const float a = x1[jj][qi] * p.scale_log2, bb = x2[jj][qi] * p.scale_log2;
                qr[(k1 >> 3) * 64 + qi * 8 + (k1 & 7)] = __float2half_rn(a * cs[jj] + bb * sn[jj]);
                qr[(k2 >> 3) * 64 + qi * 8 + (k2 & 7)] = __float2half_rn(bb * cs[jj] - a * sn[jj]);
              }
          }
          if (new_seg) {
            if (w.seg >= 2) {
              // the buffer still serves the range before the previous one until all its tiles are handed back
              const long long c0 = clock64();
              while (sh->released < first_prev) {
                if (clock64() - c0 > 4000000000LL || *reinterpret_cast<volatile int32_t*>(p.status) != 0) {
                  if (atomicCAS(p.status, 0, 1) == 0) p.status[1] = blockIdx.x, p.status[2] = 4;
                  alive = false;
                  break;
                }
              }
              if (!alive) break;
            }
            uint4* bd = reinterpret_cast<uint4*>(bbuf0 + (size_t)(w.seg & 1) * COEF_BYTES);
            const uint4* bs = reinterpret_cast<const uint4*>(p.basis16 + (int64_t)h * HEAD_DIM * RANK);
            for (int o = lane; o < 128 * (RANK / 8); o += 32) {
              const int c = o / (RANK / 8), i8 = o % (RANK / 8);
              bd[((c >> 3) * (RANK / 8) + i8) * 8 + (c & 7)] = bs[o];
            }
          }
          if (lane == 0) sh->bsel[s] = w.seg & 1, sh->first[s] = (w.it - first_cur < 2) ? 1 : 0;
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh->full[s]);
        }
        if (++s == T5_STAGES) s = 0, ph ^= 1;
      }
    } else {
      // ===================== issuing warp =====================
      // Tile n (buffer b = n & 1) goes through  A: U1 -> low[b];  B: U2 -> sdone[b];  C: U3 -> odone[b], after
      // which its stage is handed back.  A(n) needs the tile's copy landed (tiles are taken in order, so the
      // basis operand, which travels with the first tile of its range, has landed too) and U2(n-2) done (same
      // TMEM columns); B(n) needs the rotated keys of all key warps and the softmax of tile n-2 finished with
      // the score columns; C(n) needs the weights and the value levels.  The whole warp walks this state machine
      // in lockstep, so that operand descriptors stay in uniform registers; one elected lane issues.
      constexpr uint32_t ID_U1 = tc5::idesc_f16_f16(128, 128), ID_N16 = tc5::idesc_f16_f32(128, 16);
      const bool el = elect_one();
      int nA = 0, nB = 0, sA = 0, sB = 0, need_k = 8;   // key-warp arrivals that complete tile nB on its parity's counter
      uint32_t phA = 0;                                 // parity to test on full[sA]
      const uint64_t d_stage = tc5::smem_desc(smem_u32(stage0), 128, AB_SBO), d_bbuf = tc5::smem_desc(smem_u32(bbuf0), 128, AB_SBO);
      const uint64_t d_qb = tc5::smem_desc(smem_u32(qb0), 128, 2048), d_pb = tc5::smem_desc(smem_u32(pbuf0), 128, 2048);
      long long t_last = clock64();
      uint32_t idle = 0;
      bool ok = true;
      while (ok && nB < n_tiles) {
        bool progressed = false;
        // the software counters are read together (independent loads), the two hardware barriers only
        // when U1 could otherwise go
        const int kc = smem_load_acquire(&sh->kcnt[nB & 1]);
        const int nC = smem_load_acquire(&sh->ccnt);   // U3 issued so far (the other issuing warp)
        // ---- B ----
        if (nB < nA && nB < nC + 2 && kc >= need_k) {
          tc5::fence_after();
          const int s = sB, b = nB & 1;
          const uint64_t db = d_qb + (uint64_t)(s * (T5_QB_BYTES >> 4));
          if (el) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) tc5::mma_ts(tmem + TM_S + 16 * b, tmem + TM_KD + 128 * b + 8 * ks, db + 16 * ks, ID_N16, ks > 0);
            tc5::commit(smem_u32(&sh->sdone[b]));
            smem_add_release(&sh->bcnt, 1);
          }
          __syncwarp();
          ++nB;
          if (b) need_k += 8;
          if (++sB == T5_STAGES) sB = 0;
          progressed = true;
        }
        // ---- A ----
        if (nA < n_tiles && nA < nB + 2 && mbar_test_wait(&sh->full[sA], phA) &&
            (nA < 2 || mbar_test_wait(&sh->sdone[nA & 1], (uint32_t)((nA - 2) >> 1) & 1u))) {
          tc5::fence_after();
          const int s = sA, b = nA & 1;
          const uint64_t da = d_stage + (uint64_t)(s * (STAGE_BYTES >> 4)), db = d_bbuf + (uint64_t)(sh->bsel[s] * (COEF_BYTES >> 4));
          if (el) {
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) tc5::mma_ss(tmem + TM_KD + 128 * b, da + 16 * ks, db + 16 * ks, ID_U1, ks > 0);
            tc5::commit(smem_u32(&sh->low[b]));
          }
          __syncwarp();
          ++nA;
          if (++sA == T5_STAGES) sA = 0, phA ^= 1u;
          progressed = true;
        }
        if (progressed) {
          idle = 0;
        } else if ((++idle & 255u) == 0u) {
          if (idle == 256u) t_last = clock64();
          if (clock64() - t_last > 4000000000LL || *reinterpret_cast<volatile int32_t*>(p.status) != 0) {
            if (el && atomicCAS(p.status, 0, 1) == 0) p.status[1] = blockIdx.x, p.status[2] = 5;
            ok = false;
          }
        }
      }
    }
  }

  // ---- epilogue: every role ends here; the tensor memory goes back before the CTA leaves ----
  tc5::fence_before();
  __syncthreads();
  if (warp == 25) {
    tc5::fence_after();
    tc5::dealloc(tmem, TM_COLS);
  }
}

static size_t t5_smem_bytes(int rank, int group, int batch) {
  const size_t coef = (size_t)128 * rank * 2;
  return (size_t)T5_STAGES * (coef + k2b_page_block_bytes(128, group)) + (size_t)(T5_STAGES + 2) * T5_QB_BYTES + 2 * coef +
         sizeof(T5Smem) + (size_t)(2 * batch + 1) * 4 + 16;
}

template <int RANK, int GQ>
static int launch_t5(const K2bDecodeParams& prm, int grid, size_t smem, cudaStream_t s) {
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(k2b_decode_t5_kernel<RANK, GQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      configured.retract();
      set_error("bmxk_k2b_decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return BMXK_ERR_CUDA;
    }
  }
  k2b_decode_t5_kernel<RANK, GQ><<<grid, T5_THREADS, smem, s>>>(prm);
  return check_launch("bmxk_k2b_decode(tcgen05)");
}

int launch_decode_t5(const K2bDecodeParams& prm, int grid, cudaStream_t s) {
  const size_t smem = t5_smem_bytes(prm.g.rank, prm.g.group, prm.batch);
  BMXK_REQUIRE(smem <= 227 * 1024, "bmxk_k2b_decode: batch=%d too large for the tcgen05 kernel's shared memory", prm.batch);
  const bool g4 = prm.g.n_q_groups <= 4;
  if (prm.g.rank == 32) return g4 ? launch_t5<32, 4>(prm, grid, smem, s) : launch_t5<32, 8>(prm, grid, smem, s);
  return g4 ? launch_t5<16, 4>(prm, grid, smem, s) : launch_t5<16, 8>(prm, grid, smem, s);
}

}  // namespace bmxk
