// Split-KV decode over a K4 spectral key cache (per-head packs) with Hadamard + 2-bit Lloyd values, on the
// sm_100a tensor-core path.  bmx serves this codec pair through its chunked path: dequantize a block,
// M_hat = Y_hat @ dec^T, RoPE, attention in PyTorch (src/bmx/cache/chunked_attention.py:52-145, 478-530;
// src/bmx/cache/spectral.py:812-839).  Here the whole step is one persistent kernel plus the merge kernel.
//
// The kernel is the k2b tcgen05 kernel (k2b_decode_t5.cu) with the low-rank product replaced by the full
// decoder product and the residual replaced by a dequantization stage in front of it:
//
//   dequant warps (16; thread = one direction x the token pairs 2q, 2q+1 of every 8-token block):
//         tier codes (2-, 4- or 8-bit containers along tokens, as the append kernel wrote them) -> fp16
//         Y_hat = (code - offset) * scale -> shared memory in the K-major operand form, one stmatrix per
//         four 8 x 8 blocks.  Directions are visited in the pack's tier order (the decoder operand the host
//         passes has its columns in the same order), so a warp's eight directions almost always share a width.
//   U1    K_hat[128 tok x 128 ch] = Y_hat (smem) x dec^T (smem), eight K=16 steps, fp16 accumulators
//   key warps: rotate by the token's offset inside the tile, write back as the A operand of U2
//   U2, softmax warps, value warps, U3, partial records: as in the k2b kernel
//
// Page data per tile: the spectral block of (slot, head) from the key pool and the 4352-byte value block of
// the same slot from the value pool (value_blocks.cu), two bulk copies into one stage.
#include <cstring>

#include "decode_common.cuh"
#include "tc5.cuh"

namespace bmxk {

namespace {

// Warp roles: 0-3 key (all four chunks each), 4-7 softmax, 8-11 value (both 64-token halves each), 12-27 dequant (one
// direction octet each), 28-31 service (copy + U3, U1 + U2, two query rotation warps).  The dequantization is what a tile
// waits for, so it gets half of the CTA's warps; the other per-element roles need a quarter of a tile period each.
constexpr int KEY_WARPS = 4, SOFT_WARPS = 4, VAL_WARPS = 4, DQ_WARPS = 16;
constexpr int W_SOFT = KEY_WARPS, W_VAL = W_SOFT + SOFT_WARPS, W_DQ = W_VAL + VAL_WARPS;
constexpr int SVC0 = W_DQ + DQ_WARPS;
constexpr int S5_THREADS = (SVC0 + 4) * 32;
constexpr int S5_MAX_STAGES = 8;
// Registers per thread after each role resizes itself; the pool is what the launch handed out.
constexpr int REG_LAUNCH = 64, REG_KEY = 112, REG_SOFTMAX = 64, REG_VALUE = 56, REG_DEQUANT = 56, REG_SERVICE = 56;
static_assert(S5_THREADS == 1024 && REG_LAUNCH * S5_THREADS <= 65536, "launch registers exceed the register file");
static_assert(KEY_WARPS * REG_KEY + SOFT_WARPS * REG_SOFTMAX + VAL_WARPS * REG_VALUE + DQ_WARPS * REG_DEQUANT + 4 * REG_SERVICE <= (SVC0 + 4) * REG_LAUNCH,
              "register split exceeds the CTA's pool");
constexpr int QB_BYTES = 4096;        // B operand of U2 / U3: 16 rows x 128 fp16, K-major core matrices
constexpr int OPER_BYTES = 128 * 128 * 2;  // Y_hat / decoder operand: 128 rows x 128 fp16
constexpr int VBLOCK = 128 * 32 + 128 * 2;
constexpr uint32_t AB_SBO = 128 * 16;  // bytes between 8-row groups of the Y_hat / decoder operands
constexpr uint32_t TM_KD = 0, TM_V = 256, TM_S = 384, TM_O = 416, TM_COLS = 512;

struct S5Smem {
  uint64_t full[S5_MAX_STAGES], empty[S5_MAX_STAGES];
  uint64_t low[2], sdone[2], odone[2];
  uint32_t tmem_base;
  volatile int released;
  int bcnt, ccnt;
  int kcnt[2], pcnt[2], vcnt[2], ycnt[2];  // arrivals of key (8 per tile) / softmax (4) / value (4) / dequant (DQ_WARPS) warps on buffer b, never reset
  volatile int slot_ring[16];
  int slot_seq[2];
  volatile int bsel[S5_MAX_STAGES], first[S5_MAX_STAGES], ksteps[S5_MAX_STAGES];  // per stage: decoder buffer, range start, K=16 steps of U1
  volatile int head[S5_MAX_STAGES];                                               // per stage: KV head of the tile (for the dequant warps)
  float wmax[2][4][8];
  __align__(16) int flag[2][4];
  float red[2][4][16];
};

struct SpectralDecodeParams {
  int h_kv, n_q_groups, group, kblock_bytes, scale_off, n_stages;
  const __half* q;
  const uint8_t* kpages;   // [slot][head][kblock_bytes]
  const uint8_t* vpages;   // [slot][head][VBLOCK]
  const __half* dec16;     // [head][channel][position in tier order]
  const int32_t* meta;     // [head][position]: row offset | direction << 16 | bits << 24; word 0 of a head also carries (K steps - 1) << 28
  const int32_t* page_table;
  int table_stride;
  const int32_t* n_pages;
  int batch;
  const __half* rope_cos;
  const __half* rope_sin;
  int64_t pos_offset;
  uint32_t lut_lo, lut_hi;
  float lut_alpha, lut_beta;
  float scale_log2;
  float* part;
  int32_t* status;
};

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
// Four 8 x 8 fp16 blocks, each stored transposed: a thread passes (column lane / 4; rows 2 (lane % 4), + 1) of
// block m in r[m]; lane l supplies the address of row l % 8 of block l / 8.
__device__ __forceinline__ void stmatrix_x4_trans(uint32_t addr, const uint32_t (&r)[4]) {
  // no memory clobber: nothing the compiler can see reads these bytes, and the loads of the next pieces should
  // be free to move above it; the fence + release that publish the buffer carry the clobber
  asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]));
}

// Resizes the calling warpgroup's registers to N: the instruction is .inc above the launch count, .dec below it and
// left out when N is the launch count (an .inc to a smaller count is an illegal instruction).
template <int N>
__device__ __forceinline__ void set_regs() {
  if constexpr (N > REG_LAUNCH) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
  else if constexpr (N < REG_LAUNCH) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

}  // namespace

template <int GQ>
__global__ void __launch_bounds__(S5_THREADS, 1) spectral_decode_t5_kernel(const SpectralDecodeParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int G = p.n_q_groups, h_kv = p.h_kv;
  const int KB = p.kblock_bytes;
  const int STAGE_BYTES = KB + VBLOCK;
  const int STG = p.n_stages;

  uint8_t* ybuf0 = smem;                           // [2][OPER_BYTES] Y_hat per tile parity
  uint8_t* bbuf0 = ybuf0 + 2 * OPER_BYTES;         // [2][OPER_BYTES] decoder operand per range parity
  uint8_t* pbuf0 = bbuf0 + 2 * OPER_BYTES;         // [2][QB_BYTES] softmax weights per tile parity
  uint8_t* qb0 = pbuf0 + 2 * QB_BYTES;             // [STG][QB_BYTES] rotated queries
  uint8_t* stage0 = qb0 + (size_t)STG * QB_BYTES;  // [STG][key block | value block]
  S5Smem* sh = reinterpret_cast<S5Smem*>(stage0 + (size_t)STG * STAGE_BYTES);
  int* cum = reinterpret_cast<int*>(sh + 1);
  int* npg_sm = cum + p.batch + 1;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // the merge kernel is launched as this kernel's programmatic dependent (see launch_merge)
  asm volatile("griddepcontrol.launch_dependents;");
  if (warp == 0) fill_cum(cum, p.n_pages, p.batch, h_kv, 128, lane);
  for (int i = tid; i < p.batch; i += S5_THREADS) npg_sm[i] = p.n_pages[i];
  __syncthreads();
  const int total = cum[p.batch];
  const int per_cta = (total + gridDim.x - 1) / gridDim.x;
  const int f_begin = min(total, (int)blockIdx.x * per_cta);
  const int f_end = min(total, f_begin + per_cta);
  const int n_tiles = f_end - f_begin;
  if (n_tiles <= 0) return;

  // ---- prologue: zeroed operand rows (query rows beyond the group stay zero), barriers, tensor memory ----
  for (int i = tid; i < (STG + 2) * QB_BYTES / 16; i += S5_THREADS) reinterpret_cast<uint4*>(pbuf0)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (tid == 0) {
    for (int s = 0; s < STG; ++s) mbar_init(&sh->full[s], 2), mbar_init(&sh->empty[s], 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh->low[b], 1), mbar_init(&sh->sdone[b], 1), mbar_init(&sh->odone[b], 1);
      sh->kcnt[b] = sh->pcnt[b] = sh->vcnt[b] = sh->ycnt[b] = 0;
    }
    sh->released = 0, sh->bcnt = 0, sh->ccnt = 0, sh->slot_seq[0] = sh->slot_seq[1] = 0;
    fence_barrier_init();
  }
  if (warp == SVC0 + 1) {
    tc5::alloc(smem_u32(&sh->tmem_base), TM_COLS);
    tc5::relinquish();
  }
  fence_proxy_async();
  tc5::fence_before();
  __syncthreads();
  tc5::fence_after();
  const uint32_t tmem = sh->tmem_base;

  Walker w;
  w.init(cum, npg_sm, f_begin, h_kv);

  if (warp < KEY_WARPS) {
    // ===================== key warps: 32 token rows x two chunks of 16 + 16 channels =====================
    set_regs<REG_KEY>();
    constexpr int KCH = 16 / KEY_WARPS;  // chunks of 16 + 16 channels per key warp
    const int wq = warp & 3, k0 = KCH * (warp >> 2), row = 32 * wq + lane;
    const uint32_t tk = tmem + TM_KD + ((uint32_t)(32 * wq) << 16);
    // rotation by this token's offset inside the tile, for rotary pairs 16k .. 16k+15 of both chunks
    uint32_t cs_[KCH][8], sn_[KCH][8];
#pragma unroll
    for (int kk = 0; kk < KCH; ++kk)
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        cs_[kk][i] = *reinterpret_cast<const uint32_t*>(p.rope_cos + (int64_t)row * HEAD_DIM + 16 * (k0 + kk) + 2 * i);
        sn_[kk][i] = *reinterpret_cast<const uint32_t*>(p.rope_sin + (int64_t)row * HEAD_DIM + 16 * (k0 + kk) + 2 * i);
      }
    for (int n = 0; n < n_tiles; ++n) {
      const int b = n & 1;
      if (!wait_or_flag(&sh->low[b], (uint32_t)(n >> 1) & 1u, p.status, 6)) break;
      tc5::fence_after();
#pragma unroll
      for (int kk = 0; kk < KCH; ++kk) {
        const int k = k0 + kk;
        uint32_t dl[8], dh[8], out[16];
        tc5::ld16_pack(tk + 128 * b + 16 * k, dl);
        tc5::ld16_pack(tk + 128 * b + 64 + 16 * k, dh);
        tc5::wait_ld();
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __half2 klo = u32_as_h2(dl[i]), khi = u32_as_h2(dh[i]);
          const __half2 c = u32_as_h2(cs_[kk][i]), sn = u32_as_h2(sn_[kk][i]);
          out[i] = h2_as_u32(__hfma2(__hneg2(sn), khi, __hmul2(klo, c)));
          out[8 + i] = h2_as_u32(__hfma2(sn, klo, __hmul2(khi, c)));
        }
        tc5::st16(tk + 128 * b + 16 * k, out);
      }
      tc5::wait_st();
      tc5::fence_before();
      __syncwarp();
      if (lane == 0) smem_add_release(&sh->kcnt[b], 1);
    }
  } else if (warp >= W_DQ && warp < SVC0) {
    // ===================== dequant warps: tier codes -> fp16 Y_hat, the A operand of U1 =====================
    // Warp wd takes the direction octets wd, wd + DQ_WARPS, ... (positions in tier order).  Lane = (direction
    // lane / 4 of the octet, token pair q = lane % 4): for every 8-token block B it produces the half2 of tokens
    // 8B + 2q, 8B + 2q + 1 of its direction, which is exactly what a transposed stmatrix wants from it.  Four
    // blocks (32 tokens, one 8 / 16 / 32-byte piece of the direction's row) go out per stmatrix.
    // A half2 costs four instructions whatever the tier: a byte permute drops the thread's code byte(s) under the
    // fp16 exponent of 1024 in both halves, one LOP3 masks each half down to its field and flips two's-complement
    // sign bits, an exact subtraction removes 1024 and the field's offset (times the field's position in the byte),
    // and a multiply applies the scale (divided by that position, a power of two).  The tier only changes the
    // constants (selectors, mask, offsets), which each lane derives for its own direction: one compact loop serves
    // every width with no divergence, so the warp-wide stmatrix is always reached by all 32 lanes.
    set_regs<REG_DEQUANT>();
    constexpr int OCT = 16 / DQ_WARPS;
    const int wd = warp - W_DQ, q = lane & 3, dsub = lane >> 2;
    const int ngrp = 128 / p.group, gsh = (p.group == 32) ? 0 : (p.group == 64 ? 1 : 2);
    const uint32_t st_lane = (uint32_t)((lane >> 3) * 16 * 128 + (lane & 7) * 16);
    const int a2 = 4 * (q & 1);  // 2-bit containers: this thread's two fields start at bits a2 and a2 + 2 of its byte
    static_assert(OCT == 1, "one direction octet per dequant warp: its constants live in registers for a whole range");
    int s = 0;
    uint32_t fp = 0;
    // Constants of this lane's direction (position 8 wd + dsub of the head's tier order); they change with the head only.
    int cur_h = -1;
    bool active = false, has_bits = false;
    uint32_t piece = 0, wo1 = 0, wo2 = 0, wo3 = 0, sel_e = 0, sel_o = 0, mask = 0, X2 = 0, row_off = 0, sc_off = 0;
    float plo = 0.f, phi = 0.f;
    __half2 bias2 = __floats2half2_rn(0.f, 0.f);
    for (int n = 0; n < n_tiles; ++n) {
      const int b = n & 1;
      if (!wait_or_flag(&sh->full[s], fp, p.status, 13)) break;
      const int h = sh->head[s];  // left with the stage by the query rotation warp: these warps do not walk the tile list
      if (h != cur_h) {
        cur_h = h;
        const int mt = __ldg(p.meta + h * HEAD_DIM + 8 * wd + dsub);
        const int n_oct = 2 * (((__ldg(p.meta + h * HEAD_DIM) >> 28) & 7) + 1);  // octets that U1 reads for this head
        active = wd < n_oct;  // the same for the whole warp
        const int off = mt & 0xFFFF, d = (mt >> 16) & 127, bits = (mt >> 24) & 15;
        has_bits = bits != 0;
        // container width 2 / 4 / 8 bits: one 32-token piece of the row is 8 / 16 / 32 bytes
        const bool w2 = (bits == 2), w8 = (bits >= 5);
        piece = w2 ? 8u : (w8 ? 32u : 16u);
        // word (byte offset inside the piece) and byte selector of block m = 0..3 of a piece
        //   2-bit: byte 2 (m % 2) + q / 2 of word m / 2;  4-bit: byte q of word m;  8-bit: bytes 2 (q % 2), + 1 of word 2 m + q / 2
        const uint32_t wstep = w2 ? 2u : (w8 ? 8u : 4u);   // byte offset of block m's word = (m * wstep rounded down to 4) + wbase
        wo1 = wstep & ~3u, wo2 = (2u * wstep) & ~3u, wo3 = (3u * wstep) & ~3u;
        const uint32_t wbase = w8 ? 4u * (uint32_t)(q >> 1) : 0u;
        const uint32_t byte_e = w2 ? (uint32_t)(q >> 1) : (w8 ? 2u * (uint32_t)(q & 1) : (uint32_t)q);   // source byte that lands in the low half
        const uint32_t hi_inc = w8 ? 1u : 0u;                                                              // the high half takes the next byte (8-bit) or the same one
        sel_e = 0x4040u | byte_e | ((byte_e + hi_inc) << 8);
        sel_o = w2 ? sel_e + 0x0202u : sel_e;       // 2-bit: odd blocks sit two bytes further in the same word
        mask = w2 ? (((0xFF00u | (0x3u << (a2 + 2))) << 16) | (0xFF00u | (0x3u << a2))) : (w8 ? 0xFFFFFFFFu : 0xFFF0FF0Fu);
        X2 = (bits == 3) ? 0x00800008u : (w8 ? 0x00800080u : 0u);   // two's-complement fields: flip the sign bit
        // field offset still to subtract (times the field's position) and the position itself
        const float blo = w2 ? (float)(2 << a2) : (w8 ? 128.f : 8.f), bhi = w2 ? (float)(2 << (a2 + 2)) : 128.f;
        plo = w2 ? 1.f / (float)(1 << a2) : 1.f, phi = w2 ? 1.f / (float)(1 << (a2 + 2)) : (w8 ? 1.f : 0.0625f);
        bias2 = __floats2half2_rn(1024.f + blo, 1024.f + bhi);
        row_off = (uint32_t)off + wbase;
        sc_off = (uint32_t)(d * ngrp);
      }
      // the buffer still feeds U1 of tile n-2
      if (n >= 2 && !wait_or_flag(&sh->low[b], (uint32_t)((n - 2) >> 1) & 1u, p.status, 14)) break;
      if (active) {
        const uint8_t* kb = stage0 + (size_t)s * STAGE_BYTES;
        const uint8_t* rowp = kb + row_off;
        const float* scp = reinterpret_cast<const float*>(kb + p.scale_off) + sc_off;
        uint32_t st_addr = smem_u32(ybuf0 + (size_t)b * OPER_BYTES) + (uint32_t)wd * 128u + st_lane;
#pragma unroll 1
        for (int c = 0; c < 4; ++c, rowp += piece, st_addr += 4u * 16u * 128u) {
          const uint32_t wv0 = *reinterpret_cast<const uint32_t*>(rowp), wv1 = *reinterpret_cast<const uint32_t*>(rowp + wo1);
          const uint32_t wv2 = *reinterpret_cast<const uint32_t*>(rowp + wo2), wv3 = *reinterpret_cast<const uint32_t*>(rowp + wo3);
          const float scf = has_bits ? scp[c >> gsh] : 0.f;   // directions without bits: everything times zero
          const __half2 s2 = __floats2half2_rn(scf * plo, scf * phi);
          uint32_t r[4];
          r[0] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(lop3<0x6A>(prmt(wv0, 0x64646464u, sel_e), mask, X2)), bias2), s2));
          r[1] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(lop3<0x6A>(prmt(wv1, 0x64646464u, sel_o), mask, X2)), bias2), s2));
          r[2] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(lop3<0x6A>(prmt(wv2, 0x64646464u, sel_e), mask, X2)), bias2), s2));
          r[3] = h2_as_u32(__hmul2(__hsub2(u32_as_h2(lop3<0x6A>(prmt(wv3, 0x64646464u, sel_o), mask, X2)), bias2), s2));
          stmatrix_x4_trans(st_addr, r);
        }
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) smem_add_release(&sh->ycnt[b], 1);
      if (++s == STG) s = 0, fp ^= 1u;
    }
  } else if (warp >= W_VAL && warp < W_DQ) {
    // ===================== value warps: thread = channel, both 64-token halves of the tile =====================
    set_regs<REG_VALUE>();
    const int wq = warp & 3, ch = 32 * wq + lane;
    constexpr int cc0 = 0, cc1 = 2;
    const uint32_t tv = tmem + TM_V + ((uint32_t)(32 * wq) << 16);
    int s = 0;
    uint32_t fp = 0;
    for (int n = 0; n < n_tiles; ++n) {
      const int b = n & 1;
      if (!wait_or_flag(&sh->full[s], fp, p.status, 10)) break;
      // the columns still feed U3 of tile n-2
      if (n >= 2 && !wait_or_flag(&sh->odone[b], (uint32_t)((n - 2) >> 1) & 1u, p.status, 11)) break;
      tc5::fence_after();
      const uint4* vc = reinterpret_cast<const uint4*>(stage0 + (size_t)s * STAGE_BYTES + KB);
#pragma unroll 1
      for (int cc = cc0; cc < cc1; ++cc) {
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
      if (++s == STG) s = 0, fp ^= 1u;
    }
  } else if (warp >= W_SOFT && warp < W_VAL) {
    // ===================== softmax warps: thread = token row =====================
    // One set of four warps takes every tile: running (max, sum) and ONE output accumulator per range.  Scores, the
    // weight buffer and the flags alternate by tile parity (U2 / U3 of neighbouring tiles overlap with this role).
    set_regs<REG_SOFTMAX>();
    const int wq = warp & 3, row = 32 * wq + lane;
    const uint32_t tl = tmem + ((uint32_t)(32 * wq) << 16);
    float m[GQ], l[GQ], pn[GQ];
#pragma unroll
    for (int qi = 0; qi < GQ; ++qi) m[qi] = -INFINITY, l[qi] = 0.f, pn[qi] = 0.f;
    int cur_seg = -1, cur_b = 0, cur_h = 0, last_n = -1;
    bool had = false, alive = true;

    // Writes the partial record of the range that just ended.
    auto flush = [&](int b_, int h_) {
      float acc[GQ];
#pragma unroll
      for (int qi = 0; qi < GQ; ++qi) acc[qi] = 0.f;
      // U3s complete in issue order: the last tile's completion covers the whole range
      if (had && alive && !wait_or_flag(&sh->odone[last_n & 1], (uint32_t)(last_n >> 1) & 1u, p.status, 9)) alive = false;
      if (had && alive) {
        tc5::fence_after();
        uint32_t r[GQ];
        if constexpr (GQ == 4) tc5::ld4(tl + TM_O, r); else tc5::ld8(tl + TM_O, r);
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
        if (lane == 0) sh->red[0][wq][qi] = a, sh->red[0][wq][GQ + qi] = b2;
      }
      named_bar(1, 128);
      float* dst = p.part + ((blockIdx.x + (int64_t)b_ * h_kv + h_) * G) * PART_STRIDE;
#pragma unroll
      for (int qi = 0; qi < GQ; ++qi)
        if (qi < G) {
          const float L = sh->red[0][0][qi] + sh->red[0][1][qi] + sh->red[0][2][qi] + sh->red[0][3][qi];
          const float P = sh->red[0][0][GQ + qi] + sh->red[0][1][GQ + qi] + sh->red[0][2][GQ + qi] + sh->red[0][3][GQ + qi];
          dst[qi * PART_STRIDE + 2 + row] = had ? p.lut_alpha * P + p.lut_beta * acc[qi] : 0.f;
          if (row == 0) dst[qi * PART_STRIDE] = had ? m[qi] : -INFINITY, dst[qi * PART_STRIDE + 1] = had ? L : 0.f;
        }
      named_bar(1, 128);
    };

    int s = 0;
    uint32_t fp = 0;
    for (; w.it < n_tiles; w.advance(npg_sm, h_kv, p.batch), s = (s + 1 == STG) ? 0 : s + 1, fp ^= (s == 0) ? 1u : 0u) {
      const int n = w.it, e = n & 1;
      if (w.seg != cur_seg) {
        if (cur_seg >= 0) flush(cur_b, cur_h);
        cur_seg = w.seg, cur_b = w.cur.b, cur_h = w.cur.h, had = false;
#pragma unroll
        for (int qi = 0; qi < GQ; ++qi) m[qi] = -INFINITY, l[qi] = 0.f, pn[qi] = 0.f;
      }
      const uint32_t par = (uint32_t)(n >> 1) & 1u;
      const uint8_t* vblk = stage0 + (size_t)s * STAGE_BYTES + KB;
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
      named_bar(1, 128);
      const int4 fl = *reinterpret_cast<const int4*>(sh->flag[e]);
      const bool resc = (fl.x | fl.y | fl.z | fl.w) != 0;
      // the weight buffer of this parity still belongs to U3 of tile n-2
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
        named_bar(1, 128);
#pragma unroll
        for (int qi = 0; qi < GQ; ++qi) {
          const float tm = fmaxf(fmaxf(sh->wmax[e][0][qi], sh->wmax[e][1][qi]), fmaxf(sh->wmax[e][2][qi], sh->wmax[e][3][qi]));
          mnew[qi] = (qi < G && tm > m[qi] + 8.f) ? tm : m[qi];
        }
        // the accumulator is rescaled in place: U3 of tile n-1 must have finished with it (U3 of this tile waits for this
        // role's arrival below)
        if (alive && had && !wait_or_flag(&sh->odone[e ^ 1], (uint32_t)((n - 1) >> 1) & 1u, p.status, 15)) alive = false;
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
            if constexpr (GQ == 4) tc5::ld4(tl + TM_O, r); else tc5::ld8(tl + TM_O, r);
            tc5::wait_ld();
#pragma unroll
            for (int qi = 0; qi < GQ; ++qi) r[qi] = __float_as_uint(__uint_as_float(r[qi]) * f[qi]);
            if constexpr (GQ == 4) tc5::st4(tl + TM_O, r); else tc5::st8(tl + TM_O, r);
            tc5::wait_st();
          }
        }
      }
      if (alive) {
        const float norm = __half2float(reinterpret_cast<const __half*>(vblk + 128 * 32)[row]);
        __half* pb = reinterpret_cast<__half*>(pbuf0 + (size_t)e * QB_BYTES) + (row >> 3) * 64 + (row & 7);
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
    set_regs<REG_SERVICE>();  // the four service warps, as one group
    if (warp == SVC0) {
      // ===================== copy + U3 warp =====================
      constexpr uint32_t ID_N16 = tc5::idesc_f16_f32(128, 16);
      const bool el = elect_one();
      const uint64_t d_pb = tc5::smem_desc(smem_u32(pbuf0), 128, 2048);
      int nC = 0, nP = 0, sC = 0, sP = 0;
      uint32_t phP = 1;  // parity to wait for on empty[sP]: a fresh barrier passes parity 1
      long long t_last = clock64();
      uint32_t idle = 0;
      bool ok = true;
      while (ok && nC < n_tiles) {
        bool progressed = false;
        const int pc = smem_load_acquire(&sh->pcnt[nC & 1]);
        const int vc = smem_load_acquire(&sh->vcnt[nC & 1]);
        const int bdone = smem_load_acquire(&sh->bcnt);
        if (nC < bdone && pc >= 4 * ((nC >> 1) + 1) && vc >= VAL_WARPS * ((nC >> 1) + 1)) {
          tc5::fence_after();
          const int b = nC & 1;
          const uint32_t keep = sh->first[sC] ? 0u : 1u;  // the first tile of a range starts a new accumulator
          const uint64_t db = d_pb + (uint64_t)(b * (QB_BYTES >> 4));
          ++nC;
          if (el) {
            // one accumulator for the whole range: the U3s of consecutive tiles are issued by this thread in order
            tc5::mma_ts(tmem + TM_O, tmem + TM_V + 64 * b, db, ID_N16, keep);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks) tc5::mma_ts(tmem + TM_O, tmem + TM_V + 64 * b + 8 * ks, db + 16 * ks, ID_N16, 1u);
            tc5::commit(smem_u32(&sh->odone[b]));
            mbar_arrive(&sh->empty[sC]);
            smem_add_release(&sh->ccnt, 1);
            sh->released = nC;
          }
          __syncwarp();
          if (++sC == STG) sC = 0;
          progressed = true;
        }
        if (nP < n_tiles && smem_load_acquire(&sh->slot_seq[nP & 1]) > nP && mbar_test_wait(&sh->empty[sP], phP)) {
          const int h = w.cur.h, slot = sh->slot_ring[nP & 15];
          uint8_t* st = stage0 + (size_t)sP * STAGE_BYTES;
          if (el) {
            mbar_arrive_expect_tx(&sh->full[sP], (uint32_t)(KB + VBLOCK));
            bulk_g2s(st, p.kpages + ((int64_t)slot * h_kv + h) * KB, KB, &sh->full[sP]);
            bulk_g2s(st + KB, p.vpages + ((int64_t)slot * h_kv + h) * VBLOCK, VBLOCK, &sh->full[sP]);
          }
          __syncwarp();
          ++nP;
          if (++sP == STG) sP = 0, phP ^= 1u;
          if (nP < n_tiles) w.advance(npg_sm, h_kv, p.batch);
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
    } else if (warp >= SVC0 + 2) {
      // ===================== query rotation warps: tiles of parity rw =====================
      // q_rot = R(-t0) q * scale as the B operand of U2, in the K order the key warps produce: position
      // 32k + e holds channel 16k + e (e < 16) or 64 + 16k + (e - 16).  The warp that meets the first tile of
      // a (sequence, head) range also lays out that head's decoder as the B operand of U1.
      const int rw = warp - (SVC0 + 2);
      int s = 0;
      uint32_t ph = 1;
      int prev_seg = -1, first_cur = 0, first_prev = 0;
      bool alive = true;
      for (; w.it < n_tiles && alive; w.advance(npg_sm, h_kv, p.batch)) {
        const bool new_seg = (w.seg != prev_seg);
        if (new_seg) first_prev = first_cur, first_cur = w.it, prev_seg = w.seg;
        if ((w.it & 1) == rw) {
          const int b = w.cur.b, h = w.cur.h, j = w.cur.j;
          const int64_t t0 = p.pos_offset + (int64_t)j * TILE_TOKENS;
          const __half* qsrc = p.q + ((int64_t)b * h_kv + h) * G * HEAD_DIM;
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
          __half* qr = reinterpret_cast<__half*>(qb0 + (size_t)s * QB_BYTES);
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
            uint4* bd = reinterpret_cast<uint4*>(bbuf0 + (size_t)(w.seg & 1) * OPER_BYTES);
            const uint4* bs = reinterpret_cast<const uint4*>(p.dec16 + (int64_t)h * HEAD_DIM * HEAD_DIM);
            for (int o = lane; o < 128 * 16; o += 32) {
              const int c = o >> 4, i8 = o & 15;
              bd[((c >> 3) * 16 + i8) * 8 + (c & 7)] = bs[o];
            }
          }
          if (lane == 0) {
            sh->bsel[s] = w.seg & 1, sh->first[s] = (w.it == first_cur) ? 1 : 0;
            sh->ksteps[s] = ((__ldg(p.meta + h * HEAD_DIM) >> 28) & 7) + 1;
            sh->head[s] = h;
          }
          fence_proxy_async();
          __syncwarp();
          if (lane == 0) mbar_arrive(&sh->full[s]);
        }
        if (++s == STG) s = 0, ph ^= 1;
      }
    } else {
      // ===================== issuing warp: U1 and U2 =====================
      // A(n): U1 of tile n once its Y_hat is complete (the dequant warps waited for the tile's stage, so the
      // decoder operand and the stage's flags have landed too) and U2(n-2) has finished with the K columns.
      // B(n): U2 once all key warps have written the rotated keys and the softmax of tile n-2 is done with the
      // score columns.
      constexpr uint32_t ID_U1 = tc5::idesc_f16_f16(128, 128), ID_N16 = tc5::idesc_f16_f32(128, 16);
      const bool el = elect_one();
      int nA = 0, nB = 0, sA = 0, sB = 0;
      const uint64_t d_y = tc5::smem_desc(smem_u32(ybuf0), 128, AB_SBO), d_bbuf = tc5::smem_desc(smem_u32(bbuf0), 128, AB_SBO);
      const uint64_t d_qb = tc5::smem_desc(smem_u32(qb0), 128, 2048);
      long long t_last = clock64();
      uint32_t idle = 0;
      bool ok = true;
      while (ok && nB < n_tiles) {
        bool progressed = false;
        const int kc = smem_load_acquire(&sh->kcnt[nB & 1]);
        const int nC = smem_load_acquire(&sh->ccnt);
        const int yc = smem_load_acquire(&sh->ycnt[nA & 1]);
        // ---- B ----
        if (nB < nA && nB < nC + 2 && kc >= KEY_WARPS * ((nB >> 1) + 1)) {
          tc5::fence_after();
          const int b = nB & 1;
          const uint64_t db = d_qb + (uint64_t)(sB * (QB_BYTES >> 4));
          if (el) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) tc5::mma_ts(tmem + TM_S + 16 * b, tmem + TM_KD + 128 * b + 8 * ks, db + 16 * ks, ID_N16, ks > 0);
            tc5::commit(smem_u32(&sh->sdone[b]));
            smem_add_release(&sh->bcnt, 1);
          }
          __syncwarp();
          ++nB;
          if (++sB == STG) sB = 0;
          progressed = true;
        }
        // ---- A ----
        if (nA < n_tiles && nA < nB + 2 && yc >= DQ_WARPS * ((nA >> 1) + 1) &&
            (nA < 2 || mbar_test_wait(&sh->sdone[nA & 1], (uint32_t)((nA - 2) >> 1) & 1u))) {
          tc5::fence_after();
          const int b = nA & 1;
          const uint64_t da = d_y + (uint64_t)(b * (OPER_BYTES >> 4)), db = d_bbuf + (uint64_t)(sh->bsel[sA] * (OPER_BYTES >> 4));
          const int nks = sh->ksteps[sA];  // directions without bits sit last in tier order: their K steps are left out
          if (el) {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks)
              if (ks < nks) tc5::mma_ss(tmem + TM_KD + 128 * b, da + 16 * ks, db + 16 * ks, ID_U1, ks > 0);
            tc5::commit(smem_u32(&sh->low[b]));
          }
          __syncwarp();
          ++nA;
          if (++sA == STG) sA = 0;
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
  if (warp == SVC0 + 1) {
    tc5::fence_after();
    tc5::dealloc(tmem, TM_COLS);
  }
}

template <int GQ>
static int launch_s5(const SpectralDecodeParams& prm, int grid, size_t smem, cudaStream_t s) {
  static PerDeviceOnce configured;
  if (configured.first()) {
    cudaError_t e = cudaFuncSetAttribute(spectral_decode_t5_kernel<GQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) {
      configured.retract();
      set_error("bmxk_spectral_decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return BMXK_ERR_CUDA;
    }
  }
  spectral_decode_t5_kernel<GQ><<<grid, S5_THREADS, smem, s>>>(prm);
  return check_launch("bmxk_spectral_decode");
}

static size_t s5_fixed_smem(int batch) {
  return (size_t)4 * OPER_BYTES + 2 * QB_BYTES + sizeof(S5Smem) + (size_t)(2 * batch + 1) * 4 + 16;
}

}  // namespace bmxk

using namespace bmxk;

extern "C" {

size_t bmxk_spectral_decode_workspace_bytes(const bmxk_spectral_geom* g, int n_q_groups, int batch) {
  if (!g || batch <= 0 || n_q_groups <= 0) return 0;
  const size_t slots = (size_t)num_sms() + (size_t)batch * g->h_kv;  // one record per (CTA, range)
  return 256 + slots * n_q_groups * PART_STRIDE * sizeof(float);
}

int bmxk_spectral_decode(const bmxk_spectral_geom* g, int n_q_groups, const void* q, const void* kpages, const void* vpages,
                         const void* dec_f16, const int32_t* meta, const int32_t* page_table, int table_stride,
                         const int32_t* n_pages, int batch, int max_pages, const void* rope_cos, const void* rope_sin,
                         int64_t pos_offset, const void* k_tail, const void* v_tail, const int32_t* tail_len, int tail_cap,
                         const uint32_t* v_lut, const float* signs, float sm_scale, void* workspace, size_t workspace_bytes,
                         void* out, int out_dtype, float* partial_out, int phases, void* stream) {
  BMXK_REQUIRE(g != nullptr, "bmxk_spectral_decode: null geometry");
  BMXK_REQUIRE(phases >= 1 && phases <= 3, "bmxk_spectral_decode: phases=%d must be 1, 2 or 3", phases);
  BMXK_REQUIRE(g->h_kv >= 1 && g->h_kv <= 64 && n_q_groups >= 1 && n_q_groups <= 8, "bmxk_spectral_decode: h_kv=%d n_q_groups=%d",
               g->h_kv, n_q_groups);
  BMXK_REQUIRE(g->page == 128, "bmxk_spectral_decode: page=%d (the fused kernel reads 128-token pages)", g->page);
  BMXK_REQUIRE(g->group == 32 || g->group == 64 || g->group == 128, "bmxk_spectral_decode: group=%d must be 32, 64 or 128", g->group);
  BMXK_REQUIRE(g->block_bytes > 0 && g->block_bytes % 16 == 0 && g->block_bytes < 65536 && g->scale_off % 16 == 0 &&
                   g->scale_off + HEAD_DIM * (128 / g->group) * 4 <= g->block_bytes,
               "bmxk_spectral_decode: inconsistent block_bytes=%d / scale_off=%d", g->block_bytes, g->scale_off);
  BMXK_REQUIRE(batch >= 1 && (int64_t)batch * g->h_kv <= MAX_BH, "bmxk_spectral_decode: batch*h_kv=%lld out of range",
               (long long)batch * g->h_kv);
  BMXK_REQUIRE(max_pages >= 0 && tail_cap >= 0, "bmxk_spectral_decode: negative sizes");
  BMXK_REQUIRE(q && n_pages && v_lut && signs && workspace, "bmxk_spectral_decode: null pointer");
  BMXK_REQUIRE(max_pages == 0 || (kpages && vpages && dec_f16 && meta && page_table && rope_cos && rope_sin),
               "bmxk_spectral_decode: null page pools / tables");
  BMXK_REQUIRE(tail_cap == 0 || (k_tail && v_tail && tail_len), "bmxk_spectral_decode: null tail");
  BMXK_REQUIRE(out || partial_out, "bmxk_spectral_decode: no output");
  BMXK_REQUIRE(out_dtype == BMXK_DTYPE_F16 || out_dtype == BMXK_DTYPE_F32, "bmxk_spectral_decode: out_dtype=%d", out_dtype);
  BMXK_REQUIRE(workspace_bytes >= bmxk_spectral_decode_workspace_bytes(g, n_q_groups, batch), "bmxk_spectral_decode: workspace too small");
  BMXK_REQUIRE(((uintptr_t)kpages & 15) == 0 && ((uintptr_t)vpages & 15) == 0 && ((uintptr_t)dec_f16 & 15) == 0,
               "bmxk_spectral_decode: pools and the decoder operand must be 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;

  int32_t* status = reinterpret_cast<int32_t*>(workspace);
  float* part = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + 256);
  const int64_t max_tiles = (int64_t)batch * g->h_kv * max_pages;
  const int grid = (int)(max_tiles < num_sms() ? (max_tiles < 1 ? 1 : max_tiles) : num_sms());
  const float scale_log2 = sm_scale * 1.4426950408889634f;
  float alpha, beta;
  memcpy(&alpha, &v_lut[2], 4);
  memcpy(&beta, &v_lut[3], 4);

  if (max_pages > 0 && (phases & 1)) {
    SpectralDecodeParams prm;
    prm.h_kv = g->h_kv, prm.n_q_groups = n_q_groups, prm.group = g->group, prm.kblock_bytes = g->block_bytes;
    prm.scale_off = g->scale_off;
    const size_t fixed = s5_fixed_smem(batch), per_stage = (size_t)QB_BYTES + g->block_bytes + VBLOCK;
    BMXK_REQUIRE(fixed + 2 * per_stage <= 227 * 1024, "bmxk_spectral_decode: key block of %d bytes (or batch=%d) leaves no room for two stages",
                 g->block_bytes, batch);
    int n_stages = (int)((227 * 1024 - fixed) / per_stage);
    if (n_stages > S5_MAX_STAGES) n_stages = S5_MAX_STAGES;
    prm.n_stages = n_stages;
    prm.q = (const __half*)q, prm.kpages = (const uint8_t*)kpages, prm.vpages = (const uint8_t*)vpages;
    prm.dec16 = (const __half*)dec_f16, prm.meta = meta, prm.page_table = page_table, prm.table_stride = table_stride;
    prm.n_pages = n_pages, prm.batch = batch, prm.rope_cos = (const __half*)rope_cos, prm.rope_sin = (const __half*)rope_sin;
    prm.pos_offset = pos_offset, prm.lut_lo = v_lut[0], prm.lut_hi = v_lut[1], prm.lut_alpha = alpha, prm.lut_beta = beta;
    prm.scale_log2 = scale_log2, prm.part = part, prm.status = status;
    const size_t smem = fixed + (size_t)n_stages * per_stage;
    const int rc = (n_q_groups <= 4) ? launch_s5<4>(prm, grid, smem, s) : launch_s5<8>(prm, grid, smem, s);
    if (rc) return rc;
  }
  if (!(phases & 2)) return BMXK_OK;
  K2bMergeParams mp;
  mp.g.h_kv = g->h_kv, mp.g.n_q_groups = n_q_groups, mp.g.page = 128, mp.g.rank = 0, mp.g.group = g->group;
  mp.g.n_coef_heads = g->h_kv, mp.g.kbits = 0, mp.g.vbits = 2, mp.g.layout = 1;
  mp.n_sub = 1;
  mp.q = (const __half*)q, mp.n_pages = n_pages, mp.batch = batch, mp.main_grid = grid, mp.part = part;
  mp.k_tail = (const __half*)k_tail, mp.v_tail = (const __half*)v_tail, mp.tail_len = tail_cap > 0 ? tail_len : nullptr;
  mp.tail_cap = tail_cap, mp.signs = signs, mp.scale_log2 = scale_log2, mp.out = out, mp.out_dtype = out_dtype;
  mp.partial_out = partial_out;
  return launch_merge(mp, s, max_pages > 0 && (phases & 1));
}

}  // extern "C"
