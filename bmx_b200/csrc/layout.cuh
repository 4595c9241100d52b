// Native HBM layout of one k2b page and the index arithmetic shared by every kernel that
// touches it (append, export, dequant, decode).  Head dim is fixed at 128.
//
// A page is PAGE tokens (64 or 128) of ONE sequence.  For each physical page slot the pool
// holds, per KV head, one contiguous "page block":
//
//   [ K residual nibbles | K residual scales | V codes | V norms ]
//
// and, per coefficient head (1 when the key basis spans all heads, h_kv when each head has
// its own basis), one "coef block" of PAGE x rank fp16 low-rank coefficients.
//
// The bytes are the reference's (two's-complement residual nibbles, offset-free 2-bit V
// indices, fp16 scales / norms / coefficients: bmx src/bmx/cache/triton_dequant_attention.py
// :1118-1229) but ORDERED for the decode kernel: every array is cut into 16-token "warp rows"
// and, inside a warp row, into the per-lane fragments that mma.sync m16n8k16 expects, so that
// one bulk copy lands a page in shared memory and each lane reads its operands with 128-bit
// loads and no shuffles.  `bmxk_k2b_export_stacks` undoes the ordering for byte parity.
//
// Lane coordinates: lane = 4*g + t  (g = lane / 4 in 0..7, t = lane % 4).
//
// K residual (4-bit container, code for (row r, channel c)):
//   warp row wr = r / 16, rr = r % 16, token half th = rr / 8, g = rr % 8
//   n = c / 8 (8-channel tile), t = (c % 8) / 2, e = c % 2, q = n / 4, i = n % 4
//   32-bit word index  ((wr*2 + th)*32 + 4*g + t)*4 + q ; bit offset 16*e + 4*i
//   -> a lane's (token g or g+8) x (channels 8n+2t, 8n+2t+1) codes sit in matching nibbles of
//      the low and high halves of a word: one LOP3 turns them into a half2.
// K residual scale (fp16, per channel per `group` tokens):
//   half index  grp*128 + (n/4)*32 + t*8 + (n%4)*2 + e      (grp = r / group)
//   -> the four 16-byte chunks a lane reads are 64 bytes apart and the four t of a quad are
//      adjacent, so a quarter-warp's 128-bit loads fall in distinct banks
// V code (2-bit index for (row r, channel c)):
//   wr = r / 16, rr = r % 16; mt = c / 16 (16-channel tile), cc = c % 16
//   g = cc % 8, chi = cc / 8 ; t = (rr % 8) / 2, e = rr % 2, thi = rr / 8
//   A-fragment register a = 2*thi + chi  (a0..a3 of mma m16n8k16 with rows = channels,
//   k = tokens); word j = mt / 2, hs = mt % 2
//   32-bit word index  (wr*32 + 4*g + t)*4 + j ; bit offset 16*hs + 4*(2*(a&1) + e) + 2*(a>>1)
// V norm (fp16 per token): half index r.
#pragma once
#include <cstdint>

#if defined(__CUDACC__)
#define BMXK_HD __host__ __device__ __forceinline__
#else
#define BMXK_HD inline
#endif

namespace bmxk {

constexpr int HEAD_DIM = 128;

struct K2bGeom {
  int h_kv;          // KV heads
  int n_q_groups;    // query heads per KV head (GQA group), <= 8
  int page;          // tokens per page: 64 or 128
  int rank;          // low-rank coefficients per token: 16 or 32
  int group;         // K residual scale group along tokens; divides page
  int n_coef_heads;  // 1 (basis spans all heads) or h_kv (one basis per head)
  int kbits;         // K residual code width (<= 4, stored as nibbles)
  int vbits;         // V code width (2)
  int layout;        // 0: fragment order (below); 1: row order for the tcgen05 decode kernel (page 128 only)
};

BMXK_HD int k2b_kres_bytes(int page) { return page * 64; }
BMXK_HD int k2b_kscale_bytes(int page, int group) { return (page / group) * 128 * 2; }
BMXK_HD int k2b_vcode_bytes(int page) { return page * 32; }
BMXK_HD int k2b_vnorm_bytes(int page) { return page * 2; }
BMXK_HD int k2b_off_kscale(int page) { return k2b_kres_bytes(page); }
BMXK_HD int k2b_off_vcode(int page, int group) { return k2b_off_kscale(page) + k2b_kscale_bytes(page, group); }
BMXK_HD int k2b_off_vnorm(int page, int group) { return k2b_off_vcode(page, group) + k2b_vcode_bytes(page); }
BMXK_HD int k2b_page_block_bytes(int page, int group) { return k2b_off_vnorm(page, group) + k2b_vnorm_bytes(page); }
BMXK_HD int k2b_coef_block_bytes(int page, int rank) { return page * rank * 2; }

// word index (in 32-bit words from the start of the K residual array) and bit offset
BMXK_HD void k2b_kres_loc(int r, int c, int& word, int& bit) {
  const int wr = r >> 4, rr = r & 15, th = rr >> 3, g = rr & 7;
  const int n = c >> 3, t = (c & 7) >> 1, e = c & 1, q = n >> 2, i = n & 3;
  word = ((wr * 2 + th) * 32 + 4 * g + t) * 4 + q;
  bit = 16 * e + 4 * i;
}
BMXK_HD int k2b_kscale_idx(int grp, int c) {
  const int n = c >> 3, t = (c & 7) >> 1, e = c & 1;
  return grp * 128 + (n >> 2) * 32 + t * 8 + (n & 3) * 2 + e;
}
BMXK_HD void k2b_vcode_loc(int r, int c, int& word, int& bit) {
  const int wr = r >> 4, rr = r & 15;
  const int mt = c >> 4, cc = c & 15, g = cc & 7, chi = cc >> 3;
  const int t = (rr & 7) >> 1, e = rr & 1, thi = rr >> 3;
  const int a = 2 * thi + chi, j = mt >> 1, hs = mt & 1;
  word = (wr * 32 + 4 * g + t) * 4 + j;
  bit = 16 * hs + 4 * (2 * (a & 1) + e) + 2 * (a >> 1);
}
// Coefficient rows are stored with their 16-byte chunks XOR-swizzled so that ldmatrix reads of
// eight consecutive rows hit distinct shared-memory banks.  Returns the half index of (r, i).
BMXK_HD int k2b_coef_idx(int r, int i, int rank) {
  const int chunk = i >> 3, within = i & 7;
  const int sw = (rank == 32) ? ((r >> 1) & 3) : ((r >> 2) & 1);
  return r * rank + ((chunk ^ sw) << 3) + within;
}


// ---------------------------------------------------------------------------------------------
// Layout 1 ("row order", page = 128 only): the same four arrays and the same sizes, ordered for a
// decode kernel in which one thread owns one token (keys) or one channel (values) and the
// contractions run on tcgen05.mma.  Every per-thread read is a 16-byte chunk and the chunks of
// consecutive threads are adjacent, so a warp's 128-bit shared-memory loads are conflict free.
//
// K residual: chunk k (0..3) of token r is the 16 bytes at ((k*128 + r)*16).  Its four words hold
//   channels 16k..16k+7, 16k+8..16k+15, 64+16k..64+16k+7, 64+16k+8..64+16k+15; inside a word the
//   low half carries the even channels and the high half the odd ones (nibble i = channel pair i),
//   so one LOP3 yields a half2 of two adjacent channels.
// K residual scale: half index grp*128 + c.
// V code: chunk cc (0..1) of channel c is the 16 bytes at ((cc*128 + c)*16); word j of it holds
//   tokens 64cc+16j .. +15: token tau < 8 at bit 4*tau, token tau >= 8 at bit 4*(tau-8)+2.
// V norm: half index r.
// Coefficients: the K-major, unswizzled operand form of tcgen05.mma: 8-row x 16-byte core
//   matrices, half index ((r/8)*(rank/8) + i/8)*64 + (r%8)*8 + i%8.
// ---------------------------------------------------------------------------------------------
BMXK_HD void k2b_kres_loc(int lay, int r, int c, int& word, int& bit) {
  if (lay == 0) return k2b_kres_loc(r, c, word, bit);
  const int hi = c >> 6, cc = c & 63, k = cc >> 4, j = 2 * hi + ((cc & 15) >> 3);
  word = (k * 128 + r) * 4 + j;
  bit = 16 * (c & 1) + 4 * ((c & 7) >> 1);
}
BMXK_HD int k2b_kscale_idx(int lay, int grp, int c) { return lay == 0 ? k2b_kscale_idx(grp, c) : grp * 128 + c; }
BMXK_HD void k2b_vcode_loc(int lay, int r, int c, int& word, int& bit) {
  if (lay == 0) return k2b_vcode_loc(r, c, word, bit);
  const int tau = r & 15;
  word = ((r >> 6) * 128 + c) * 4 + ((r & 63) >> 4);
  bit = tau < 8 ? 4 * tau : 4 * (tau - 8) + 2;
}
BMXK_HD int k2b_coef_idx(int lay, int r, int i, int rank) {
  if (lay == 0) return k2b_coef_idx(r, i, rank);
  return ((r >> 3) * (rank >> 3) + (i >> 3)) * 64 + (r & 7) * 8 + (i & 7);
}

}  // namespace bmxk
