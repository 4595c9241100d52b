/* bmxk -- C ABI of the B200 (sm_100a) packed KV-cache kernels behind the bmx cache API.
 *
 * Every entry point takes plain device pointers, sizes and a cudaStream_t (passed as void*),
 * returns 0 on success or a BMXK_ERR_* code, never throws, never synchronises the host and
 * never allocates device memory: callers own pages, workspaces and outputs.  After a non-zero
 * return, bmxk_last_error() describes the failure (thread-local string).
 *
 * "bmx:" citations name the reference function an entry point stands in for, by path inside
 * the bmx project.
 */
#ifndef BMXK_H_
#define BMXK_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BMXK_OK 0
#define BMXK_ERR_INVALID 1 /* bad argument, shape or alignment; nothing was launched */
#define BMXK_ERR_CUDA 2    /* a CUDA runtime call or kernel launch failed */
#define BMXK_ERR_DEVICE 3  /* a kernel reported a bounded wait that ran out (see status word) */

#define BMXK_DTYPE_F16 0
#define BMXK_DTYPE_BF16 1
#define BMXK_DTYPE_F32 2

/* Geometry of a k2b cache (head dim is 128).  Mirrors the fields bmx reads off its specs:
 * bmx: src/bmx/cache/specs.py:82-91 and src/bmx/cache/packed_streaming.py:425-438. */
typedef struct bmxk_k2b_geom {
  int32_t h_kv;         /* KV heads */
  int32_t n_q_groups;   /* query heads per KV head, 1..8 */
  int32_t page;         /* tokens per page: 64 or 128 */
  int32_t rank;         /* low-rank key coefficients per token: 16 or 32 */
  int32_t group;        /* token group of the key-residual scale; divides page; 32, 64 or 128 */
  int32_t n_coef_heads; /* 1: one basis over all heads (bmx default); h_kv: one basis per head */
  int32_t kbits;        /* key-residual bits, 2..4 (stored as two's-complement nibbles) */
  int32_t vbits;        /* value code bits: 2 */
  int32_t layout;       /* byte order inside a page block (the exported tensors do not depend on it):
                           0 = per-lane fragment order, read by the mma.sync decode kernel (page 64 or 128);
                           1 = row order, read by the tcgen05 decode kernel (page 128 only) */
} bmxk_k2b_geom;

int bmxk_version(void);
const char* bmxk_last_error(void);

/* ---- bit packing ---------------------------------------------------------------------- */
/* bmx: src/bmx/cache/triton_dequant_attention.py:49-100 pack_codes / unpack_codes.
 * codes int16 (rows, C) with values in [0, 2^bits); packed uint8 (rows, C*bits/8); bits 2 or 4. */
int bmxk_pack_u(const int16_t* codes, uint8_t* packed, int64_t rows, int64_t C, int bits, void* stream);
int bmxk_unpack_u(const uint8_t* packed, int16_t* codes, int64_t rows, int64_t C, int bits, void* stream);
/* bmx: src/bmx/cache/triton_dequant_attention.py:103-165 pack_signed_codes / unpack_signed_codes.
 * codes int8 (rows, N), N even, values in the signed `bits` range; packed uint8 (rows, N/2). */
int bmxk_pack_s4(const int8_t* codes, uint8_t* packed, int64_t rows, int64_t N, int bits, void* stream);
int bmxk_unpack_s4(const uint8_t* packed, int8_t* codes, int64_t rows, int64_t N, int bits, void* stream);

/* ---- k2b page pool -------------------------------------------------------------------- */
/* Bytes of one (slot, head) page block and of one (slot, coef head) coefficient block.
 * Pool arrays are  pages[n_slots][h_kv][page_block_bytes]  and
 * coefs[n_slots][n_coef_heads][coef_block_bytes], both 16-byte aligned. */
size_t bmxk_k2b_page_block_bytes(const bmxk_k2b_geom* g);
size_t bmxk_k2b_coef_block_bytes(const bmxk_k2b_geom* g);

/* Quantize-on-append: packs n_seq * n_pages full pages.
 * bmx: src/bmx/cache/packed_streaming.py:475-580 (_pack_k_block, _pack_v_block) over
 *      src/bmx/cache/codecs.py:616-636, 677-695, 786-796 and src/bmx/quant/rtn.py:23-44.
 * k_pre, v: sources of dtype `src_dtype`, element (seq s, head h, token t, channel c) at
 *   base + s*stride_seq + h*stride_head + t*stride_tok + c  (elements); page p of a sequence
 *   covers tokens [p*page, (p+1)*page).  k_pre is the PRE-RoPE key.
 * basis_f32: (h_kv*128, rank) float32 frozen basis used for the projection Us = M @ V;
 *   for n_coef_heads == h_kv the projection of head h uses rows [h*128, (h+1)*128) only.
 * signs: 128 float32 (+1/-1) of the value rotation; codebook: 2^vbits float32 ascending levels.
 * slots: int32 [n_seq * n_pages] physical slot of each page (device memory). */
int bmxk_k2b_append(const bmxk_k2b_geom* g, const void* k_pre, const void* v, int src_dtype,
                    int64_t stride_seq, int64_t stride_head, int64_t stride_tok, const float* basis_f32,
                    const float* signs, const float* codebook, const int32_t* slots, int n_seq, int n_pages,
                    void* pages, void* coefs, void* stream);

/* The same append with the coefficients given instead of projected: us_f32 (n_seq, n_pages*page, rank) float32 = M @ V
 * over ALL heads of a basis that spans all heads (n_coef_heads must be 1), e.g. the sum over GPUs of the partial
 * projections of the heads each one holds (bmx projects on one device: src/bmx/cache/packed_streaming.py:513-520).
 * They are rounded to fp16 into the coefficient blocks; residual, scales, codes and values as in bmxk_k2b_append,
 * with basis_f32 = the rows of the basis that belong to THIS call's h_kv heads, (h_kv*128, rank). */
int bmxk_k2b_append_coefs(const bmxk_k2b_geom* g, const void* k_pre, const void* v, int src_dtype, int64_t stride_seq,
                          int64_t stride_head, int64_t stride_tok, const float* us_f32, const float* basis_f32,
                          const float* signs, const float* codebook, const int32_t* slots, int n_seq, int n_pages,
                          void* pages, void* coefs, void* stream);

/* Rewrites n pages into the exact tensors bmx's stack builder produces, for byte parity.
 * bmx: src/bmx/cache/triton_dequant_attention.py:1118-1229 build_kv_stacked_k2b(pack_k, pack_v).
 * us (n, n_coef_heads, page, rank) fp16; res_int_packed (n, h_kv*128, page/2) u8;
 * res_scale (n, h_kv*128, page/group) fp16; v_idx_packed (n, page, h_kv*128/4) u8;
 * v_norm (n, page, h_kv) fp16.  slots: int32[n] in device memory. */
int bmxk_k2b_export_stacks(const bmxk_k2b_geom* g, const void* pages, const void* coefs, const int32_t* slots,
                           int n, void* us, uint8_t* res_int_packed, void* res_scale, uint8_t* v_idx_packed,
                           void* v_norm, void* stream);

/* Dequantizes n pages to float32 (n, page, h_kv*128) pre-RoPE keys and values.
 * bmx: src/bmx/cache/codecs.py:799-842 dequant_packed (lowrank_rtn_channel, turboquant_mse_perhead).
 * basis_f16: (h_kv*128, rank) fp16 stored basis.  Either output may be NULL. */
int bmxk_k2b_dequant_pages(const bmxk_k2b_geom* g, const void* pages, const void* coefs, const void* basis_f16,
                           const float* signs, const float* codebook, const int32_t* slots, int n, float* k_out,
                           float* v_out, void* stream);

/* The dense prefill route's dequantizer: the first n_pages pages of `batch` sequences (page_table rows of table_stride
 * entries) -> keys rotated at their positions (float32 arithmetic, one rounding) and values, as fp16 or bf16
 * (out_dtype) written into (batch, h_kv, row_stride, 128) tensors at rows 0 .. n_pages*page - 1; the caller appends the
 * fp16 window behind them.  bmx: src/bmx/cache/chunked_attention.py:320-395 _prefill_dense_attention, which dequantizes
 * to float32, rotates and casts.  rope_cos / rope_sin: fp16 (positions, 128), both NULL for keys stored rotated.
 * Either output may be NULL. */
int bmxk_k2b_dequant_dense(const bmxk_k2b_geom* g, const void* pages, const void* coefs, const void* basis_f16,
                           const float* signs, const float* codebook, const int32_t* page_table, int table_stride,
                           int n_pages, int batch, const void* rope_cos, const void* rope_sin, int64_t pos_offset,
                           void* k_out, void* v_out, int64_t row_stride, int out_dtype, void* stream);

/* ---- k2b split-KV decode ---------------------------------------------------------------- */
/* Workspace (bytes) for a decode call over at most max_pages pages per sequence. */
size_t bmxk_k2b_decode_workspace_bytes(const bmxk_k2b_geom* g, int batch, int max_pages);

/* One decode step of dequant-attention for `batch` independent sequences.
 * bmx: src/bmx/cache/triton_dequant_attention.py:1232-1368 fused_decode_attention_k2b, with
 *      :324-360 _tail_partial and :409-461 _fused_merge_kernel folded in.
 * q: (batch, h_kv*n_q_groups, 128) fp16, already RoPE'd at the current position.
 * basis_f16: (h_kv*128, rank) fp16.  page_table: int32 (batch, table_stride) slot ids;
 * n_pages: int32 [batch] committed pages per sequence (device memory: the launch does not
 * depend on their values).  rope_cos/rope_sin: fp16 (>= max position, 128) tables as bmx keeps
 * them (bmx: src/bmx/cache/packed_streaming.py:94-113); a committed token at position t is
 * rotated at read.  k_tail/v_tail: fp16 (batch, h_kv, tail_cap, 128) recent window, keys
 * post-RoPE; tail_len: int32 [batch].  v_lut: 4 x uint32 in HOST memory {lo bytes, hi bytes,
 * alpha bits, beta bits} from bmxk_k2b_make_v_lut.  signs: 128 float32.  sm_scale: softmax scale.
 * out: (batch, h_kv*n_q_groups, 128), dtype out_dtype (F16 or F32).
 * If partial_out is non-NULL the merged but un-normalised state is written instead of `out`:
 * float32 (batch, heads, 130) = {max (log2 units), sum, 128 x accumulator}, for cross-GPU
 * sequence splits (merge with bmxk_merge_partials).
 * phases: 3 runs the whole step; 1 launches only the page-streaming kernel and 2 only the merge
 * kernel (same arguments), so that a caller can time them apart.
 * workspace: device memory of bmxk_k2b_decode_workspace_bytes(), zero-filled once by the caller
 * (its first 16 bytes are a status word that a kernel sets only if a bounded wait ran out). */
int bmxk_k2b_decode(const bmxk_k2b_geom* g, const void* q, const void* pages, const void* coefs,
                    const void* basis_f16, const int32_t* page_table, int table_stride, const int32_t* n_pages,
                    int batch, int max_pages, const void* rope_cos, const void* rope_sin, int64_t pos_offset,
                    const void* k_tail, const void* v_tail, const int32_t* tail_len, int tail_cap,
                    const uint32_t* v_lut, const float* signs, float sm_scale, void* workspace,
                    size_t workspace_bytes, void* out, int out_dtype, float* partial_out, int phases,
                    void* stream);

/* Causal attention of n_q new query positions per sequence over the committed pages and the fp16 window, without
 * building dense K / V for the context: each 128-token page is dequantized into shared memory and attended there.
 * bmx: src/bmx/cache/chunked_attention.py:320-395 _prefill_dense_attention (dequantize every page, then SDPA with the
 * causal mask), reached from chunked_dequant_attention(is_prefill=True) at :454-476.
 * q, out: fp16 (batch, heads, n_q, 128).  Query row i of every sequence sits at position q_pos0 + i; committed token t of
 * page j at pos_offset + 128 j + t, window slot r at pos_offset + 128 n_pages[s] + r; a key is visible to a query iff
 * its position is not larger.  Row-order pools (layout 1, 128-token pages) only.  status: device int32[4], zero on
 * entry (a bounded wait that ran out is reported there, see bmxk_check_workspace_status). */
int bmxk_k2b_prefill(const bmxk_k2b_geom* g, const void* q, int n_q, int64_t q_pos0, const void* pages, const void* coefs,
                     const void* basis_f16, const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch,
                     const void* rope_cos, const void* rope_sin, int64_t pos_offset, const void* k_tail, const void* v_tail,
                     const int32_t* tail_len, int tail_cap, const uint32_t* v_lut, const float* signs, float sm_scale,
                     int32_t* status, void* out, void* stream);

/* The same attention with the visible pages of every block of query positions shared out over n_split CTAs (1..64), which
 * write partial records into `workspace` (bmxk_k2b_prefill_workspace_bytes; 16-byte aligned device memory) for a merge
 * kernel launched behind them: for few query rows against a long context, where one CTA per block would walk every page
 * alone and most SMs would idle (bmx's split-KV decode kernels do the same for a single row:
 * src/bmx/cache/triton_dequant_attention.py:409-461).  n_split = 1 is bmxk_k2b_prefill; the split is the tcgen05 kernel's,
 * where the mma.sync kernel runs (q or out not 16-byte aligned, or selected) n_split is taken as 1. */
size_t bmxk_k2b_prefill_workspace_bytes(const bmxk_k2b_geom* g, int n_q, int batch, int n_split);
int bmxk_k2b_prefill_split(const bmxk_k2b_geom* g, const void* q, int n_q, int64_t q_pos0, const void* pages, const void* coefs,
                           const void* basis_f16, const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch,
                           const void* rope_cos, const void* rope_sin, int64_t pos_offset, const void* k_tail, const void* v_tail,
                           const int32_t* tail_len, int tail_cap, const uint32_t* v_lut, const float* signs, float sm_scale,
                           int32_t* status, void* out, int n_split, void* workspace, size_t workspace_bytes, void* stream);

/* Which kernel bmxk_k2b_prefill launches (process-wide; no counterpart in bmx).  0 (default): the tcgen05 kernel when q
 * and out are 16-byte aligned, else the mma.sync kernel; 1: always the mma.sync kernel.  Both give the same attention
 * within the path's tolerance. */
int bmxk_k2b_prefill_select(int kernel);

/* Decode step for hosts that must not allocate device memory.  (This entry point has no counterpart in
 * bmx; it exists for embedding.)
 *
 * Some hosts of this library cannot call cudaMalloc where they decode: an inference server that gave
 * every free byte of HBM to its KV-page pool at start-up has nothing left to carve a workspace from,
 * and a plugin loaded into another runtime's process may be forbidden to touch the CUDA allocator at
 * all.  bmxk_k2b_decode needs a caller-owned workspace for its per-CTA partial states; this variant
 * uses a scratch array that is part of the library image instead and takes no workspace argument.
 * Same arguments, same kernels and same results as bmxk_k2b_decode(..., phases = 3) with `out`.
 *
 * Limits and rules:
 *  - the scratch is BMXK_STATIC_SCRATCH_BYTES (2 MiB) per GPU, resident from the moment the library is
 *    loaded on that GPU until the process exits; a call whose
 *    bmxk_k2b_decode_workspace_bytes(g, batch, max_pages) exceeds it is rejected with
 *    BMXK_ERR_INVALID and a message naming both sizes.  With 148 SMs the limit in (sequence, KV head) pairs is
 *    (2 MiB - 256) / (n_sub * n_q_groups * 520) - 148, n_sub = 2 for layout 1 (the default for 128-token pages)
 *    and 1 for layout 0: layout 1 holds 356 pairs at 4 query heads per KV head and 104 at 8; layout 0 holds 860
 *    and 356;
 *  - the first call on each device looks up the scratch's device address (one cudaGetSymbolAddress,
 *    no allocation) with that device current; make that first call before any stream capture begins;
 *  - it calls no cudaMalloc / cudaFree and no allocating library routine; it issues one 256-byte
 *    cudaMemsetAsync on `stream` to clear the status word, because the scratch keeps the previous
 *    call's contents;
 *  - every call on a GPU shares the one scratch: two calls whose kernels overlap on that GPU (different
 *    streams, or different threads) race on it and produce garbage.  Serialise them, or give the
 *    concurrent ones bmxk_k2b_decode with their own workspaces. */
#define BMXK_STATIC_SCRATCH_BYTES (2 * 1024 * 1024)
int bmxk_k2b_decode_static(const bmxk_k2b_geom* g, const void* q, const void* pages, const void* coefs,
                           const void* basis_f16, const int32_t* page_table, int table_stride,
                           const int32_t* n_pages, int batch, int max_pages, const void* rope_cos,
                           const void* rope_sin, int64_t pos_offset, const void* k_tail, const void* v_tail,
                           const int32_t* tail_len, int tail_cap, const uint32_t* v_lut, const float* signs,
                           float sm_scale, void* out, int out_dtype, void* stream);
/* Status word of the built-in scratch on the current device (no counterpart in bmx).  The caller of
 * bmxk_k2b_decode_static holds no workspace pointer, so bmxk_check_workspace_status cannot serve it: this
 * reads the same four words from the built-in scratch (one 16-byte cudaMemcpyAsync on `stream` and a
 * synchronisation of `stream`; no allocation) and returns BMXK_ERR_DEVICE, with the site in bmxk_last_error(),
 * if a bounded wait of the last bmxk_k2b_decode_static call ran out.  The next call clears the word, so check
 * after the call whose result matters.  Before the first bmxk_k2b_decode_static call on a device: BMXK_OK. */
int bmxk_k2b_decode_static_status(void* stream);

/* Host helper: fp16 lookup table for the value codebook.  Picks four fp16 levels h_i and an
 * affine map so that codebook[i] = alpha + beta * h_i to ~1e-6, which lets the kernel feed
 * fp16 levels to the tensor cores without a systematic per-level rounding error.
 * out_lut[0] = low bytes of h_0..h_3, out_lut[1] = high bytes, out_lut[2] = alpha, [3] = beta
 * (float bit patterns). */
int bmxk_k2b_make_v_lut(const float* codebook, uint32_t* out_lut);

/* ---- plain RTN caches (bmx arms rtn_token / rtn_channel) -------------------------------- */
/* Geometry of an RTN cache (head dim 128).  Keys are post-RoPE.
 * bmx: src/bmx/cache/codecs.py:720-725, src/bmx/quant/rtn.py:23-53 (symmetric, no zero point). */
typedef struct bmxk_rtn_geom {
  int32_t h_kv;
  int32_t n_q_groups; /* 1..8 */
  int32_t page;       /* 64 or 128 */
  int32_t k_arm;      /* 0: rtn_token (groups of channels per token); 1: rtn_channel (groups of tokens per channel) */
  int32_t k_group;    /* 32, 64 or 128; for rtn_channel it must divide page */
  int32_t v_group;    /* value arm is rtn_token; 32, 64 or 128 */
  int32_t kbits;      /* 2..4, stored as two's-complement nibbles */
  int32_t vbits;      /* 2, stored as two's-complement 2-bit fields */
} bmxk_rtn_geom;

size_t bmxk_rtn_page_block_bytes(const bmxk_rtn_geom* g);   /* pool: pages[n_slots][h_kv][bytes] */
size_t bmxk_rtn_decode_workspace_bytes(const bmxk_rtn_geom* g, int batch, int max_pages);

/* Quantize-on-append of n_seq * n_pages full pages; sources addressed as in bmxk_k2b_append.
 * bmx: src/bmx/cache/packed_streaming.py:643-678 -> quantize_packed("rtn_token" | "rtn_channel"). */
int bmxk_rtn_append(const bmxk_rtn_geom* g, const void* k, const void* v, int src_dtype, int64_t stride_seq,
                    int64_t stride_head, int64_t stride_tok, const int32_t* slots, int n_seq, int n_pages,
                    void* pages, void* stream);

/* Rewrites n pages into bmx's containers and/or dequantizes them; any output may be NULL.
 * bmx: src/bmx/cache/triton_dequant_attention.py:1390-1451 build_kv_stacked_packed and
 *      src/bmx/cache/codecs.py:807-811 dequant_packed.
 * k_codes int8: rtn_token (n, h_kv, page, 128); rtn_channel (n, h_kv*128, page)   [Q_int of the block dict]
 * k_scales fp16: rtn_token (n, h_kv, page, 128/k_group); rtn_channel (n, h_kv*128, page/k_group)
 * v_codes int8 (n, h_kv, page, 128); v_scales fp16 (n, h_kv, page, 128/v_group)
 * k_deq, v_deq float32 (n, page, h_kv*128) = code * fp16 scale. */
int bmxk_rtn_export(const bmxk_rtn_geom* g, const void* pages, const int32_t* slots, int n, int8_t* k_codes,
                    void* k_scales, int8_t* v_codes, void* v_scales, float* k_deq, float* v_deq, void* stream);

/* One decode step over RTN pages + the fp16 window; arguments as in bmxk_k2b_decode.
 * bmx: src/bmx/cache/triton_dequant_attention.py:580-832 fused_decode_attention_packed (+ tail, merge). */
int bmxk_rtn_decode(const bmxk_rtn_geom* g, const void* q, const void* pages, const int32_t* page_table,
                    int table_stride, const int32_t* n_pages, int batch, int max_pages, const void* k_tail,
                    const void* v_tail, const int32_t* tail_len, int tail_cap, float sm_scale, void* workspace,
                    size_t workspace_bytes, void* out, int out_dtype, float* partial_out, void* stream);

/* ---- K4 spectral key codec, per-head packs ------------------------------------------------ */
/* bmx: src/bmx/cache/spectral.py:174-220 (SpectralPack), :631-645 (tier_columns), :703-839 (packed codec).
 * Each KV head has a 128 x 128 encoder and decoder and a bit width per encoded direction, a member of
 * {0, 2, 3, 4, 5, 6, 8}.  The page block of one (slot, head) holds, for every direction with bits, a row of
 * page codes in bmx's container for its tier (2/4 bits offset-binary, 3 bits in two's-complement nibbles,
 * 5/6/8 bits as int8) at byte offset col_off[head][direction], then float32 scales [direction][page/group]
 * at scale_off.  The host lays directions out by tier (bmx_b200.kernels.spectral_layout). */
typedef struct bmxk_spectral_geom {
  int32_t h_kv;
  int32_t page;        /* 64 or 128 */
  int32_t group;       /* token group of the scales; divides page */
  int32_t block_bytes; /* bytes of one (slot, head) page block, the same for every head */
  int32_t scale_off;   /* byte offset of the scales inside a block (multiple of 4) */
} bmxk_spectral_geom;

/* Quantize-on-append of pre-RoPE keys: Y = M @ enc, per-direction RTN with 10 step-refinement rounds.
 * bmx: spectral_quantize_packed(M, pack, mse_scale=True), src/bmx/cache/spectral.py:765-809.
 * enc: (h_kv, 128, 128) float32, enc[h][c][j]; col_bits, col_off: int32 (h_kv, 128) in device memory. */
int bmxk_spectral_append(const bmxk_spectral_geom* g, const void* k_pre, int src_dtype, int64_t stride_seq,
                         int64_t stride_head, int64_t stride_tok, const float* enc, const int32_t* col_bits,
                         const int32_t* col_off, const int32_t* slots, int n_seq, int n_pages, void* pages,
                         void* stream);

/* Unpacks and/or dequantizes n pages.  bmx: spectral_dequant_packed, src/bmx/cache/spectral.py:812-839.
 * codes int8 (n, h_kv, 128, page) signed levels per direction (0 for directions without bits);
 * scales float32 (n, h_kv, 128, page/group); k_out float32 (n, page, h_kv*128) = Y_hat @ dec^T with
 * dec (h_kv, 128, 128) float32, dec[h][c][j].  Any output may be NULL. */
int bmxk_spectral_dequant_pages(const bmxk_spectral_geom* g, const void* pages, const float* dec,
                                const int32_t* col_bits, const int32_t* col_off, const int32_t* slots, int n,
                                int8_t* codes, float* scales, float* k_out, void* stream);

/* Value-only page blocks, for caches whose keys live in a pool of their own (the spectral codec): the
 * per-head Hadamard + 2-bit Lloyd value codec of bmx (`turboquant_mse_perhead`, src/bmx/cache/codecs.py:616-636;
 * called per page from PackedStreamingLayer._pack_v_block, src/bmx/cache/packed_streaming.py:544-580).
 * One block per (slot, head), bmxk_vblock_bytes() = 4352 bytes: 2-bit codes of 128 tokens x 128 channels, then
 * 128 fp16 norms, ordered as the value part of a k2b page block of layout 1.  v: element (seq s, head h, token t,
 * channel c) at base + s*stride_seq + h*stride_head + t*stride_tok + c; slots: int32 (n_seq * n_pages). */
size_t bmxk_vblock_bytes(void);
int bmxk_vblock_append(int h_kv, const void* v, int src_dtype, int64_t stride_seq, int64_t stride_head, int64_t stride_tok,
                       const float* signs, const float* codebook, const int32_t* slots, int n_seq, int n_pages, void* vpages,
                       void* stream);
/* Blocks -> bmx's stacked containers: v_idx_packed uint8 (n, 128, h_kv*128/4), v_norm fp16 (n, 128, h_kv)
 * (bmx: build_kv_stacked_k2b, src/bmx/cache/triton_dequant_attention.py:1118-1229, pack_v=True). */
int bmxk_vblock_export(int h_kv, const void* vpages, const int32_t* slots, int n, uint8_t* v_idx_packed, void* v_norm,
                       void* stream);

/* One decode step over a spectral key pool + a value-block pool + the fp16 window, fused: the tier codes are
 * dequantized on chip, decoded (Y_hat @ dec^T on tcgen05.mma), rotated and attended without K_hat ever reaching
 * HBM.  bmx runs this codec pair through its chunked path (src/bmx/cache/packed_streaming.py:832-1064 attend ->
 * src/bmx/cache/chunked_attention.py:478-530 with _dequant_block :52-145 and spectral_dequant_packed,
 * src/bmx/cache/spectral.py:812-839); this entry point replaces that call for decode.
 * g: the key pool's geometry (page must be 128).  dec_f16: (h_kv, 128, 128) fp16, dec_f16[h][c][k] = dec[h][c][d_k]
 * with d_k the k-th direction of head h in tier order (directions with bits first, by ascending bits, then by
 * ascending index; directions without bits last).  meta: int32 (h_kv, 128), meta[h][k] = col_off[h][d_k] |
 * d_k << 16 | bits[h][d_k] << 24, and meta[h][0] also carries (ceil(max(used_h, 1) / 16) - 1) << 28, used_h being
 * the number of directions of head h that have bits: the decoder product runs over that many 16-direction steps
 * only.  Everything else as in
 * bmxk_k2b_decode; the workspace size comes from bmxk_spectral_decode_workspace_bytes. */
size_t bmxk_spectral_decode_workspace_bytes(const bmxk_spectral_geom* g, int n_q_groups, int batch);
int bmxk_spectral_decode(const bmxk_spectral_geom* g, int n_q_groups, const void* q, const void* kpages, const void* vpages,
                         const void* dec_f16, const int32_t* meta, const int32_t* page_table, int table_stride,
                         const int32_t* n_pages, int batch, int max_pages, const void* rope_cos, const void* rope_sin,
                         int64_t pos_offset, const void* k_tail, const void* v_tail, const int32_t* tail_len, int tail_cap,
                         const uint32_t* v_lut, const float* signs, float sm_scale, void* workspace, size_t workspace_bytes,
                         void* out, int out_dtype, float* partial_out, int phases, void* stream);

/* Merges n_parts partial states (n_parts, rows, 130) float32 -> out (rows, 128).
 * bmx: src/bmx/cache/triton_dequant_attention.py:409-461 _fused_merge_kernel (same formula,
 * max carried in log2 units). */
int bmxk_merge_partials(const float* parts, int n_parts, int rows, void* out, int out_dtype, void* stream);

/* The same merge across the GPUs of one node without a library collective (bmx has no multi-GPU path; the formula is
 * the split merge above).  Each rank owns an exchange buffer that every other rank maps (CUDA IPC); one kernel per
 * rank and step stores the rank's (rows, 130) state into its slot of EVERY rank's buffer (peer stores over NVLink),
 * raises a flag there, waits -- bounded by wait_limit_cycles -- until all ranks' flags of this step stand in its own
 * buffer, and merges from local memory into out (rows, 128).  No kernel loads from a peer and nothing is multicast.
 *   bmxk_xchg_alloc   allocates and zeroes this rank's buffer (cudaMalloc) and returns its 64-byte IPC handle;
 *   bmxk_xchg_open    maps a peer's buffer from its handle;  bmxk_xchg_close / bmxk_xchg_free undo the two.
 *   bmxk_xchg_merge   buffers: HOST array of `world` device pointers (index = rank, this rank's own included);
 *                     step: 1, 2, 3, ... the same on every rank, one call per step per rank, in order; or 0 = the step
 *                     after the last one this rank's buffer has completed (no per-step argument: the launch can sit in
 *                     a CUDA graph);
 *                     status: int32[4] in this rank's device memory, zero; a wait that runs out writes
 *                     {1, block, 32 + the rank that never arrived} there and the kernel returns without a result. */
size_t bmxk_xchg_bytes(int rows, int world);
int bmxk_xchg_alloc(int rows, int world, void** buffer, void* ipc_handle_64);
int bmxk_xchg_open(const void* ipc_handle_64, void** peer_buffer);
int bmxk_xchg_close(void* peer_buffer);
int bmxk_xchg_free(void* buffer);
int bmxk_xchg_merge(const float* part, int rows, int rank, int world, void* const* buffers, int step, int64_t wait_limit_cycles,
                    int32_t* status, void* out, int out_dtype, void* stream);

/* ---- recent window ------------------------------------------------------------------------ */
/* One decode step's new token into the fp16 window that precedes quantization.
 * bmx: src/bmx/cache/packed_streaming.py:582-628 (PackedStreamingLayer.update: the torch.cat of the new token
 * onto the fp16 tail tensors; here the window is preallocated and the token is written in place).
 * k_post (post-RoPE key, what attention over the window reads), v and k_src (the key the page quantizer will
 * read later: pre-RoPE for k2b) are sources of dtype `src_dtype` with element (seq s, head h, channel c) at
 * base + s*stride_seq + h*stride_head + c.  Windows are fp16 [batch][h_kv][tail_cap][128]; the token goes to
 * position t of every (sequence, head) and tail_len[s] becomes t + 1 (device int32[batch]). */
int bmxk_window_append(const void* k_post, const void* v, const void* k_src, int src_dtype, int64_t stride_seq,
                       int64_t stride_head, void* k_win, void* v_win, void* k_src_win, int32_t* tail_len, int batch,
                       int h_kv, int tail_cap, int t, void* stream);

/* The same append with the position read from tail_len[s] on the device (and advanced there), so that the launch
 * has no per-step argument and an (append, decode) pair can be captured once in a CUDA graph and replayed per
 * token.  counters: device int32[batch], zero before the first call and left zero by every call (the blocks of a
 * sequence count themselves there; the last one advances tail_len[s]).  A full window (tail_len[s] == tail_cap: the
 * host skipped a flush) writes nothing and sets *status to 2 when status is not NULL (the decode workspace's first
 * word: bmxk_check_workspace_status reports it). */
int bmxk_window_append_devpos(const void* k_post, const void* v, const void* k_src, int src_dtype, int64_t stride_seq,
                              int64_t stride_head, void* k_win, void* v_win, void* k_src_win, int32_t* tail_len,
                              int32_t* counters, int32_t* status, int batch, int h_kv, int tail_cap, void* stream);

/* After pages were committed out of the windows: the remaining tokens [off, off + rest) of every (sequence, head) move to
 * the front of the three windows in one launch, tail_len[s] becomes rest and, when n_pages is not NULL, n_pages[s] grows by
 * pages_added.  bmx slices its tail tensors instead (src/bmx/cache/packed_streaming.py:700-730).  k_src_win may be k_win. */
int bmxk_window_shift(void* k_win, void* v_win, void* k_src_win, int batch, int h_kv, int tail_cap, int off, int rest,
                      int32_t* tail_len, int32_t* n_pages, int pages_added, void* stream);

/* slots_out[s * n + i] = page_table[s][n_pages[s] + i]: the pool slots of the next n pages of every sequence, read on the
 * device (page counts are device-resident), so that a flush step -- token in, pages quantized out of the windows into
 * these slots, windows shifted, decode -- has no per-step argument and replays as a CUDA graph like any other step. */
int bmxk_gather_next_slots(const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch, int n,
                           int32_t* slots_out, void* stream);

/* A decode step's inputs in one launch (no counterpart in bmx, whose step starts from device tensors): the append of
 * bmxk_window_append_devpos for fp16 sources, plus the step's queries q_src (batch, h_kv*n_q_groups, 128) fp16 staged
 * into q_dst.  q_src, k_post, v and k_src may be PINNED HOST memory (cudaHostAlloc / torch pin_memory: mapped into the
 * device's address space): the kernel is then the host-to-device copy of the step.  Likewise the `out` of the decode
 * entry points may be pinned host memory: the merge kernel stores the result there directly. */
int bmxk_step_ingest(const void* q_src, void* q_dst, int n_q_groups, const void* k_post, const void* v, const void* k_src,
                     int64_t stride_seq, int64_t stride_head, void* k_win, void* v_win, void* k_src_win, int32_t* tail_len,
                     int32_t* counters, int32_t* status, int batch, int h_kv, int tail_cap, void* stream);


/* Reads back the status word of the last decode on this workspace (host-synchronising; for
 * tests and diagnostics).  Returns BMXK_ERR_DEVICE if a bounded wait ran out. */
int bmxk_check_workspace_status(const void* workspace, void* stream);

/* Self-test of the bounded device waits (no counterpart in bmx).  Every wait inside the decode kernels (on a bulk
 * copy, a tensor-core completion or another warp) gives up after a cycle limit, writes (1, block, site) to the status
 * word and lets the kernel end, so that a lost arrival costs an error code and not the GPU.  This launches one warp
 * that waits, with that same routine, on a barrier nothing ever arrives on; after `limit_cycles` (1e3 .. 2e8 SM
 * cycles, i.e. at most ~0.1 s) it must return with status = {1, 0, 77, 2}.  status: device int32[4], zeroed by the
 * caller; read it with bmxk_check_workspace_status, which must then return BMXK_ERR_DEVICE. */
int bmxk_selftest_bounded_wait(int32_t* status, int64_t limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BMXK_H_ */
