// Parameters shared by the two paged-prefill kernels (mma.sync and tcgen05) and the launcher of the second.
#pragma once
#include "decode_common.cuh"

namespace bmxk {

struct PrefillParams {
  K2bGeom g;
  const __half* q;
  int n_q;
  int64_t q_pos0;
  const uint8_t* pages;
  const __half* coefs;
  const __half* basis16;
  const int32_t* page_table;
  int table_stride;
  const int32_t* n_pages;
  const __half* rope_cos;
  const __half* rope_sin;
  int64_t pos_offset;
  const __half* k_tail;
  const __half* v_tail;
  const int32_t* tail_len;
  int tail_cap;
  uint32_t lut_lo, lut_hi;
  float lut_alpha, lut_beta;
  const float* signs;
  float scale_log2;
  __half* out;
  int32_t* status;
  // Split of the page range over CTAs (tcgen05 kernel only): n_split > 1 makes every CTA take one share of its block's
  // visible pages (the last share also the window) and write a partial record per row -- 128 accumulators, running
  // maximum (log2 units), sum of weights, 2 unused -- to `part`; prefill_merge_kernel combines them into `out`.
  int n_split;
  float* part;
};
constexpr int PF_PART_STRIDE = 132;  // floats per (row, share) record: 16-byte aligned rows

// tcgen05 prefill kernel (k2b_prefill_t5.cu); the mma.sync kernel's grid with x multiplied by n_split.  Needs q, out and the
// window 16-byte aligned.  With n_split > 1 the merge kernel is launched behind it.
int launch_prefill_t5(const PrefillParams& prm, dim3 grid, cudaStream_t s);

}  // namespace bmxk
