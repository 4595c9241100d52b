// Library plumbing (version, last-error string, launch check) and the standalone bit-packing
// kernels of the C ABI.
#include <cstdarg>
#include <cstring>

#include "common.cuh"

namespace bmxk {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return BMXK_ERR_CUDA;
  }
  return BMXK_OK;
}

// One thread per output byte.  Unsigned codes, 8/bits per byte, code c at bit bits*(c % per_byte).
__global__ void pack_u_kernel(const int16_t* __restrict__ codes, uint8_t* __restrict__ packed, int64_t n_bytes,
                              int bits) {
  const int per = 8 / bits;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_bytes; i += (int64_t)gridDim.x * blockDim.x) {
    uint32_t b = 0;
    for (int k = 0; k < per; ++k) b |= (uint32_t)((uint8_t)codes[i * per + k]) << (bits * k);
    packed[i] = (uint8_t)b;
  }
}
__global__ void unpack_u_kernel(const uint8_t* __restrict__ packed, int16_t* __restrict__ codes, int64_t n_bytes,
                                int bits) {
  const int per = 8 / bits;
  const uint32_t mask = (1u << bits) - 1u;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_bytes; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t b = packed[i];
    for (int k = 0; k < per; ++k) codes[i * per + k] = (int16_t)((b >> (bits * k)) & mask);
  }
}
// Signed codes as two's-complement nibbles, low nibble first.
__global__ void pack_s4_kernel(const int8_t* __restrict__ codes, uint8_t* __restrict__ packed, int64_t n_bytes) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_bytes; i += (int64_t)gridDim.x * blockDim.x) {
    const uint32_t lo = (uint32_t)codes[2 * i] & 0xF, hi = (uint32_t)codes[2 * i + 1] & 0xF;
    packed[i] = (uint8_t)(lo | (hi << 4));
  }
}
__global__ void unpack_s4_kernel(const uint8_t* __restrict__ packed, int8_t* __restrict__ codes, int64_t n_bytes) {
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n_bytes; i += (int64_t)gridDim.x * blockDim.x) {
    const int b = packed[i];
    codes[2 * i] = (int8_t)(((b & 0xF) ^ 8) - 8);
    codes[2 * i + 1] = (int8_t)((((b >> 4) & 0xF) ^ 8) - 8);
  }
}

static inline int grid_for(int64_t n, int block) {
  int64_t g = (n + block - 1) / block;
  const int64_t cap = 148 * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace bmxk

using namespace bmxk;

namespace bmxk {

constexpr int WIN_HEAD_DIM = 128;

// One decode step's new token into the fp16 recent window: post-RoPE key, value and the page-source key of every
// (sequence, head) at position t, and the window length t + 1 for every sequence.  One block per (sequence, head).
template <typename T>
__global__ void window_append_kernel(const T* __restrict__ k_post, const T* __restrict__ v, const T* __restrict__ k_src,
                                     int64_t stride_seq, int64_t stride_head, __half* __restrict__ k_win,
                                     __half* __restrict__ v_win, __half* __restrict__ k_src_win, int32_t* __restrict__ tail_len,
                                     int h_kv, int tail_cap, int t) {
  const int bh = blockIdx.x, b = bh / h_kv, h = bh % h_kv, c = threadIdx.x;
  const int64_t src = (int64_t)b * stride_seq + (int64_t)h * stride_head + c;
  const int64_t dst = ((int64_t)bh * tail_cap + t) * WIN_HEAD_DIM + c;
  k_win[dst] = __float2half_rn(load_as_float<T>(k_post + src));
  v_win[dst] = __float2half_rn(load_as_float<T>(v + src));
  k_src_win[dst] = __float2half_rn(load_as_float<T>(k_src + src));
  if (h == 0 && c == 0) tail_len[b] = t + 1;
}

// The same append with the position taken from device memory: every block (one per sequence and head) reads
// tail_len[b] and writes its head's token there; the block of a sequence that finishes last (a per-sequence
// counter tells) advances tail_len[b] and clears the counter, so no block can read the new position.  Nothing in the
// launch depends on the step, so a captured CUDA graph of (append, decode) can be replayed token after token.
template <typename T>
__global__ void window_append_devpos_kernel(const T* __restrict__ k_post, const T* __restrict__ v, const T* __restrict__ k_src,
                                            int64_t stride_seq, int64_t stride_head, __half* __restrict__ k_win,
                                            __half* __restrict__ v_win, __half* __restrict__ k_src_win,
                                            int32_t* __restrict__ tail_len, int32_t* __restrict__ counters,
                                            int32_t* __restrict__ status, int h_kv, int tail_cap) {
  const int bh = blockIdx.x, b = bh / h_kv, h = bh % h_kv, c = threadIdx.x;
  const int t = *reinterpret_cast<volatile int32_t*>(tail_len + b);
  if (t >= 0 && t < tail_cap) {
    const int64_t src = (int64_t)b * stride_seq + (int64_t)h * stride_head + c;
    const int64_t dst = ((int64_t)bh * tail_cap + t) * WIN_HEAD_DIM + c;
    k_win[dst] = __float2half_rn(load_as_float<T>(k_post + src));
    v_win[dst] = __float2half_rn(load_as_float<T>(v + src));
    k_src_win[dst] = __float2half_rn(load_as_float<T>(k_src + src));
  } else if (c == 0 && status) {
    atomicCAS(status, 0, 2);  // the window is full: the host should have flushed; report instead of writing outside
  }
  __syncthreads();  // every thread of this block has read the position
  if (c == 0) {
    __threadfence();
    if (atomicAdd(counters + b, 1) == h_kv - 1) {  // all blocks of the sequence have read the position
      counters[b] = 0;
      if (t >= 0 && t < tail_cap) tail_len[b] = t + 1;
    }
  }
}

// A decode step's inputs in one launch: the new token goes into the windows as in window_append_devpos_kernel, and the
// step's queries are staged into device memory (block (sequence, kv head) copies the n_q_groups query rows of its head).
// The sources may be pinned host memory mapped into the device's address space: the kernel then IS the host-to-device
// copy of the step (a few KB per block over PCIe), which saves the copy engine's separate launch.
__global__ void step_ingest_kernel(const __half* __restrict__ q_src, __half* __restrict__ q_dst, int n_q_groups,
                                   const __half* __restrict__ k_post, const __half* __restrict__ v, const __half* __restrict__ k_src,
                                   int64_t stride_seq, int64_t stride_head, __half* __restrict__ k_win, __half* __restrict__ v_win,
                                   __half* __restrict__ k_src_win, int32_t* __restrict__ tail_len, int32_t* __restrict__ counters,
                                   int32_t* __restrict__ status, int h_kv, int tail_cap) {
  const int bh = blockIdx.x, b = bh / h_kv, h = bh % h_kv, c = threadIdx.x;
  const int t = *reinterpret_cast<volatile int32_t*>(tail_len + b);
  const int64_t src = (int64_t)b * stride_seq + (int64_t)h * stride_head + c;
  // all loads first (they cross PCIe when the sources are host memory), then the stores
  const __half kp = k_post[src], vv = v[src], ks = k_src[src];
  __half qv[8];
  for (int g = 0; g < n_q_groups; ++g) qv[g] = q_src[((int64_t)bh * n_q_groups + g) * WIN_HEAD_DIM + c];
  for (int g = 0; g < n_q_groups; ++g) q_dst[((int64_t)bh * n_q_groups + g) * WIN_HEAD_DIM + c] = qv[g];
  if (t >= 0 && t < tail_cap) {
    const int64_t dst = ((int64_t)bh * tail_cap + t) * WIN_HEAD_DIM + c;
    k_win[dst] = kp, v_win[dst] = vv, k_src_win[dst] = ks;
  } else if (c == 0 && status) {
    atomicCAS(status, 0, 2);
  }
  __syncthreads();
  if (c == 0) {
    __threadfence();
    if (atomicAdd(counters + b, 1) == h_kv - 1) {
      counters[b] = 0;
      if (t >= 0 && t < tail_cap) tail_len[b] = t + 1;
    }
  }
}

// After a flush: the tokens [off, off + rest) of every (sequence, head) window move to the front, the device-side window
// length becomes `rest` and the device-side page count grows by `pages_added`.  One block per (sequence, head); the move
// goes forward in chunks of 2048 elements, each read completely before it is written (source and destination overlap
// when rest > off).  k_src_win may alias k_win (caches that quantize post-RoPE keys): it is then moved once.
__global__ void window_shift_kernel(__half* __restrict__ k_win, __half* __restrict__ v_win, __half* __restrict__ k_src_win, int tail_cap,
                                    int off, int rest, int h_kv, int32_t* __restrict__ tail_len, int32_t* __restrict__ n_pages,
                                    int pages_added) {
  const int bh = blockIdx.x, tid = threadIdx.x;
  __half* bufs[3] = {k_win, v_win, (k_src_win == k_win) ? nullptr : k_src_win};
  const int total = rest * WIN_HEAD_DIM;  // elements to move per window; a multiple of 8
  for (int w = 0; w < 3; ++w) {
    if (!bufs[w]) continue;
    uint4* base = reinterpret_cast<uint4*>(bufs[w] + (int64_t)bh * tail_cap * WIN_HEAD_DIM);
    const int shift4 = off * WIN_HEAD_DIM / 8, n4 = total / 8;
    for (int c0 = 0; c0 < n4; c0 += 256) {
      const int i = c0 + tid;
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (i < n4) x = base[shift4 + i];
      __syncthreads();  // the whole chunk is in registers before any of it is overwritten
      if (i < n4) base[i] = x;
      __syncthreads();
    }
  }
  if (tid == 0 && bh % h_kv == 0) {
    const int b = bh / h_kv;
    tail_len[b] = rest;
    if (n_pages) n_pages[b] += pages_added;
  }
}

// slots_out[b * n + i] = page_table[b][n_pages[b] + i]: the slots of the next n pages of every sequence, looked up on the
// device so that a captured flush step needs no per-step argument.
__global__ void gather_next_slots_kernel(const int32_t* __restrict__ page_table, int table_stride, const int32_t* __restrict__ n_pages,
                                         int batch, int n, int32_t* __restrict__ slots_out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < batch * n) {
    const int b = i / n, j = i % n;
    slots_out[i] = page_table[(int64_t)b * table_stride + n_pages[b] + j];
  }
}

}  // namespace bmxk

extern "C" {

int bmxk_version(void) { return 100; }
const char* bmxk_last_error(void) { return g_err; }

int bmxk_pack_u(const int16_t* codes, uint8_t* packed, int64_t rows, int64_t C, int bits, void* stream) {
  BMXK_REQUIRE(bits == 2 || bits == 4, "bmxk_pack_u: bits must be 2 or 4 (got %d)", bits);
  BMXK_REQUIRE(rows >= 0 && C >= 0 && C % (8 / bits) == 0, "bmxk_pack_u: C=%lld must be a multiple of %d",
               (long long)C, 8 / bits);
  const int64_t n = rows * C * bits / 8;
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(codes && packed, "bmxk_pack_u: null pointer");
  pack_u_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(codes, packed, n, bits);
  return check_launch("bmxk_pack_u");
}
int bmxk_unpack_u(const uint8_t* packed, int16_t* codes, int64_t rows, int64_t C, int bits, void* stream) {
  BMXK_REQUIRE(bits == 2 || bits == 4, "bmxk_unpack_u: bits must be 2 or 4 (got %d)", bits);
  BMXK_REQUIRE(rows >= 0 && C >= 0 && C % (8 / bits) == 0, "bmxk_unpack_u: C=%lld must be a multiple of %d",
               (long long)C, 8 / bits);
  const int64_t n = rows * C * bits / 8;
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(codes && packed, "bmxk_unpack_u: null pointer");
  unpack_u_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(packed, codes, n, bits);
  return check_launch("bmxk_unpack_u");
}
int bmxk_pack_s4(const int8_t* codes, uint8_t* packed, int64_t rows, int64_t N, int bits, void* stream) {
  BMXK_REQUIRE(bits >= 1 && bits <= 4, "bmxk_pack_s4: bits must be in [1,4] (got %d)", bits);
  BMXK_REQUIRE(rows >= 0 && N >= 0 && N % 2 == 0, "bmxk_pack_s4: N=%lld must be even", (long long)N);
  const int64_t n = rows * N / 2;
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(codes && packed, "bmxk_pack_s4: null pointer");
  pack_s4_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(codes, packed, n);
  return check_launch("bmxk_pack_s4");
}
int bmxk_unpack_s4(const uint8_t* packed, int8_t* codes, int64_t rows, int64_t N, int bits, void* stream) {
  BMXK_REQUIRE(bits >= 1 && bits <= 4, "bmxk_unpack_s4: bits must be in [1,4] (got %d)", bits);
  BMXK_REQUIRE(rows >= 0 && N >= 0 && N % 2 == 0, "bmxk_unpack_s4: N=%lld must be even", (long long)N);
  const int64_t n = rows * N / 2;
  if (n == 0) return BMXK_OK;
  BMXK_REQUIRE(codes && packed, "bmxk_unpack_s4: null pointer");
  unpack_s4_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(packed, codes, n);
  return check_launch("bmxk_unpack_s4");
}

int bmxk_window_append(const void* k_post, const void* v, const void* k_src, int src_dtype, int64_t stride_seq,
                       int64_t stride_head, void* k_win, void* v_win, void* k_src_win, int32_t* tail_len, int batch,
                       int h_kv, int tail_cap, int t, void* stream) {
  BMXK_REQUIRE(k_post && v && k_src && k_win && v_win && k_src_win && tail_len, "bmxk_window_append: null pointer");
  BMXK_REQUIRE(batch >= 1 && h_kv >= 1 && tail_cap >= 1, "bmxk_window_append: batch=%d h_kv=%d tail_cap=%d", batch, h_kv, tail_cap);
  BMXK_REQUIRE(t >= 0 && t < tail_cap, "bmxk_window_append: position %d outside the window of %d tokens", t, tail_cap);
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = batch * h_kv;
  if (src_dtype == BMXK_DTYPE_F16)
    window_append_kernel<__half><<<grid, WIN_HEAD_DIM, 0, s>>>((const __half*)k_post, (const __half*)v, (const __half*)k_src, stride_seq,
                                                            stride_head, (__half*)k_win, (__half*)v_win, (__half*)k_src_win, tail_len,
                                                            h_kv, tail_cap, t);
  else if (src_dtype == BMXK_DTYPE_BF16)
    window_append_kernel<__nv_bfloat16><<<grid, WIN_HEAD_DIM, 0, s>>>((const __nv_bfloat16*)k_post, (const __nv_bfloat16*)v,
                                                                   (const __nv_bfloat16*)k_src, stride_seq, stride_head, (__half*)k_win,
                                                                   (__half*)v_win, (__half*)k_src_win, tail_len, h_kv, tail_cap, t);
  else if (src_dtype == BMXK_DTYPE_F32)
    window_append_kernel<float><<<grid, WIN_HEAD_DIM, 0, s>>>((const float*)k_post, (const float*)v, (const float*)k_src, stride_seq,
                                                          stride_head, (__half*)k_win, (__half*)v_win, (__half*)k_src_win, tail_len, h_kv,
                                                          tail_cap, t);
  else
    BMXK_REQUIRE(false, "bmxk_window_append: src_dtype=%d", src_dtype);
  return check_launch("bmxk_window_append");
}

int bmxk_window_append_devpos(const void* k_post, const void* v, const void* k_src, int src_dtype, int64_t stride_seq,
                              int64_t stride_head, void* k_win, void* v_win, void* k_src_win, int32_t* tail_len, int32_t* counters,
                              int32_t* status, int batch, int h_kv, int tail_cap, void* stream) {
  BMXK_REQUIRE(k_post && v && k_src && k_win && v_win && k_src_win && tail_len && counters, "bmxk_window_append_devpos: null pointer");
  BMXK_REQUIRE(batch >= 1 && h_kv >= 1 && tail_cap >= 1, "bmxk_window_append_devpos: batch=%d h_kv=%d tail_cap=%d", batch, h_kv, tail_cap);
  cudaStream_t s = (cudaStream_t)stream;
  if (src_dtype == BMXK_DTYPE_F16)
    window_append_devpos_kernel<__half><<<batch * h_kv, WIN_HEAD_DIM, 0, s>>>((const __half*)k_post, (const __half*)v, (const __half*)k_src,
                                                                     stride_seq, stride_head, (__half*)k_win, (__half*)v_win,
                                                                     (__half*)k_src_win, tail_len, counters, status, h_kv, tail_cap);
  else if (src_dtype == BMXK_DTYPE_BF16)
    window_append_devpos_kernel<__nv_bfloat16><<<batch * h_kv, WIN_HEAD_DIM, 0, s>>>((const __nv_bfloat16*)k_post, (const __nv_bfloat16*)v,
                                                                            (const __nv_bfloat16*)k_src, stride_seq, stride_head,
                                                                            (__half*)k_win, (__half*)v_win, (__half*)k_src_win, tail_len,
                                                                            counters, status, h_kv, tail_cap);
  else if (src_dtype == BMXK_DTYPE_F32)
    window_append_devpos_kernel<float><<<batch * h_kv, WIN_HEAD_DIM, 0, s>>>((const float*)k_post, (const float*)v, (const float*)k_src,
                                                                   stride_seq, stride_head, (__half*)k_win, (__half*)v_win,
                                                                   (__half*)k_src_win, tail_len, counters, status, h_kv, tail_cap);
  else
    BMXK_REQUIRE(false, "bmxk_window_append_devpos: src_dtype=%d", src_dtype);
  return check_launch("bmxk_window_append_devpos");
}

int bmxk_step_ingest(const void* q_src, void* q_dst, int n_q_groups, const void* k_post, const void* v, const void* k_src,
                     int64_t stride_seq, int64_t stride_head, void* k_win, void* v_win, void* k_src_win, int32_t* tail_len,
                     int32_t* counters, int32_t* status, int batch, int h_kv, int tail_cap, void* stream) {
  BMXK_REQUIRE(q_src && q_dst && k_post && v && k_src && k_win && v_win && k_src_win && tail_len && counters, "bmxk_step_ingest: null pointer");
  BMXK_REQUIRE(batch >= 1 && h_kv >= 1 && tail_cap >= 1 && n_q_groups >= 1 && n_q_groups <= 8,
               "bmxk_step_ingest: batch=%d h_kv=%d tail_cap=%d n_q_groups=%d", batch, h_kv, tail_cap, n_q_groups);
  step_ingest_kernel<<<batch * h_kv, WIN_HEAD_DIM, 0, (cudaStream_t)stream>>>(
      (const __half*)q_src, (__half*)q_dst, n_q_groups, (const __half*)k_post, (const __half*)v, (const __half*)k_src, stride_seq, stride_head,
      (__half*)k_win, (__half*)v_win, (__half*)k_src_win, tail_len, counters, status, h_kv, tail_cap);
  return check_launch("bmxk_step_ingest");
}

int bmxk_window_shift(void* k_win, void* v_win, void* k_src_win, int batch, int h_kv, int tail_cap, int off, int rest,
                      int32_t* tail_len, int32_t* n_pages, int pages_added, void* stream) {
  BMXK_REQUIRE(k_win && v_win && k_src_win && tail_len, "bmxk_window_shift: null pointer");
  BMXK_REQUIRE(batch >= 1 && h_kv >= 1 && tail_cap >= 1 && off >= 0 && rest >= 0 && off + rest <= tail_cap,
               "bmxk_window_shift: batch=%d h_kv=%d tail_cap=%d off=%d rest=%d", batch, h_kv, tail_cap, off, rest);
  window_shift_kernel<<<batch * h_kv, 256, 0, (cudaStream_t)stream>>>((__half*)k_win, (__half*)v_win, (__half*)k_src_win, tail_cap, off, rest,
                                                                     h_kv, tail_len, n_pages, pages_added);
  return check_launch("bmxk_window_shift");
}

int bmxk_gather_next_slots(const int32_t* page_table, int table_stride, const int32_t* n_pages, int batch, int n, int32_t* slots_out,
                           void* stream) {
  BMXK_REQUIRE(page_table && n_pages && slots_out, "bmxk_gather_next_slots: null pointer");
  BMXK_REQUIRE(batch >= 1 && n >= 1 && table_stride >= n, "bmxk_gather_next_slots: batch=%d n=%d table_stride=%d", batch, n, table_stride);
  gather_next_slots_kernel<<<(batch * n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(page_table, table_stride, n_pages, batch, n, slots_out);
  return check_launch("bmxk_gather_next_slots");
}

}  // extern "C"
