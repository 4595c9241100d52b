// Pieces shared by the split-KV decode kernels (k2b and RTN): the flat tile decomposition, the cursor
// that walks it, the partial-state record and the merge kernel's parameters.
#pragma once
#include "common.cuh"

namespace bmxk {

constexpr int TILE_TOKENS = 128;
constexpr int PART_STRIDE = 130;  // per query head: max (log2 units), sum, 128 accumulators
constexpr int MAX_BH = 4096;      // (sequence, head) pairs per call

// Tiles per (sequence, head) and the flat decomposition, recomputed identically by every CTA of both
// kernels from the device-resident page counts.
__device__ __forceinline__ int tiles_of(int n_pages, int page) { return (n_pages * page + TILE_TOKENS - 1) / TILE_TOKENS; }

// cum[b] = tiles of sequences < b, times h_kv.  Filled by one warp; cum has batch + 1 entries.
__device__ __forceinline__ void fill_cum(int* cum, const int32_t* n_pages, int batch, int h_kv, int page, int lane) {
  int run = 0;
  for (int b0 = 0; b0 < batch; b0 += 32) {
    const int b = b0 + lane;
    int v = (b < batch) ? tiles_of(n_pages[b], page) * h_kv : 0;
    int incl = v;
#pragma unroll
    for (int m = 1; m < 32; m <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, m);
      if (lane >= m) incl += o;
    }
    if (b < batch) cum[b] = run + incl - v;
    run += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) cum[batch] = run;
}

// Walks the flat tile list without divisions: (sequence b, head h, tile j of tiles_b) advance by one.
struct TileCursor {
  int b, h, j, tiles_b;
  __device__ __forceinline__ void init(const int* cum, const int* npg, int f, int page) {
    b = 0;
    while (cum[b + 1] <= f) ++b;
    tiles_b = tiles_of(npg[b], page);
    const int rel = f - cum[b];
    h = rel / tiles_b, j = rel - h * tiles_b;
  }
  __device__ __forceinline__ void next(const int* npg, int h_kv, int page, int batch) {
    if (++j == tiles_b) {
      j = 0;
      if (++h == h_kv) {
        h = 0;
        do { ++b; } while (b < batch && npg[b] == 0);
        tiles_b = (b < batch) ? tiles_of(npg[b], page) : 1;
      }
    }
  }
};

struct K2bMergeParams {
  K2bGeom g;
  const __half* q;
  const int32_t* n_pages;
  int batch;
  int main_grid;
  const float* part;
  const __half* k_tail;
  const __half* v_tail;
  const int32_t* tail_len;
  int tail_cap;
  const float* signs;
  float scale_log2;
  void* out;
  int out_dtype;
  float* partial_out;
  int n_sub;  // partial records per (CTA, sequence, head): record of sub s sits s*(main_grid + batch*h_kv) slots further
};

struct K2bDecodeParams {
  K2bGeom g;
  const __half* q;
  const uint8_t* pages;
  const __half* coefs;
  const __half* basis16;
  const int32_t* page_table;
  int table_stride;
  const int32_t* n_pages;
  int batch;
  const __half* rope_cos;
  const __half* rope_sin;
  int64_t pos_offset;
  uint32_t lut_lo, lut_hi;
  float lut_alpha, lut_beta;
  float scale_log2;  // softmax scale * log2(e)
  float* part;       // (grid + batch*h_kv, n_q_groups, PART_STRIDE)
  int32_t* status;
  int n_stages;
};

constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // ~2 s at 2 GHz

__device__ __forceinline__ bool wait_or_flag(uint64_t* bar, uint32_t parity, int32_t* status, int where,
                                             long long limit = WAIT_LIMIT_CYCLES) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  // try_wait parks the warp for a hardware-chosen time per poll; the error flag and the clock are looked at
  // once in a while only.
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 255u) == 0u) {
      if (*reinterpret_cast<volatile int32_t*>(status) != 0) return false;  // another wait already gave up
      if (clock64() - t0 > limit) {  // a copy or an arrival was lost; report and leave
        if (atomicCAS(status, 0, 1) == 0) {
          status[1] = blockIdx.x;
          status[2] = where;
        }
        return false;
      }
    }
  }
}

// The same bounded wait for a warp whose wake-up latency sits on the critical path (the issuing warp of the
// tcgen05 kernel): it spins on the non-blocking test instead of parking.
__device__ __forceinline__ bool spin_or_flag(uint64_t* bar, uint32_t parity, int32_t* status, int where) {
  if (mbar_test_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t spin = 1;; ++spin) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((spin & 1023u) == 0u) {
      if (*reinterpret_cast<volatile int32_t*>(status) != 0) return false;
      if (clock64() - t0 > 4000000000LL) {
        if (atomicCAS(status, 0, 1) == 0) {
          status[1] = blockIdx.x;
          status[2] = where;
        }
        return false;
      }
    }
  }
}

// SM count of the current device (cached) and the launcher of the merge kernel (defined in k2b_decode.cu).
int num_sms();
// `after_main`: the page-streaming kernel of the same step was launched just before on the same stream.  The merge
// kernel is then launched as its programmatic dependent: its blocks may start while that kernel drains, attend over
// the fp16 window (which that kernel does not write) and wait for it only before they read the partial states.
int launch_merge(const K2bMergeParams& mp, cudaStream_t s, bool after_main = false);
// tcgen05 decode kernel for layout-1 pools (k2b_decode_t5.cu); two partial records per slot (one per tile parity)
int launch_decode_t5(const K2bDecodeParams& prm, int grid, cudaStream_t s);

}  // namespace bmxk
