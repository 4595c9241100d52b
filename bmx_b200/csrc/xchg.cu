// Cross-GPU merge of split-sequence partial states without a library collective.
//
// A sequence whose pages are split across the GPUs of one node ends a decode step with one small exchange: every
// rank holds (rows x 130) floats -- per query head the running maximum, the sum and the 128 accumulators of ITS pages
// -- and every rank needs the merge of all of them (bmx's split merge, src/bmx/cache/triton_dequant_attention.py
// :409-461, applied across ranks).  One kernel per rank does the exchange and the merge:
//
//   push   each block stores its rows of the local state into slot `rank` of EVERY rank's exchange buffer (plain
//          peer stores over NVLink; the own buffer is a local store), then a system-scope fence;
//   flag   the last block to finish raises flag[rank] = step in every rank's buffer (release, system scope);
//   wait   every block polls the `world` flags of its OWN buffer (acquire, system scope) until all carry this step;
//          the wait is bounded: past the limit it records (block, site) in the status word and the kernel returns;
//   merge  every block merges its rows from the own buffer: local loads only.
//
// No kernel ever loads from another GPU's memory, nothing is multicast, and no rank's kernel waits for another
// launch on its own GPU.  Buffers alternate by step parity: rank A can only be one step ahead of rank B (its step
// s+1 kernel needs B's flag s+1, which B raises after its step s kernel has ended), so slot parity (s+2)&1 is never
// written while somebody still reads step s.
#include <cuda_runtime.h>

#include <cstring>

#include "common.cuh"
#include "decode_common.cuh"

namespace bmxk {

namespace {

constexpr int XCHG_MAX_WORLD = 16;
constexpr int XCHG_THREADS = 128;

struct XchgParams {
  const float* part;   // (rows, 130) local partial state
  int rows, rank, world, step;
  uint8_t* bufs[XCHG_MAX_WORLD];  // every rank's exchange buffer as mapped into this process
  long long limit;
  int32_t* status;
  void* out;
  int out_dtype;
};

__host__ __device__ inline size_t xchg_data_floats(int rows, int world) { return (size_t)2 * world * rows * PART_STRIDE; }
__host__ __device__ inline size_t xchg_flag_off(int rows, int world) { return (xchg_data_floats(rows, world) * sizeof(float) + 127) / 128 * 128; }
// flags: int32 [2][XCHG_MAX_WORLD], then local words: the push counters int32 [2], the count of blocks that have ended,
// and the number of the last step this rank completed
__host__ __device__ inline size_t xchg_total_bytes(int rows, int world) { return xchg_flag_off(rows, world) + (2 * XCHG_MAX_WORLD + 4) * sizeof(int32_t) + 112; }

__device__ __forceinline__ void st_release_sys(int32_t* p, int32_t v) { asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int32_t ld_acquire_sys(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(XCHG_THREADS) xchg_merge_kernel(const XchgParams p) {
  __shared__ int ok_sm;
  const int t = threadIdx.x;
  const size_t slot = (size_t)p.rows * PART_STRIDE;
  uint8_t* own = p.bufs[p.rank];
  int32_t* own_flags = reinterpret_cast<int32_t*>(own + xchg_flag_off(p.rows, p.world));
  int32_t* ended = own_flags + 2 * XCHG_MAX_WORLD + 2;
  int32_t* last_step = own_flags + 2 * XCHG_MAX_WORLD + 3;
  // step 0 = "the step after the last one this rank completed", kept in the buffer: a launch without a per-step
  // argument, which a CUDA graph can replay
  const int step = p.step > 0 ? p.step : *reinterpret_cast<volatile int32_t*>(last_step) + 1;
  const int parity = step & 1;
  int32_t* counter = own_flags + 2 * XCHG_MAX_WORLD + parity;
  if (t == 0) ok_sm = 1;

  // ---- push: my rows into slot `rank` of every rank's buffer ----
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    const float* src = p.part + (size_t)row * PART_STRIDE;
    const float a = src[t];
    const float b = (t < PART_STRIDE - XCHG_THREADS) ? src[XCHG_THREADS + t] : 0.f;
    for (int r = 0; r < p.world; ++r) {
      float* dst = reinterpret_cast<float*>(p.bufs[r]) + ((size_t)parity * p.world + p.rank) * slot + (size_t)row * PART_STRIDE;
      dst[t] = a;
      if (t < PART_STRIDE - XCHG_THREADS) dst[XCHG_THREADS + t] = b;
    }
  }
  __threadfence_system();
  __syncthreads();
  // ---- flag: the last block to get here publishes the whole state on every rank ----
  if (t == 0) {
    const int prev = atomicAdd(counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *counter = 0;  // next used two steps from now, after this kernel has ended
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        st_release_sys(reinterpret_cast<int32_t*>(p.bufs[r] + xchg_flag_off(p.rows, p.world)) + parity * XCHG_MAX_WORLD + p.rank, step);
    }
  }
  // ---- wait: all ranks' flags in my own buffer ----
  if (t < p.world) {
    const int32_t* f = own_flags + parity * XCHG_MAX_WORLD + t;
    const long long t0 = clock64();
    bool ok = true;
    for (uint32_t spin = 1; ld_acquire_sys(f) != step; ++spin) {
      if ((spin & 63u) == 0u) {
        if (*reinterpret_cast<volatile int32_t*>(p.status) != 0) { ok = false; break; }
        if (clock64() - t0 > p.limit) {
          if (atomicCAS(p.status, 0, 1) == 0) p.status[1] = blockIdx.x, p.status[2] = 32 + t;  // site 32 + r: rank r never arrived
          ok = false;
          break;
        }
      }
    }
    if (!ok) ok_sm = 0;
  }
  __syncthreads();
  if (!ok_sm) return;  // the step counter stays where it was: the exchange is out of step from here on
  // ---- merge: my rows over all ranks' states, from local memory ----
  const float* base = reinterpret_cast<const float*>(own) + (size_t)parity * p.world * slot;
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    float M = -INFINITY;
    // L2 reads (__ldcg): these lines were written by other GPUs since this SM may last have cached them
    for (int r = 0; r < p.world; ++r) M = fmaxf(M, __ldcg(base + (size_t)r * slot + (size_t)row * PART_STRIDE));
    float l = 0.f, acc = 0.f;
    for (int r = 0; r < p.world; ++r) {
      const float* ps = base + (size_t)r * slot + (size_t)row * PART_STRIDE;
      const float m_r = __ldcg(ps);
      const float f = (m_r == -INFINITY) ? 0.f : ex2_approx(m_r - M);
      l += __ldcg(ps + 1) * f;
      acc += __ldcg(ps + 2 + t) * f;
    }
    const float res = acc / l;
    if (p.out_dtype == BMXK_DTYPE_F32)
      reinterpret_cast<float*>(p.out)[(size_t)row * HEAD_DIM + t] = res;
    else
      reinterpret_cast<__half*>(p.out)[(size_t)row * HEAD_DIM + t] = __float2half_rn(res);
  }
  // ---- the last block to end records the step (every block has read the old value by now) ----
  if (t == 0 && atomicAdd(ended, 1) == (int)gridDim.x - 1) {
    *ended = 0;
    *last_step = step;
  }
}

}  // namespace

}  // namespace bmxk

using namespace bmxk;

extern "C" {

size_t bmxk_xchg_bytes(int rows, int world) {
  if (rows <= 0 || world <= 0 || world > XCHG_MAX_WORLD) return 0;
  return xchg_total_bytes(rows, world);
}

int bmxk_xchg_alloc(int rows, int world, void** buffer, void* ipc_handle_64) {
  BMXK_REQUIRE(buffer && ipc_handle_64, "bmxk_xchg_alloc: null argument");
  BMXK_REQUIRE(rows >= 1 && world >= 1 && world <= XCHG_MAX_WORLD, "bmxk_xchg_alloc: rows=%d world=%d (world at most %d)", rows, world,
               XCHG_MAX_WORLD);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
  void* ptr = nullptr;
  const size_t bytes = xchg_total_bytes(rows, world);
  cudaError_t e = cudaMalloc(&ptr, bytes);  // an allocation of its own: an IPC handle names a whole cudaMalloc block
  if (e == cudaSuccess) e = cudaMemset(ptr, 0, bytes);
  cudaIpcMemHandle_t h;
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) {
    if (ptr) cudaFree(ptr);
    set_error("bmxk_xchg_alloc: %s", cudaGetErrorString(e));
    return BMXK_ERR_CUDA;
  }
  memcpy(ipc_handle_64, &h, 64);
  *buffer = ptr;
  return BMXK_OK;
}

int bmxk_xchg_open(const void* ipc_handle_64, void** peer_buffer) {
  BMXK_REQUIRE(ipc_handle_64 && peer_buffer, "bmxk_xchg_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, ipc_handle_64, 64);
  void* ptr = nullptr;
  const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    set_error("bmxk_xchg_open: %s", cudaGetErrorString(e));
    return BMXK_ERR_CUDA;
  }
  *peer_buffer = ptr;
  return BMXK_OK;
}

int bmxk_xchg_close(void* peer_buffer) {
  if (!peer_buffer) return BMXK_OK;
  const cudaError_t e = cudaIpcCloseMemHandle(peer_buffer);
  if (e != cudaSuccess) {
    set_error("bmxk_xchg_close: %s", cudaGetErrorString(e));
    return BMXK_ERR_CUDA;
  }
  return BMXK_OK;
}

int bmxk_xchg_free(void* buffer) {
  if (!buffer) return BMXK_OK;
  const cudaError_t e = cudaFree(buffer);
  if (e != cudaSuccess) {
    set_error("bmxk_xchg_free: %s", cudaGetErrorString(e));
    return BMXK_ERR_CUDA;
  }
  return BMXK_OK;
}

int bmxk_xchg_merge(const float* part, int rows, int rank, int world, void* const* buffers, int step, int64_t wait_limit_cycles,
                    int32_t* status, void* out, int out_dtype, void* stream) {
  BMXK_REQUIRE(part && buffers && status && out, "bmxk_xchg_merge: null pointer");
  BMXK_REQUIRE(rows >= 1 && world >= 1 && world <= XCHG_MAX_WORLD && rank >= 0 && rank < world, "bmxk_xchg_merge: rows=%d rank=%d world=%d",
               rows, rank, world);
  BMXK_REQUIRE(step >= 0, "bmxk_xchg_merge: step=%d (1, 2, 3, ... or 0 for the buffer's own count)", step);
  BMXK_REQUIRE(wait_limit_cycles >= 1000 && wait_limit_cycles <= 8000000000LL, "bmxk_xchg_merge: wait limit %lld cycles out of range",
               (long long)wait_limit_cycles);
  BMXK_REQUIRE(out_dtype == BMXK_DTYPE_F16 || out_dtype == BMXK_DTYPE_F32, "bmxk_xchg_merge: out_dtype=%d", out_dtype);
  XchgParams p;
  p.part = part, p.rows = rows, p.rank = rank, p.world = world, p.step = step, p.limit = wait_limit_cycles;
  p.status = status, p.out = out, p.out_dtype = out_dtype;
  for (int r = 0; r < XCHG_MAX_WORLD; ++r) p.bufs[r] = nullptr;
  for (int r = 0; r < world; ++r) {
    BMXK_REQUIRE(buffers[r] != nullptr, "bmxk_xchg_merge: no buffer for rank %d", r);
    p.bufs[r] = reinterpret_cast<uint8_t*>(buffers[r]);
  }
  // every block must be resident at once (blocks wait for one another's pushes through the flag): one per SM at most
  const int grid = rows < num_sms() ? rows : num_sms();
  xchg_merge_kernel<<<grid, XCHG_THREADS, 0, (cudaStream_t)stream>>>(p);
  return check_launch("bmxk_xchg_merge");
}

}  // extern "C"
