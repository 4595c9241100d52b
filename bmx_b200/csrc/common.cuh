// Shared pieces of the bmxk library: status codes, the last-error string, launch checks and
// the sm_100a PTX wrappers (mbarrier, bulk async copy, ldmatrix, mma.sync) the kernels use.
#pragma once
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#include "../../include/bmxk.h"
#include "layout.cuh"

namespace bmxk {

// Thread-local message behind bmxk_last_error(); every entry point returns a status instead of
// throwing or aborting.
void set_error(const char* fmt, ...);
int check_launch(const char* what);

#define BMXK_REQUIRE(cond, ...)            \
  do {                                     \
    if (!(cond)) {                         \
      ::bmxk::set_error(__VA_ARGS__);      \
      return BMXK_ERR_INVALID;             \
    }                                      \
  } while (0)

// Launch configuration that belongs to a device (opt-in shared-memory sizes, the SM count) is kept per device: one
// process may drive several GPUs, and cudaFuncSetAttribute only affects the device that is current when it is called.
constexpr int MAX_DEVICES = 64;
inline int current_device() {
  int d = 0;
  if (cudaGetDevice(&d) != cudaSuccess || d < 0 || d >= MAX_DEVICES) d = 0;
  return d;
}
// One flag per device; `test_and_set()` returns true the first time it is called with a given device current.  Two
// threads racing on the first call both see true: what follows (setting an attribute) is idempotent.
struct PerDeviceOnce {
  volatile unsigned char done[MAX_DEVICES] = {};
  bool first() {
    const int d = current_device();
    if (done[d]) return false;
    done[d] = 1;
    return true;
  }
  void retract() { done[current_device()] = 0; }  // the set-up failed: try again on the next call
};

// Device-side status word layout (int32[4], owned by the caller's workspace):
//   [0] non-zero once any bounded wait gave up, [1] block that gave up, [2] where, [3] spare.
constexpr int STATUS_WORDS = 4;

#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that may park the thread for up to `ns` nanoseconds (it wakes as soon as the phase completes), so
// that a waiting warp leaves the issue slots to the warps that work.
__device__ __forceinline__ bool mbar_try_wait_parked(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Shared-memory atomics that are themselves the synchronisation point (release on the way in, acquire on the
// way out, CTA scope), so that no separate fence is needed around them.
__device__ __forceinline__ int smem_add_acq_rel(int* addr, int v) {
  int old;
  asm volatile("atom.acq_rel.cta.shared::cta.add.u32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(addr)), "r"(v) : "memory");
  return old;
}
__device__ __forceinline__ void smem_or_release(int* addr, int v) {
  asm volatile("red.release.cta.shared::cta.or.b32 [%0], %1;" ::"r"(smem_u32(addr)), "r"(v) : "memory");
}
__device__ __forceinline__ int smem_exch_acquire(int* addr, int v) {
  int old;
  asm volatile("atom.acquire.cta.shared::cta.exch.b32 %0, [%1], %2;" : "=r"(old) : "r"(smem_u32(addr)), "r"(v) : "memory");
  return old;
}
// Arrival counters in shared memory for a consumer that polls several of them with plain loads (an mbarrier
// test costs ~70 cycles and they cannot overlap; loads can): release on the producer's add, acquire on the load.
__device__ __forceinline__ void smem_add_release(int* addr, int v) {
  asm volatile("red.release.cta.shared::cta.add.u32 [%0], %1;" ::"r"(smem_u32(addr)), "r"(v) : "memory");
}
__device__ __forceinline__ int smem_load_acquire(const int* addr) {
  int v;
  asm volatile("ld.acquire.cta.shared::cta.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(addr)) : "memory");
  return v;
}
// Non-blocking test of a phase, for a thread that polls several barriers in turn (try_wait may park the
// thread for a hardware-chosen time before it reports "not yet").
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll may itself block for a hardware-chosen
// time) and returns false, so a lost copy can never hang the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, uint32_t limit = (1u << 22)) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}
// 1-D bulk async copy global -> this CTA's shared memory, completion counted in bytes on `bar`.
// Source, destination and size are multiples of 16 bytes.  Local HBM only; never multicast.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(f16x2 pair) += A(16x16 f16) * B(16x8 f16), fp16 accumulate
__device__ __forceinline__ void mma_f16acc(uint32_t& d0, uint32_t& d1, uint32_t a0, uint32_t a1, uint32_t a2,
                                           uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0,%1}, {%2,%3,%4,%5}, {%6,%7}, {%0,%1};"
               : "+r"(d0), "+r"(d1)
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// D(f32 x4) += A * B, fp32 accumulate
__device__ __forceinline__ void mma_f32acc(float& c0, float& c1, float& c2, float& c3, uint32_t a0, uint32_t a1,
                                           uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c0), "+f"(c1), "+f"(c2), "+f"(c3)
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// transpose of an 8x8 matrix of 16-bit elements spread over the warp in mma fragment order
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
template <int LUT>
__device__ __forceinline__ uint32_t lop3(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t d;
  asm("lop3.b32 %0, %1, %2, %3, %4;" : "=r"(d) : "r"(a), "r"(b), "r"(c), "n"(LUT));
  return d;
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
template <typename T>
__device__ __forceinline__ float load_as_float(const T* p);
template <>
__device__ __forceinline__ float load_as_float<__half>(const __half* p) { return __half2float(*p); }
template <>
__device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float load_as_float<float>(const float* p) { return *p; }

// Orthonormal 128-point FWHT of a row held 4 elements per lane (lane L owns channels 4L..4L+3).
// Same butterflies as the reference (h = 1, 2, 4, ..: low index gets a+b, high index a-b), then one
// true division by float32(sqrt(128)).
__device__ __forceinline__ void fwht128_warp(float (&x)[4], int lane) {
  {  // h = 1
    const float a0 = x[0] + x[1], a1 = x[0] - x[1], a2 = x[2] + x[3], a3 = x[2] - x[3];
    x[0] = a0, x[1] = a1, x[2] = a2, x[3] = a3;
  }
  {  // h = 2
    const float a0 = x[0] + x[2], a1 = x[1] + x[3], a2 = x[0] - x[2], a3 = x[1] - x[3];
    x[0] = a0, x[1] = a1, x[2] = a2, x[3] = a3;
  }
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {  // h = 4*m
    const bool hi = (lane & m) != 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float o = __shfl_xor_sync(0xffffffffu, x[k], m);
      x[k] = hi ? (o - x[k]) : (x[k] + o);
    }
  }
  const float s = 11.313708498984761f;  // float32(128 ** 0.5)
#pragma unroll
  for (int k = 0; k < 4; ++k) x[k] = x[k] / s;
}

#endif  // __CUDACC__

}  // namespace bmxk
