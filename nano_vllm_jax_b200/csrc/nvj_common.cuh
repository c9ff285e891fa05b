// Shared device helpers for the sm_100a paged KV-cache kernels: bf16 unpacking,
// mbarrier / bulk-copy wrappers with bounded waits, and small warp utilities.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/nvj_b200.h"

namespace nvj {

constexpr unsigned kFullMask = 0xffffffffu;

// Longest time any device-side wait may poll before the kernel gives up, flags
// NVJ_DEV_TIMEOUT and runs to its end without waiting any more.  Waits on a CTA's own copies use this
// fixed bound; waits on another GPU (the token gather) take the process-wide limit set by
// nvj_set_wait_limit_ns, whose default is this value.
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;
unsigned long long wait_limit_ns();  // host: the current process-wide limit

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ---- bf16 pair unpack: a 32-bit word holds elements (2i, 2i+1) = (low, high).
__device__ __forceinline__ float2 bf16x2_to_float2(uint32_t w) {
  float2 r;
  r.x = __uint_as_float(w << 16);
  r.y = __uint_as_float(w & 0xffff0000u);
  return r;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// d = a * b + c on packed fp32 pairs (one FFMA2 on sm_100).
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  return __ffma2_rn(a, b, c);
}

// ---- mbarrier (shared::cta) ------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  // Make the initialised barriers visible to the async proxy before first use.
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory and is set by the first
// waiter of the CTA that runs out of time; once set, every wait returns at once
// so that all warps reach the end of the kernel (results are then invalid and
// the status word says so).
static __device__ __noinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity,
                                            volatile int* abort_flag, int32_t* status,
                                            unsigned long long limit_ns) {
  const unsigned long long t0 = global_timer_ns();
  for (uint32_t i = 0;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 31u) == 31u) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        if (status) atomicOr(status, NVJ_DEV_TIMEOUT);
        return false;
      }
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity,
                                          volatile int* abort_flag, int32_t* status,
                                          unsigned long long limit_ns = kWaitLimitNs) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;
  return mbar_wait_slow(bar, parity, abort_flag, status, limit_ns);
}

// ---- 1-D bulk async copy global -> this CTA's shared memory -----------------
// Source and destination 16-byte aligned, size a multiple of 16 bytes.  The
// copy signals `bar` with complete_tx for `bytes`.  The lines are marked evict-first in L2:
// the callers stream K/V blocks that are read once per launch, and keeping them from
// displacing each other's in-flight lines measured 1.7% on the 1.3 GB decode step.
__device__ __forceinline__ void bulk_g2s(uint32_t smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint32_t bar) {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_dst), "l"(gmem_src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}

// Order this thread's earlier generic-proxy writes before later async-proxy
// (bulk copy) reads of the same memory.
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---- loads that must see other CTAs' recent global writes -------------------
__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float2 ld_cg_f32x2(const float* p) {
  float2 v;
  asm volatile("ld.global.cg.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
  return v;
}

// Streaming 16-byte load that does not allocate in L1 (read-once data).
__device__ __forceinline__ uint4 ld_nc_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Once-per-device set-up on the host (a kernel attribute, a cached device property), safe when several host
// threads make their first call together: the set-up itself must be idempotent (two threads may both run it),
// the flag is published with release / acquire.
constexpr int kMaxDevices = 64;
struct PerDeviceFlags {
  std::atomic<int> v[kMaxDevices];
};
// Returns the current device ordinal, or -1.
inline int current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}
template <class F>
inline bool once_per_device(PerDeviceFlags& flags, F&& setup) {
  const int dev = current_device();
  if (dev < 0) return false;
  if (flags.v[dev].load(std::memory_order_acquire) != 0) return true;
  if (!setup(dev)) return false;
  flags.v[dev].store(1, std::memory_order_release);
  return true;
}

__host__ __device__ __forceinline__ int dtype_size(int dt) {
  return dt == NVJ_F32 ? 4 : 2;
}

}  // namespace nvj
