// Execution-platform shims: the scheduler, the step engine and the data path are
// written once and compiled twice, as sm_100a device code (a thread block of
// several warps) and as host code in which one OS thread plays a whole block
// (thread id 0, block size 1).  Only this header knows the difference.
//
// Memory-ordering vocabulary (replaces the reference's volatile accesses plus
// __threadfence_system, src/collectives_ofccl/device/ofccl_prims_simple.h:118-205):
//   ld_acquire_sys / st_release_sys  - flag words other GPUs or the host write / read
//   ld_relaxed_sys                   - payload that must not come from a stale L1 line
//   fence_sys                        - orders a block's payload stores before its flag store
#pragma once
#include <stdint.h>
#include <cuda_runtime.h>

#if defined(__CUDA_ARCH__)
#define DF_DEVICE_CODE 1
#else
#define DF_DEVICE_CODE 0
#include <time.h>
#include <sched.h>
#endif

#define DF_HD __host__ __device__ __forceinline__
#define DF_HD_NOINLINE __host__ __device__ __noinline__

namespace dfccl {

DF_HD int df_tid() {
#if DF_DEVICE_CODE
  return threadIdx.x;
#else
  return 0;
#endif
}
DF_HD int df_nthreads() {
#if DF_DEVICE_CODE
  return blockDim.x;
#else
  return 1;
#endif
}
DF_HD int df_lane() {
#if DF_DEVICE_CODE
  return threadIdx.x & 31;
#else
  return 0;
#endif
}
DF_HD int df_warpsize() {
#if DF_DEVICE_CODE
  return 32;
#else
  return 1;
#endif
}
DF_HD void df_sync() {
#if DF_DEVICE_CODE
  __syncthreads();
#endif
}
// true on every lane iff pred holds on every lane of the calling warp
DF_HD bool df_warp_all(bool pred) {
#if DF_DEVICE_CODE
  return __all_sync(0xffffffffu, pred);
#else
  return pred;
#endif
}
DF_HD void df_warp_sync() {
#if DF_DEVICE_CODE
  __syncwarp();
#endif
}

// ThreadSanitizer understands acquire / release pairs but not stand-alone fences.  The engine orders payload
// accesses with "relaxed flag access + one fence"; in a sanitizer build of the host twin the relaxed flag
// accesses are promoted to acquire / release, which is stronger, so that the tool sees the same ordering.
#if defined(__SANITIZE_THREAD__)
#define DF_HOST_RELAXED_LD __ATOMIC_ACQUIRE
#define DF_HOST_RELAXED_ST __ATOMIC_RELEASE
#else
#define DF_HOST_RELAXED_LD __ATOMIC_RELAXED
#define DF_HOST_RELAXED_ST __ATOMIC_RELAXED
#endif

// Control words shared between host threads and the (host twin of the) device code.
DF_HD uint32_t ctl_load(const volatile uint32_t* p) {
#if DF_DEVICE_CODE
  return *p;
#else
  return __atomic_load_n((const uint32_t*)p, __ATOMIC_ACQUIRE);
#endif
}
DF_HD void ctl_store(volatile uint32_t* p, uint32_t v) {
#if DF_DEVICE_CODE
  *p = v;
#else
  __atomic_store_n((uint32_t*)p, v, __ATOMIC_RELEASE);
#endif
}

DF_HD uint64_t ld_acquire_sys_u64(const volatile uint64_t* p) {
#if DF_DEVICE_CODE
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
#else
  return __atomic_load_n((const uint64_t*)p, __ATOMIC_ACQUIRE);
#endif
}
DF_HD uint64_t ld_relaxed_sys_u64(const volatile uint64_t* p) {
#if DF_DEVICE_CODE
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
#else
  return __atomic_load_n((const uint64_t*)p, DF_HOST_RELAXED_LD);
#endif
}
DF_HD uint32_t ld_acquire_sys_u32(const volatile uint32_t* p) {
#if DF_DEVICE_CODE
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
#else
  return __atomic_load_n((const uint32_t*)p, __ATOMIC_ACQUIRE);
#endif
}
DF_HD void st_release_sys_u64(volatile uint64_t* p, uint64_t v) {
#if DF_DEVICE_CODE
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#else
  __atomic_store_n((uint64_t*)p, v, __ATOMIC_RELEASE);
#endif
}
// release at GPU scope: for words that only blocks of this GPU read (cheaper than a system-scope fence)
DF_HD void st_release_gpu_u64(volatile uint64_t* p, uint64_t v) {
#if DF_DEVICE_CODE
  asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#else
  __atomic_store_n((uint64_t*)p, v, __ATOMIC_RELEASE);
#endif
}
DF_HD uint32_t ld_relaxed_sys_u32(const volatile uint32_t* p) {
#if DF_DEVICE_CODE
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
#else
  return __atomic_load_n((const uint32_t*)p, DF_HOST_RELAXED_LD);
#endif
}
DF_HD void st_relaxed_sys_u64(volatile uint64_t* p, uint64_t v) {
#if DF_DEVICE_CODE
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
#else
  __atomic_store_n((uint64_t*)p, v, DF_HOST_RELAXED_ST);
#endif
}
DF_HD void st_release_sys_u32(volatile uint32_t* p, uint32_t v) {
#if DF_DEVICE_CODE
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
#else
  __atomic_store_n((uint32_t*)p, v, __ATOMIC_RELEASE);
#endif
}
DF_HD void fence_sys() {
#if DF_DEVICE_CODE
  __threadfence_system();
#else
  __atomic_thread_fence(__ATOMIC_SEQ_CST);
#endif
}
DF_HD void fence_gpu() {
#if DF_DEVICE_CODE
  __threadfence();
#else
  __atomic_thread_fence(__ATOMIC_SEQ_CST);
#endif
}
DF_HD uint32_t atomic_add_u32(uint32_t* p, uint32_t v) {
#if DF_DEVICE_CODE
  return atomicAdd(p, v);
#else
  return __atomic_fetch_add(p, v, __ATOMIC_ACQ_REL);
#endif
}
DF_HD unsigned long long atomic_add_u64(unsigned long long* p, unsigned long long v) {
#if DF_DEVICE_CODE
  return atomicAdd(p, v);
#else
  return __atomic_fetch_add(p, v, __ATOMIC_ACQ_REL);
#endif
}
DF_HD uint32_t atomic_cas_u32(uint32_t* p, uint32_t expect, uint32_t desired) {
#if DF_DEVICE_CODE
  return atomicCAS(p, expect, desired);
#else
  __atomic_compare_exchange_n(p, &expect, desired, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE);
  return expect;
#endif
}
DF_HD uint32_t atomic_exch_u32(uint32_t* p, uint32_t v) {
#if DF_DEVICE_CODE
  return atomicExch(p, v);
#else
  return __atomic_exchange_n(p, v, __ATOMIC_ACQ_REL);
#endif
}

DF_HD uint64_t df_now_ns() {
#if DF_DEVICE_CODE
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
#else
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (uint64_t)ts.tv_sec * 1000000000ull + (uint64_t)ts.tv_nsec;
#endif
}
DF_HD void df_backoff(uint32_t ns) {
#if DF_DEVICE_CODE
  __nanosleep(ns);
#else
  (void)ns;
  sched_yield();
#endif
}

// 16-byte payload accesses that bypass L1 (the daemon outlives the kernels that
// produce its inputs, so a cached line could be one submission old).
DF_HD uint4 ld16(const void* p) {
#if DF_DEVICE_CODE
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
#else
  uint4 v;
  __builtin_memcpy(&v, p, 16);
  return v;
#endif
}
DF_HD void st16(void* p, uint4 v) {
#if DF_DEVICE_CODE
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
#else
  __builtin_memcpy(p, &v, 16);
#endif
}
}  // namespace dfccl
