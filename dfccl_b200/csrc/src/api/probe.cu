// Probe kernels: what the fabric gives to plain loads and stores of peer memory, and how long
// a flag takes from one GPU to another.  Their numbers are the inputs of the tuner's cost model
// (topo.cu: linkGBs, perBlockGBs, hopUs) and decided which load instruction the data path uses.
// No counterpart in the reference, whose model constants are compiled in
// (src/graph/topo.h:14-18, src/graph/tuning.cc:56-73).
#include "../comm/comm.h"
#include "../common/log.h"
#include "../device/platform.h"

namespace dfccl {
namespace {

enum LoadKind { LD_RELAXED_SYS = 0, LD_VOLATILE = 1, LD_CG = 2, LD_WEAK = 3, LD_NC = 4 };

template <int KIND> __device__ __forceinline__ uint4 probeLoad(const uint4* p) {
  uint4 v;
  if (KIND == LD_RELAXED_SYS) asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else if (KIND == LD_VOLATILE) asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else if (KIND == LD_CG) asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else if (KIND == LD_NC) asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else v = *p;
  return v;
}

// dst[i] = src[i] over n 16-byte packs; U packs per thread per trip.
template <int KIND, int U>
__global__ void __launch_bounds__(512) probeCopyKernel(const uint4* __restrict__ src, uint4* __restrict__ dst, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t base = (size_t)blockIdx.x * blockDim.x + threadIdx.x; base < n; base += stride * U) {
    uint4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) if (base + u * stride < n) v[u] = probeLoad<KIND>(src + base + u * stride);
#pragma unroll
    for (int u = 0; u < U; ++u) if (base + u * stride < n) dst[base + u * stride] = v[u];
  }
}

template <int KIND>
void launchCopy(int unroll, int blocks, const uint4* s, uint4* d, size_t n, cudaStream_t st) {
  switch (unroll) {
    case 1: probeCopyKernel<KIND, 1><<<blocks, 512, 0, st>>>(s, d, n); break;
    case 2: probeCopyKernel<KIND, 2><<<blocks, 512, 0, st>>>(s, d, n); break;
    case 4: probeCopyKernel<KIND, 4><<<blocks, 512, 0, st>>>(s, d, n); break;
    case 8: probeCopyKernel<KIND, 8><<<blocks, 512, 0, st>>>(s, d, n); break;
    default: probeCopyKernel<KIND, 16><<<blocks, 512, 0, st>>>(s, d, n); break;
  }
}

// Flag ping-pong between two ranks: rank 0 writes k into the peer's word, the peer answers k into
// rank 0's word.  Every wait is bounded; on expiry the kernel stores an error and returns.
__global__ void probePingPongKernel(volatile uint64_t* mine, volatile uint64_t* theirs, int iAmFirst, int iters,
                                    uint64_t base, uint64_t limitNs, uint32_t* err) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  for (int k = 1; k <= iters; ++k) {
    const uint64_t want = base + k;
    if (iAmFirst) st_release_sys_u64(theirs, want);
    const uint64_t t0 = df_now_ns();
    while (ld_acquire_sys_u64(mine) < want) {
      if (df_now_ns() - t0 > limitNs) { *err = 1; return; }
    }
    if (!iAmFirst) st_release_sys_u64(theirs, want);
  }
}

}  // namespace
}  // namespace dfccl

using namespace dfccl;

// Copy `bytes` between this rank's heap and `peer`'s heap with the library's own kernels.
//   direction 0: read peer -> write local      direction 1: read local -> write peer
//   loadKind: 0 ld.relaxed.sys  1 ld.volatile  2 ld.global.cg  3 plain  4 ld.global.nc
// Collective over the two ranks involved only in the sense that both heaps must exist; only the
// caller moves data.  Returns the mean device time of one copy in microseconds.
extern "C" __attribute__((visibility("default")))
ncclResult_t dfcclProbePeerCopy(ncclComm_t comm, int peer, size_t bytes, int direction, int loadKind, int unroll, int blocks,
                                int iters, double* usOut) {
  if (!comm || !usOut || peer < 0 || peer >= comm->nranks || comm->backend != dfcclBackendCuda) return ncclInvalidArgument;
  bytes &= ~(size_t)15;
  if (bytes == 0 || iters < 1 || blocks < 1) return ncclInvalidArgument;
  uint64_t off = 0;
  DFCHECK(comm->heap->alloc(bytes, &off, false));
  // symmetric use: the peer allocates the same amount in the same order, so the offset there is valid memory
  // of this probe as long as both ranks call it in step; only offsets inside the peer's live probe area are touched
  char* local = comm->heap->base() + off;
  char* remote = comm->peerHeap[peer] + off;
  const uint4* src = (const uint4*)(direction == 0 ? remote : local);
  uint4* dst = (uint4*)(direction == 0 ? local : remote);
  const size_t n = bytes / 16;
  cudaEvent_t e0, e1;
  CUDACHECK(cudaEventCreate(&e0));
  CUDACHECK(cudaEventCreate(&e1));
  auto once = [&] {
    switch (loadKind) {
      case LD_RELAXED_SYS: launchCopy<LD_RELAXED_SYS>(unroll, blocks, src, dst, n, 0); break;
      case LD_VOLATILE: launchCopy<LD_VOLATILE>(unroll, blocks, src, dst, n, 0); break;
      case LD_CG: launchCopy<LD_CG>(unroll, blocks, src, dst, n, 0); break;
      case LD_NC: launchCopy<LD_NC>(unroll, blocks, src, dst, n, 0); break;
      default: launchCopy<LD_WEAK>(unroll, blocks, src, dst, n, 0); break;
    }
  };
  for (int i = 0; i < 3; ++i) once();
  CUDACHECK(cudaDeviceSynchronize());
  CUDACHECK(cudaEventRecord(e0, 0));
  for (int i = 0; i < iters; ++i) once();
  CUDACHECK(cudaEventRecord(e1, 0));
  CUDACHECK(cudaEventSynchronize(e1));
  float ms = 0;
  CUDACHECK(cudaEventElapsedTime(&ms, e0, e1));
  *usOut = (double)ms * 1e3 / iters;
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  DFCHECK(comm->heap->free(off));
  return ncclSuccess;
}

// Round-trip time of a flag between this rank and `peer` (both call it, the lower rank starts).
extern "C" __attribute__((visibility("default")))
ncclResult_t dfcclProbeFlagRoundTrip(ncclComm_t comm, int peer, int iters, double* usOut) {
  if (!comm || !usOut || peer < 0 || peer >= comm->nranks || peer == comm->rank || comm->backend != dfcclBackendCuda) return ncclInvalidArgument;
  // reuse two words of the send / recv flag block of this pair (direction 0, channel 7 is never used by 1-channel transfers here)
  FlagSlot* mine = (FlagSlot*)(comm->heap->base() + comm->p2pFlagsOff) + ((size_t)0 * comm->nranks + peer) * 8 + 7;
  FlagSlot* theirs = (FlagSlot*)(comm->peerHeap[peer] + comm->peerP2pFlagsOff[peer]) + ((size_t)0 * comm->nranks + comm->rank) * 8 + 7;
  uint32_t* err = nullptr;
  CUDACHECK(cudaMalloc((void**)&err, 4));
  CUDACHECK(cudaMemset(err, 0, 4));
  static uint64_t base = 0;
  cudaEvent_t e0, e1;
  CUDACHECK(cudaEventCreate(&e0));
  CUDACHECK(cudaEventCreate(&e1));
  DFCHECK(comm->boot->barrier());
  // warm-up exchange, then the timed one
  probePingPongKernel<<<1, 32>>>(&mine->sendOff, &theirs->sendOff, comm->rank < peer, 16, base, 2000000000ull, err);
  base += 16;
  CUDACHECK(cudaDeviceSynchronize());
  DFCHECK(comm->boot->barrier());
  CUDACHECK(cudaEventRecord(e0, 0));
  probePingPongKernel<<<1, 32>>>(&mine->sendOff, &theirs->sendOff, comm->rank < peer, iters, base, 2000000000ull, err);
  base += iters;
  CUDACHECK(cudaEventRecord(e1, 0));
  CUDACHECK(cudaEventSynchronize(e1));
  float ms = 0;
  CUDACHECK(cudaEventElapsedTime(&ms, e0, e1));
  uint32_t herr = 0;
  CUDACHECK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
  cudaFree(err);
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  if (herr) { DF_WARN("flag probe: the peer did not answer within 2 s"); return dfcclTimeout; }
  *usOut = (double)ms * 1e3 / iters;
  return ncclSuccess;
}

// ---------------------------------------------------------------------------------------------------------------
// Round trip "stream releases a word -> a resident kernel answers -> stream continues": the cost of one
// stream-ordered submission as the daemon sees it, without any collective in between.  An echo kernel (one thread)
// waits for word A to reach k and answers by writing k to word B; the timed stream alternates "write A = k" and
// "wait until B >= k".  Both steps exist in two forms: a stream memory operation, or a one-thread kernel.
//   mode bit 0: the write is a kernel (else cuStreamWriteValue64)
//   mode bit 1: the wait is a kernel  (else cuStreamWaitValue64)
//   mode bit 2: the write also stores a mirror word in pinned host memory (batched with the device word when both
//               are memory operations, a second store of the same kernel otherwise)
// `delayUs`: the echo kernel answers that long after it saw the release (the time a collective would take), which
// shows how the cost of the wait depends on how long the stream has been parked on it; the result includes it.
// Every wait is bounded by `limitNs`; a wait that runs out stores an error and the kernels return.
#include <cuda.h>
namespace dfccl {
namespace {

__global__ void probeEchoKernel(volatile uint64_t* a, volatile uint64_t* b, int iters, uint64_t limitNs, uint64_t delayNs, uint32_t* err) {
  if (threadIdx.x != 0) return;
  const uint64_t t0 = df_now_ns();
  for (int k = 1; k <= iters; ++k) {
    while (ld_relaxed_sys_u64(a) < (uint64_t)k) {
      if (df_now_ns() - t0 > limitNs || *(volatile uint32_t*)err) { *err = 1; return; }
    }
    if (delayNs) { const uint64_t t1 = df_now_ns(); while (df_now_ns() - t1 < delayNs) {} }   // "the collective"
    st_relaxed_sys_u64(b, (uint64_t)k);
  }
}
__global__ void probeWriteKernel(volatile uint64_t* a, volatile uint64_t* mirror, uint64_t v) {
  if (mirror) *mirror = v;
  st_relaxed_sys_u64(a, v);
}
__global__ void probeWaitKernel(volatile uint64_t* b, uint64_t v, uint64_t limitNs, uint32_t* err) {
  const uint64_t t0 = df_now_ns();
  while (ld_relaxed_sys_u64(b) < v) {
    if (df_now_ns() - t0 > limitNs || *(volatile uint32_t*)err) { *err = 2; return; }
  }
}

}  // namespace
}  // namespace dfccl

extern "C" __attribute__((visibility("default")))
ncclResult_t dfcclProbeStreamRoundTrip(int mode, int iters, int delayUs, double* usOut) {
  if (!usOut || iters < 1 || iters > 400 || mode < 0 || mode > 7 || delayUs > 1000) return ncclInvalidArgument;
  typedef CUresult (*FnW)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);
  typedef CUresult (*FnB)(CUstream, unsigned int, CUstreamBatchMemOpParams*, unsigned int);
  void *fw = nullptr, *fwait = nullptr, *fb = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuStreamWriteValue64", &fw, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) fw = nullptr;
  if (cudaGetDriverEntryPoint("cuStreamWaitValue64", &fwait, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) fwait = nullptr;
  if (cudaGetDriverEntryPoint("cuStreamBatchMemOp", &fb, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) fb = nullptr;
  (void)cudaGetLastError();
  const bool kWrite = mode & 1, kWait = mode & 2, mirror = mode & 4;
  if ((!kWrite && !fw) || (!kWait && !fwait) || (mirror && !kWrite && !fb)) return ncclInvalidUsage;
  uint64_t* words = nullptr;
  uint64_t* hostWord = nullptr;
  uint32_t* err = nullptr;
  CUDACHECK(cudaMalloc((void**)&words, 512));
  CUDACHECK(cudaMemset(words, 0, 512));
  CUDACHECK(cudaMalloc((void**)&err, 4));
  CUDACHECK(cudaMemset(err, 0, 4));
  CUDACHECK(cudaHostAlloc((void**)&hostWord, 64, cudaHostAllocMapped));
  *hostWord = 0;
  volatile uint64_t* a = words;
  volatile uint64_t* b = words + 32;       // another 256-byte line
  cudaStream_t sEcho, s;
  CUDACHECK(cudaStreamCreateWithFlags(&sEcho, cudaStreamNonBlocking));
  CUDACHECK(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  cudaEvent_t e0, e1;
  CUDACHECK(cudaEventCreate(&e0));
  CUDACHECK(cudaEventCreate(&e1));
  const uint64_t limitNs = 2000000000ull;
  ncclResult_t res = ncclSuccess;
  CUDACHECK(cudaDeviceSynchronize());
  probeEchoKernel<<<1, 32, 0, sEcho>>>(a, b, iters, limitNs, (uint64_t)(delayUs < 0 ? 0 : delayUs) * 1000ull, err);
  CUDACHECK(cudaEventRecord(e0, s));
  for (int k = 1; k <= iters && res == ncclSuccess; ++k) {
    if (kWrite) probeWriteKernel<<<1, 1, 0, s>>>(a, mirror ? hostWord : nullptr, (uint64_t)k);
    else if (mirror) {
      CUstreamBatchMemOpParams ops[2];
      memset(ops, 0, sizeof(ops));
      ops[0].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_64;
      ops[0].writeValue.address = (CUdeviceptr)(uintptr_t)a;
      ops[0].writeValue.value64 = (cuuint64_t)k;
      ops[1].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_64;
      ops[1].writeValue.address = (CUdeviceptr)(uintptr_t)hostWord;
      ops[1].writeValue.value64 = (cuuint64_t)k;
      if (((FnB)fb)((CUstream)s, 2, ops, 0) != CUDA_SUCCESS) res = ncclUnhandledCudaError;
    } else if (((FnW)fw)((CUstream)s, (CUdeviceptr)(uintptr_t)a, (cuuint64_t)k, 0) != CUDA_SUCCESS) res = ncclUnhandledCudaError;
    if (kWait) probeWaitKernel<<<1, 1, 0, s>>>(b, (uint64_t)k, limitNs, err);
    else if (((FnW)fwait)((CUstream)s, (CUdeviceptr)(uintptr_t)b, (cuuint64_t)k, CU_STREAM_WAIT_VALUE_GEQ) != CUDA_SUCCESS) res = ncclUnhandledCudaError;
  }
  if (res != ncclSuccess) {
    // release the echo kernel (and any wait already enqueued): the error word ends every bounded wait
    uint32_t one = 1;
    cudaMemcpyAsync(err, &one, 4, cudaMemcpyHostToDevice, 0);
    if (fw) { ((FnW)fw)((CUstream)s, (CUdeviceptr)(uintptr_t)b, (cuuint64_t)iters + 1, 0); }
  }
  CUDACHECK(cudaEventRecord(e1, s));
  CUDACHECK(cudaStreamSynchronize(s));
  CUDACHECK(cudaStreamSynchronize(sEcho));
  float ms = 0;
  CUDACHECK(cudaEventElapsedTime(&ms, e0, e1));
  uint32_t herr = 0;
  CUDACHECK(cudaMemcpy(&herr, err, 4, cudaMemcpyDeviceToHost));
  cudaEventDestroy(e0); cudaEventDestroy(e1);
  cudaStreamDestroy(s); cudaStreamDestroy(sEcho);
  cudaFree(words); cudaFree(err); cudaFreeHost(hostWord);
  if (res != ncclSuccess) return res;
  if (herr) { DF_WARN("stream round-trip probe: a wait ran out (%u)", herr); return dfcclTimeout; }
  *usOut = (double)ms * 1e3 / iters;
  return ncclSuccess;
}

// ---------------------------------------------------------------------------------------------------------------
// What single memory operations of the daemon's control path cost on this machine, measured by one thread with the
// nanosecond timer: reads and writes of pinned host memory (every one crosses PCIe), fences of the three scopes
// after stores to device and to host memory, a device-memory atomic.  Results in nanoseconds per operation:
//   [0] ld.relaxed.sys of a host word          [1] st to a host word (posted), no fence
//   [2] st host word + fence.sys               [3] st device word + fence.sys
//   [4] st device word + fence.gpu             [5] fence.sys with nothing outstanding
//   [6] atomicAdd on a device word             [7] ld.relaxed.sys of a device word, loads independent of one another
//   [8] st device word + fence.acq_rel.sys     [9] st device word + fence.acq_rel.gpu
//   [10] ld.relaxed.sys of a device word, each load's address depending on the previous value (a round trip)
//   [11] st.release.sys to a device word       [12] one read of the nanosecond timer
namespace dfccl {
namespace {
__global__ void probeMemOpsKernel(volatile uint64_t* host, volatile uint64_t* dev, int iters, uint64_t* out) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  uint64_t acc = 0, t0, t1;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) acc += ld_relaxed_sys_u64(host);
  t1 = df_now_ns(); out[0] = (t1 - t0) / iters;
  __threadfence_system();
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) st_relaxed_sys_u64(host + 8, (uint64_t)i);
  t1 = df_now_ns(); out[1] = (t1 - t0) / iters;
  __threadfence_system();
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) { st_relaxed_sys_u64(host + 8, (uint64_t)i); __threadfence_system(); }
  t1 = df_now_ns(); out[2] = (t1 - t0) / iters;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) { st_relaxed_sys_u64(dev + 8, (uint64_t)i); __threadfence_system(); }
  t1 = df_now_ns(); out[3] = (t1 - t0) / iters;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) { st_relaxed_sys_u64(dev + 8, (uint64_t)i); __threadfence(); }
  t1 = df_now_ns(); out[4] = (t1 - t0) / iters;
  __threadfence_system();
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) __threadfence_system();
  t1 = df_now_ns(); out[5] = (t1 - t0) / iters;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) acc += atomicAdd((unsigned long long*)(dev + 16), 1ull);
  t1 = df_now_ns(); out[6] = (t1 - t0) / iters;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) acc += ld_relaxed_sys_u64(dev + 24);
  t1 = df_now_ns(); out[7] = (t1 - t0) / iters;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) { st_relaxed_sys_u64(dev + 8, (uint64_t)i); asm volatile("fence.acq_rel.sys;" ::: "memory"); }
  t1 = df_now_ns(); out[8] = (t1 - t0) / iters;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) { st_relaxed_sys_u64(dev + 8, (uint64_t)i); asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
  t1 = df_now_ns(); out[9] = (t1 - t0) / iters;
  uint64_t idx = 0;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) idx = ld_relaxed_sys_u64(dev + 32 + (idx & 1));      // both words hold 0: a dependent chain
  t1 = df_now_ns(); out[10] = (t1 - t0) / iters;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) st_release_sys_u64(dev + 8, (uint64_t)i);
  t1 = df_now_ns(); out[11] = (t1 - t0) / iters;
  t0 = df_now_ns();
  for (int i = 0; i < iters; ++i) acc += df_now_ns();
  t1 = df_now_ns(); out[12] = (t1 - t0) / iters;
  out[13] = acc + idx;
}
}  // namespace
}  // namespace dfccl

extern "C" __attribute__((visibility("default")))
ncclResult_t dfcclProbeMemoryOps(int iters, uint64_t nsOut[13]) {
  if (!nsOut || iters < 1 || iters > 10000) return ncclInvalidArgument;
  uint64_t *host = nullptr, *dev = nullptr, *out = nullptr;
  CUDACHECK(cudaHostAlloc((void**)&host, 256, cudaHostAllocMapped));
  memset(host, 0, 256);
  CUDACHECK(cudaMalloc((void**)&dev, 512));
  CUDACHECK(cudaMemset(dev, 0, 512));
  CUDACHECK(cudaMalloc((void**)&out, 14 * sizeof(uint64_t)));
  probeMemOpsKernel<<<1, 32>>>(host, dev, 8, out);          // warm-up
  probeMemOpsKernel<<<1, 32>>>(host, dev, iters, out);
  uint64_t h[14];
  cudaError_t e = cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
  cudaFree(dev); cudaFree(out); cudaFreeHost(host);
  if (e != cudaSuccess) { (void)cudaGetLastError(); return ncclUnhandledCudaError; }
  for (int i = 0; i < 13; ++i) nsOut[i] = h[i];
  return ncclSuccess;
}
