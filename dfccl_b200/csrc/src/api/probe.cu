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
