// The allocation-free entry point declared in dfccl_noalloc.h: the stream-ordered
// collective kernel, restricted to one rank, with all of its scratch in a static
// device array.  Nothing in this file calls cudaMalloc, cudaFree, cudaHostAlloc or any
// routine of the library that does (no communicator, no heap).
#include "dfccl_noalloc.h"
#include "../common/log.h"
#include "../device/daemon_impl.h"
#include <cstring>
#include <mutex>

namespace dfccl {
namespace {

constexpr int kMaxBlocks = 16;
// layout of the array (offsets in bytes); everything below kStageSend is control state
constexpr size_t kRdOff = 0;                                        // RankDev
constexpr size_t kCtlOff = 4096;                                    // DaemonCtl
constexpr size_t kDynOff = 8192;                                    // CollDyn[kMaxBlocks]
constexpr size_t kFlagsOff = 16384;                                 // FlagSlot[kMaxBlocks]
constexpr size_t kHeaderBytes = 64u << 10;
constexpr size_t kStageSend = kHeaderBytes;
constexpr size_t kStageRecv = kHeaderBytes + DFCCL_NOALLOC_MAX_BYTES;
static_assert(sizeof(RankDev) <= kCtlOff - kRdOff, "control block does not fit");
static_assert(sizeof(CollDyn) * kMaxBlocks <= kFlagsOff - kDynOff, "per-block state does not fit");
static_assert(sizeof(FlagSlot) * kMaxBlocks <= kHeaderBytes - kFlagsOff, "flag words do not fit");
static_assert(kStageRecv + DFCCL_NOALLOC_MAX_BYTES == DFCCL_NOALLOC_SCRATCH_BYTES, "array size and layout disagree");

// The scratch itself.  In host code this name is only a handle for cudaGetSymbolAddress;
// the device address obtained there is what kernels receive.
static __device__ __align__(256) unsigned char g_noallocScratch[DFCCL_NOALLOC_SCRATCH_BYTES];

__global__ void __launch_bounds__(512, 1) dfcclNoAllocKernel(unsigned char* scratch, CollStatic cs, uint64_t send,
                                                              uint64_t recv, uint32_t epoch, uint32_t sqeFlags) {
  __shared__ BlockShared sh;
  standaloneBlockMain((RankDev*)(scratch + kRdOff), blockIdx.x, &sh, &cs, send, recv, epoch, sqeFlags);
}

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char* g_base[kMaxDevices];        // device address of the array, per device, once set up
uint32_t g_epoch[kMaxDevices];

// Once per device, with that device current: find the array, clear its control words, write the
// control block.  Synchronous copies into existing memory only.
ncclResult_t setUp(int dev, unsigned char** out) {
  std::lock_guard<std::mutex> l(g_mu);
  if (g_base[dev]) { *out = g_base[dev]; return ncclSuccess; }
  unsigned char* ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_noallocScratch);
  if (e != cudaSuccess || ptr == nullptr) {
    DF_WARN("dfcclAllReduceNoAlloc: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
    (void)cudaGetLastError();
    return ncclUnhandledCudaError;
  }
  CUDACHECK(cudaMemset(ptr, 0, kHeaderBytes));
  RankDev rd;
  memset(&rd, 0, sizeof(rd));
  rd.ctl = (DaemonCtl*)(ptr + kCtlOff);
  rd.dyn = (CollDyn*)(ptr + kDynOff);
  rd.nBlocks = kMaxBlocks;
  rd.maxColls = 1;
  rd.spinBudget = 4096;
  rd.headTries = 1;
  rd.waitTimeoutNs = 1000000000ull;          // one rank never waits; the limit is there all the same
  CUDACHECK(cudaMemcpy(ptr + kRdOff, &rd, sizeof(rd), cudaMemcpyHostToDevice));
  cudaFuncAttributes fa;                      // load the kernel now rather than at its first launch
  CUDACHECK(cudaFuncGetAttributes(&fa, dfcclNoAllocKernel));
  // The clear and the copy above ran on the legacy default stream; the caller's stream may be a non-blocking one
  // that is not ordered after it.  Wait here (allocates nothing) so that no kernel can start before the control
  // block is in place.
  CUDACHECK(cudaDeviceSynchronize());
  g_base[dev] = ptr;
  *out = ptr;
  return ncclSuccess;
}

}  // namespace
}  // namespace dfccl

using namespace dfccl;

extern "C" __attribute__((visibility("default")))
ncclResult_t dfcclAllReduceNoAlloc(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype,
                                   float scale, cudaStream_t stream) {
  if (!sendbuff || !recvbuff) { DF_WARN("dfcclAllReduceNoAlloc: null buffer"); return ncclInvalidArgument; }
  if ((int)datatype < 0 || (int)datatype >= ncclNumTypes) { DF_WARN("dfcclAllReduceNoAlloc: invalid datatype %d", (int)datatype); return ncclInvalidArgument; }
  if (count == 0) return ncclSuccess;
  const size_t bytes = count * (size_t)dtypeSize(datatype);
  if (bytes > DFCCL_NOALLOC_MAX_BYTES || bytes / (size_t)dtypeSize(datatype) != count) {
    DF_WARN("dfcclAllReduceNoAlloc: %zu bytes requested, the static scratch serves at most %u bytes per call", bytes, DFCCL_NOALLOC_MAX_BYTES);
    return ncclInvalidArgument;
  }
  int dev = 0;
  CUDACHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ncclInvalidArgument;
  unsigned char* base = nullptr;
  DFCHECK(setUp(dev, &base));
  CollStatic cs;
  memset(&cs, 0, sizeof(cs));
  cs.kind = dfcclCollAllReduce; cs.inType = cs.outType = datatype; cs.op = OP_SUM;
  cs.nranks = 1; cs.rank = 0; cs.root = 0; cs.algo = dfcclAlgoOneShot; cs.valid = 1;
  cs.scale = (double)scale; cs.count = count;
  int nb = (int)(bytes / (256u << 10));
  cs.nBlocks = nb < 1 ? 1 : nb > kMaxBlocks ? kMaxBlocks : nb;
  cs.stagingSendOff = kStageSend; cs.stagingRecvOff = kStageRecv;     // "heap" offsets are offsets into the array
  cs.peerHeap[0] = (char*)base;
  cs.myFlags = (FlagSlot*)(base + kFlagsOff);
  cs.peerFlags[0] = cs.myFlags;
  uint32_t epoch;
  { std::lock_guard<std::mutex> l(g_mu); epoch = ++g_epoch[dev]; }
  dfcclNoAllocKernel<<<cs.nBlocks, 512, 0, stream>>>(base, cs, (uint64_t)(uintptr_t)sendbuff, (uint64_t)(uintptr_t)recvbuff,
                                                     epoch, SQE_SEND_STAGED | SQE_RECV_STAGED);
  CUDACHECK(cudaGetLastError());
  return ncclSuccess;
}

// Status word of the calls made so far on the current device: 0, or the CollStatus of the first kernel that gave
// up (the kernels keep it in the array's control block).  Reads four bytes with a synchronous copy; it reports on
// every kernel that has finished by then, so synchronise the streams you care about first.  Allocates nothing.
extern "C" __attribute__((visibility("default")))
ncclResult_t dfcclNoAllocStatus(uint32_t* status) {
  if (!status) return ncclInvalidArgument;
  int dev = 0;
  CUDACHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return ncclInvalidArgument;
  unsigned char* base = nullptr;
  { std::lock_guard<std::mutex> l(g_mu); base = g_base[dev]; }
  *status = 0;
  if (!base) return ncclSuccess;              // no call was made on this device yet
  DaemonCtl ctl;
  CUDACHECK(cudaMemcpy(&ctl, base + kCtlOff, sizeof(ctl), cudaMemcpyDeviceToHost));
  *status = ctl.pad;
  return ncclSuccess;
}
