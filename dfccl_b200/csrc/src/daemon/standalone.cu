// Stream-ordered execution of one collective: a plain kernel on the caller's stream
// that runs the same step engine as the daemon (device/engine.h), with waits that
// are retried until a time limit instead of being preempted.
#include "../device/daemon_impl.h"
#include "../device/launch.h"
#include "../common/log.h"

namespace dfccl {

__global__ void __launch_bounds__(512, 1) dfcclCollKernel(RankDev* rd, CollStatic cs, uint64_t send, uint64_t recv,
                                                            uint32_t epoch, uint32_t sqeFlags) {
  __shared__ BlockShared sh;
  standaloneBlockMain(rd, blockIdx.x, &sh, &cs, send, recv, epoch, sqeFlags);
}

ncclResult_t launchStandaloneCuda(RankDev* rd, const CollStatic& cs, uint64_t send, uint64_t recv, uint32_t epoch,
                                  uint32_t sqeFlags, int threads, cudaStream_t stream) {
  dfcclCollKernel<<<cs.nBlocks, threads, 0, stream>>>(rd, cs, send, recv, epoch, sqeFlags);
  CUDACHECK(cudaGetLastError());
  return ncclSuccess;
}

ncclResult_t warmDaemonKernel();
ncclResult_t warmRuntimeKernels() {
  cudaFuncAttributes a;
  CUDACHECK(cudaFuncGetAttributes(&a, dfcclCollKernel));
  return warmDaemonKernel();
}

}  // namespace dfccl
