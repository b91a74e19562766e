// Kernel entry points of the device runtime.  All logic lives in the shared
// headers (device/daemon_impl.h, device/engine.h, device/datapath.h); this file
// only binds them to __global__ functions for sm_100a.
#include "../device/daemon_impl.h"
#include "../device/launch.h"
#include "../common/log.h"

namespace dfccl {

__global__ void __launch_bounds__(512, 1) dfcclDaemonKernel(RankDev** ranks, int blocksPerRank) {
  __shared__ BlockShared sh;
  const int vr = blockIdx.x / blocksPerRank, b = blockIdx.x % blocksPerRank;
  daemonBlockMain(ranks[vr], b, &sh);
}

ncclResult_t launchDaemonCuda(RankDev** devRankTable, int nRanks, int blocksPerRank, int threads, cudaStream_t stream) {
  dim3 grid(nRanks * blocksPerRank), block(threads);
  if (nRanks > 1) {
    void* args[] = {&devRankTable, &blocksPerRank};
    CUDACHECK(cudaLaunchCooperativeKernel((void*)dfcclDaemonKernel, grid, block, args, 0, stream));
  } else {
    dfcclDaemonKernel<<<grid, block, 0, stream>>>(devRankTable, blocksPerRank);
    CUDACHECK(cudaGetLastError());
  }
  return ncclSuccess;
}

ncclResult_t warmDaemonKernel() {
  cudaFuncAttributes a;
  CUDACHECK(cudaFuncGetAttributes(&a, dfcclDaemonKernel));
  return ncclSuccess;
}

ncclResult_t daemonMaxResidentBlocks(int device, int threads, int* blocks) {
  int perSm = 0, sms = 0;
  CUDACHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&perSm, dfcclDaemonKernel, threads, 0));
  CUDACHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
  *blocks = perSm * sms;
  return ncclSuccess;
}

}  // namespace dfccl
