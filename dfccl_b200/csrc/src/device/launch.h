// Host-callable launchers of the device runtime (CUDA) and of its host-thread twin.
#pragma once
#include "types.h"
#include "dfccl.h"

namespace dfccl {

// Persistent daemon for `nRanks` rank contexts that share one device: one launch,
// grid = nRanks * blocksPerRank.  With more than one rank the launch is cooperative,
// so that all blocks are co-resident (blocks of different ranks wait on one another).
ncclResult_t launchDaemonCuda(RankDev** devRankTable, int nRanks, int blocksPerRank, int threads, cudaStream_t stream);

// One collective as a plain kernel on the caller's stream (stream-ordered nccl* interface).
ncclResult_t launchStandaloneCuda(RankDev* rd, const CollStatic& cs, uint64_t send, uint64_t recv, uint32_t epoch,
                                  uint32_t sqeFlags, int threads, cudaStream_t stream);

// Force the lazily loaded kernels of the runtime into the context (no launch).
ncclResult_t warmRuntimeKernels();

// Largest grid of the daemon kernel that is guaranteed co-resident on `device`.
ncclResult_t daemonMaxResidentBlocks(int device, int threads, int* blocks);

// Host backend: the same code with one OS thread per block.  Both calls block until
// every "block" has returned.
void runDaemonHost(RankDev** rankTable, int nRanks, int blocksPerRank);
void runStandaloneHost(RankDev* rd, const CollStatic& cs, uint64_t send, uint64_t recv, uint32_t epoch, uint32_t sqeFlags);

}  // namespace dfccl
