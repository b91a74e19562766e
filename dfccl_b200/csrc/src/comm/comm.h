// Communicator object behind ncclComm_t.
//
// Same user-visible role as the reference's ncclComm (src/include/comm.h:88-213,
// created by src/init.cc:907-990): rank / size / device, rendezvous, error state,
// user reduction ops.  What it owns is different: instead of channels, rings,
// trees, proxy threads and per-peer connectors it holds the mapping of every
// member's symmetric heap plus one small block of flag words for the
// stream-ordered collectives, because every collective here is direct loads and
// stores on peer memory.
#pragma once
#include <memory>
#include <mutex>
#include <vector>
#include "dfccl.h"
#include "../bootstrap/bootstrap.h"
#include "../device/types.h"
#include "../mem/heap.h"
#include "../mem/mcast.h"
#include "../net/net.h"

namespace dfccl {
struct DaemonLauncher;

// Ranks of one process that share a device (or are all on the host backend) and
// therefore one daemon launch.
struct LoopGroup {
  int nranks = 0;
  int device = 0;
  dfcclBackend_t backend = dfcclBackendCuda;
  std::shared_ptr<DaemonLauncher> launcher;
  std::mutex mu;
};

struct UserRedOp { bool live = false; double scalar = 1.0; };

}  // namespace dfccl

struct ncclComm {
  int rank = 0, nranks = 1, device = 0;
  dfcclBackend_t backend = dfcclBackendCuda;
  uint64_t commHash = 0;
  std::shared_ptr<dfccl::Bootstrap> boot;
  dfccl::Heap* heap = nullptr;
  bool ownsHeap = false;
  std::vector<dfccl::HeapHandle> handles;
  std::vector<char*> peerHeap;                 // heap base of every member as mapped here
  // stream-ordered engine
  dfccl::RankDev* saRd = nullptr;              // device copy (host memory on the host backend)
  dfccl::RankDev saRdHost{};
  dfccl::DaemonCtl* ctl = nullptr;             // pinned
  uint64_t saFlagsOff = 0;
  std::vector<uint64_t> peerSaFlagsOff;
  uint64_t p2pFlagsOff = 0;
  std::vector<uint64_t> peerP2pFlagsOff;
  std::vector<uint32_t> sendSeq, recvSeq;      // per peer
  uint64_t pushOff = 0, pushSlotBytes = 0;     // slots of the push schedule of the stream-ordered entry points
  std::vector<uint64_t> peerPushOff;
  uint64_t scratchOff[2] = {0, 0};             // staging for buffers outside the heap (send, recv)
  uint64_t scratchBytes[2] = {0, 0};
  uint32_t opCount = 0;
  uint32_t splitCount = 0;
  std::mutex mu;
  ncclResult_t asyncError = ncclSuccess;
  std::vector<dfccl::UserRedOp> userOps;
  std::shared_ptr<dfccl::LoopGroup> loop;      // set for loopback / InitAll groups
  bool aborted = false;
  dfccl::NvlsArena* nvls = nullptr;            // switch-multicast arena (opt-in), null when absent
  // network mode: members that cannot map each other's memory (other hosts, or DFCCL_FORCE_NET=1);
  // collectives are staged through host memory and run over rings of network connections
  bool netMode = false;
  // bounce mode: GPUs of one host without peer access; the heap is registered host shared memory that every member
  // maps, and the schedules run on it unchanged (no multicast arena, no fused tensor-core operators)
  bool shmMode = false;
  std::unique_ptr<dfccl::NetRing> netRing;     // ring of the stream-ordered entry points
};

namespace dfccl {

// heap selection: `inherit` (a parent's heap, for split) > a private heap > the process heap of the device
ncclResult_t commCreate(std::shared_ptr<Bootstrap> boot, dfcclBackend_t backend, int device, bool privateHeap,
                        std::shared_ptr<LoopGroup> loop, ncclComm** out, Heap* inherit = nullptr);
ncclResult_t commDestroy(ncclComm* comm);
dfcclBackend_t defaultBackend();
void setDefaultBackend(dfcclBackend_t b);
int daemonThreads(dfcclBackend_t be);
int daemonBlocks(dfcclBackend_t be);
// Reduction operator bookkeeping shared by both interfaces: maps ncclAvg / user ops to (op, scale, postDiv).
ncclResult_t resolveRedOp(ncclComm* comm, ncclRedOp_t op, ncclDataType_t type, int nranks, int* devOp, double* scale, int* postDiv);
// Heap of (backend, device), created on first use and shared by all communicators of the process.
ncclResult_t processHeap(dfcclBackend_t backend, int device, Heap** out);

// Small all-reduces go out in one hop (push schedule) unless a schedule was pinned or DFCCL_PUSH=0.
bool pushEligible(const ncclComm* comm, int kind, size_t bytes, int pinnedAlgo);
size_t pushMaxBytes();

// Can this all-reduce run on the NVLS schedule of this communicator?  (arena present, sum, supported types, 16-byte multiple)
bool nvlsEligible(const ncclComm* comm, int kind, int inType, int outType, int devOp, int postDiv, size_t count);

// Network mode: copy the operands to the host, run the ring algorithm over `ring`, copy the result back.
// `stream` (cuda backend) is drained first; the call returns when the result is in `recv`.
ncclResult_t netStagedCollective(ncclComm* comm, NetRing* ring, const NetCollDesc& d, const void* send, void* recv, cudaStream_t stream);

// Reduce-scatter (sum; f32 / bf16 / f16) and all-gather on the multimem schedule: only when pinned at registration.
bool nvlsEligibleRsAg(const ncclComm* comm, int kind, int inType, int outType, int devOp, int postDiv, size_t count);

// The engine behind the stream-ordered entry points.
ncclResult_t commCollective(ncclComm* comm, int kind, const void* send, void* recv, size_t count, ncclDataType_t type,
                            ncclRedOp_t op, int root, cudaStream_t stream);

}  // namespace dfccl
