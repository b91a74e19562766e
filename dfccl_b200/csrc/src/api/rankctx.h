// Rank context of the register-then-submit interface and the host threads around
// the daemon.
//
// Reference counterparts: struct ofcclRankCtx (src/include/enqueue_ofccl.h:95-173),
// prepare / finalize (src/enqueue_ofccl.cc:750-845,1284-1557), sqWrite / cqRead
// (:616-739), the poller thread (:908-965), the kernel-launching observer thread
// (:847-906,967-985) and destroy (:1581-1662).  What is kept: the life cycle, the
// two host threads and their roles, the relaunch handshake through a count of
// outstanding submissions.  What is new: a launcher object that several rank
// contexts of one device share (their daemons are one kernel), completion entries
// that validate themselves by a generation number instead of a host-side CAS on
// pinned memory, stream-ordered submit / wait through stream memory operations,
// per-collective status and a blocking wait, statistics, host-side fault hooks.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>
#include "../comm/comm.h"
#include "../device/types.h"

namespace dfccl {

struct CollEntry {
  dfcclCollInfo info{};
  ncclComm* comm = nullptr;
  CollStatic cs{};
  uint64_t flagsOff = 0, flagsBytes = 0;
  uint64_t pushOff = 0, pushBytes = 0;       // slots of the push schedule (small all-reduces)
  uint64_t stagingOff[2] = {0, 0}, stagingBytes[2] = {0, 0};
  CallbackFunc cb = nullptr;
  void* cbArgs = nullptr;
  uint64_t submitted = 0, completed = 0;     // guarded by ctx->mu
  uint64_t triggerSeq = 0;
  uint32_t lastStatus = 0;
  std::shared_ptr<NetRing> ring;             // network-mode communicators: this collective's own ring of connections
  // fused tensor-parallel operator (dfcclPrepareFusedGemm): one heap block per member holds its rendezvous words,
  // counters and receive areas; the daemon never sees these ids
  dfcclFusedInfo fused{};                    // kind == 0: an ordinary collective
  uint64_t fusedOff = 0, fusedBytes = 0;
  uint64_t peerFusedOff[DF_MAX_RANKS] = {};
};

// Workers of the network path.  Every submission in flight needs a thread of its own (two ranks may submit the
// same two collectives in opposite orders, so nothing may queue behind a blocked one); threads are created when
// more jobs are in flight than workers exist and are kept for the life of the context, so that a training run
// costs as many threads as it has collectives in flight at once, not one per submission.
struct NetWorkers {
  std::mutex mu;
  std::condition_variable cv;
  std::deque<std::function<void()>> jobs;
  std::vector<std::thread> threads;
  int idle = 0;
  bool stop = false;
  bool post(std::function<void()> job);       // false: no thread could be created
  void shutdown();
};

struct DaemonLauncher {
  dfcclBackend_t backend = dfcclBackendCuda;
  int device = 0;
  int expected = 1;                          // rank contexts that must attach before the first launch
  int blocks = 1, threads = 1;
  std::vector<ofcclRankCtx*> members;
  std::vector<ofcclRankCtx*> retired;        // destroyed members of a shared daemon, released with the launcher
  RankDev** devTable = nullptr;              // device array of RankDev* (host array on the host backend)
  cudaStream_t stream = nullptr;
  std::thread observer;
  std::mutex mu;
  std::condition_variable cv;
  bool wake = false, stop = false, started = false;
  uint64_t launches = 0;
  ~DaemonLauncher();
};

}  // namespace dfccl

struct ofcclRankCtx {
  int rank = 0, device = 0;
  dfcclBackend_t backend = dfcclBackendCuda;
  bool deviceChosen = false, finalized = false, destroyed = false;
  std::map<int, dfccl::CollEntry> colls;
  int maxCollId = -1;
  // queues (pinned)
  uint64_t sqTail = 0;                         // entries pushed into the device ring so far (guarded by mu)
  uint64_t sqMinFrontier = 0;                  // lower bound of what every block has consumed (refreshed when the ring looks full)
  volatile uint64_t* hostFrontier = nullptr;   // pinned, [nBlocks]: written by the blocks
  cudaStream_t sqStream = nullptr;             // carries nothing but the memory operations that fill the device ring
  uint32_t* devAbort = nullptr;                // device word the daemon polls for an abort request
  volatile uint64_t* hostCq = nullptr;
  dfccl::DaemonCtl* ctl = nullptr;
  uint32_t sqCap = 0, cqCap = 0;
  uint64_t cqHead = 0;
  // device side
  dfccl::RankDev rdHost{};
  dfccl::RankDev* rdDev = nullptr;
  int nBlocks = 1;
  int wantBlocks = 0, wantThreads = 0;   // dfcclSetDaemonGeometry; 0 = environment / default
  // threads
  std::shared_ptr<dfccl::DaemonLauncher> launcher;
  int launcherSlot = 0;
  bool holdOnWait = true;                     // dfcclStreamWait keeps an instance of the daemon resident (see dfcclSetHoldOnWait)
  std::thread poller;
  dfccl::NetWorkers netWorkers;               // submissions on network-mode communicators run here
  std::vector<dfccl::CollEntry*> byId;        // collId -> entry (built at finalize: no tree walk on the hot path)
  std::atomic<int64_t> netPending{0};         // submissions running on the host network path (not the daemon's business)
  std::mutex mu;                      // submissions, callbacks table, counters
  std::condition_variable pollCv;     // poller sleeps here while nothing is outstanding
  std::condition_variable doneCv;     // dfcclWait
  std::atomic<int64_t> remaining{0};  // submissions without a delivered completion
  std::atomic<int64_t> untriggered{0};// of those, stream-ordered ones whose stream has not reached the trigger yet
  std::atomic<bool> stopPoller{false};
  int64_t checkInterval = 10000;      // CHECK_REMAINING_SQE_INTERVAL
  // stats / faults
  std::atomic<uint64_t> sqes{0}, cqes{0}, cbs{0}, sqFull{0}, fusedLaunches{0};
  int64_t faultDrop = 0, faultDelayUs = 0, faultFreezeMs = 0;
  ncclResult_t asyncError = ncclSuccess;
  // stream memory operations (cuda backend)
  void* fnWrite64 = nullptr;
  void* fnWait64 = nullptr;
  void* fnBatch = nullptr;
  // host-visible mirror of the trigger words: the stream writes both, the poller watches the mirror and
  // wakes the launcher when a released submission finds the daemon parked
  volatile uint64_t* hostTrig = nullptr;                    // pinned, [maxColls]
  std::vector<std::pair<int, uint64_t>> pendingTrig;        // (collId, value) not yet seen in the mirror; guarded by mu
  // wake-up path of stream-ordered submits: an event after the trigger, a side stream that waits for it
  // and runs the host function, so that the caller's stream never waits for a CPU thread
  cudaStream_t wakeStream = nullptr;
  std::vector<cudaEvent_t> wakeEvents;
  uint64_t wakeTurn = 0;
};
