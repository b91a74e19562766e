#include "rankctx.h"
#include "../common/nvtx.h"
#include "../common/log.h"
#include "../common/param.h"
#include "../device/datapath.h"
#include "../device/engine.h"
#include "../device/launch.h"
#include "../topo/topo.h"
#include "../gemm/gemm.h"
#include <algorithm>
#include <chrono>
#include <cstring>
#include <cuda.h>
#include <fstream>

using namespace dfccl;

#define DF_API extern "C" __attribute__((visibility("default")))

static ncclResult_t launchFromCaller(ofcclRankCtx* ctx);     // defined with the stream-ordered entry points below

namespace dfccl {

__global__ void dfcclWriteWordKernel(volatile uint64_t* p, uint64_t v) {
  __threadfence_system();
  *p = v;
}

// Fallback of the wake-up path when stream memory operations are unavailable: a host function (on a
// side stream) publishes the host mirror of a trigger word once the caller's stream has passed the
// trigger.  Normally the stream writes the mirror itself (see submit).
static void CUDART_CB triggerReached(void* arg) {
  auto* p = (std::pair<ofcclRankCtx*, std::pair<int, uint64_t>>*)arg;
  __atomic_store_n((uint64_t*)&p->first->hostTrig[p->second.first], p->second.second, __ATOMIC_RELEASE);
  delete p;
}

// Stream-ordered release of a trigger word that can be captured in a CUDA graph: the word counts the releases of
// its collective, so a replayed launch releases the next submission whatever its number is.
__global__ void dfcclBumpWordKernel(volatile uint64_t* word, volatile uint64_t* mirror) {
  __threadfence_system();                // what this stream's kernels produced, before the release
  const uint64_t v = *word + 1;
  *word = v;
  if (mirror) *mirror = v;
}

// Fallback of the ring fill when stream memory operations are unavailable: one thread writes the entry, then the tail.
__global__ void dfcclPushSqeKernel(Sqe* slot, Sqe q, volatile uint64_t* tail, uint64_t newTail) {
  *slot = q;
  __threadfence_system();
  *tail = newTail;
}

// Append one entry to the device-resident submission ring (caller holds ctx->mu).  The host writes the ring: four
// 64-bit words of the entry and then the tail, as one batch of stream memory operations on a stream that carries
// nothing else, so the daemon finds its work in device memory.  (The reference's daemon polls a ring in pinned host
// memory, src/collectives_ofccl/device/enqueue_ofccl_dev.cu:85-173; here a load of host memory by a block costs a
// PCIe round trip, and such loads from tens of blocks queue behind one another.)
static ncclResult_t pushSqe(ofcclRankCtx* ctx, const Sqe& q) {
  const uint64_t tail = ctx->sqTail;
  Sqe* slot = ctx->rdHost.devSq + (tail & (ctx->sqCap - 1));
  volatile uint64_t* tailWord = (volatile uint64_t*)((char*)ctx->rdDev + offsetof(RankDev, devSqTail));
  if (ctx->backend != dfcclBackendCuda) {
    *slot = q;
    __atomic_store_n((uint64_t*)tailWord, tail + 1, __ATOMIC_RELEASE);
  } else if (ctx->fnBatch) {
    typedef CUresult (*Fn)(CUstream, unsigned int, CUstreamBatchMemOpParams*, unsigned int);
    uint64_t w[4];
    memcpy(w, &q, sizeof(w));
    CUstreamBatchMemOpParams ops[5];
    memset(ops, 0, sizeof(ops));
    for (int i = 0; i < 4; ++i) {
      ops[i].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_64;
      ops[i].writeValue.address = (CUdeviceptr)(uintptr_t)((uint64_t*)slot + i);
      ops[i].writeValue.value64 = w[i];
    }
    ops[4].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_64;      // every write is preceded by a fence: the entry is there before the tail
    ops[4].writeValue.address = (CUdeviceptr)(uintptr_t)tailWord;
    ops[4].writeValue.value64 = tail + 1;
    CUresult r = ((Fn)ctx->fnBatch)((CUstream)ctx->sqStream, 5, ops, 0);
    if (r != CUDA_SUCCESS) { DF_WARN("cuStreamBatchMemOp failed (%d)", (int)r); return ncclUnhandledCudaError; }
  } else {
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != ctx->device) cudaSetDevice(ctx->device);
    dfcclPushSqeKernel<<<1, 1, 0, ctx->sqStream>>>(slot, q, tailWord, tail + 1);
    cudaError_t e = cudaGetLastError();
    if (prev != ctx->device) cudaSetDevice(prev);
    if (e != cudaSuccess) { DF_WARN("submission ring fill failed: %s", cudaGetErrorString(e)); return ncclUnhandledCudaError; }
  }
  ctx->sqTail = tail + 1;
  return ncclSuccess;
}

// Entries the slowest block has consumed, as the blocks report it (pinned words they store to).
static uint64_t minFrontier(ofcclRankCtx* ctx) {
  uint64_t m = ~0ull;
  for (int b = 0; b < ctx->nBlocks; ++b) m = std::min<uint64_t>(m, __atomic_load_n((const uint64_t*)&ctx->hostFrontier[b], __ATOMIC_ACQUIRE));
  return m;
}

bool NetWorkers::post(std::function<void()> job) {
  std::lock_guard<std::mutex> l(mu);
  jobs.push_back(std::move(job));
  if ((int)jobs.size() > idle) {
    try {
      threads.emplace_back([this] {
        std::unique_lock<std::mutex> lk(mu);
        for (;;) {
          ++idle;
          cv.wait(lk, [&] { return stop || !jobs.empty(); });
          --idle;
          if (jobs.empty()) return;              // stop, and nothing left to run
          std::function<void()> j = std::move(jobs.front());
          jobs.pop_front();
          lk.unlock();
          j();
          lk.lock();
        }
      });
    } catch (const std::system_error&) {
      if ((int)jobs.size() > idle) { jobs.pop_back(); return false; }     // nobody would ever run it
    }
  }
  cv.notify_one();
  return true;
}

void NetWorkers::shutdown() {
  std::vector<std::thread> ts;
  {
    std::lock_guard<std::mutex> l(mu);
    stop = true;
    ts.swap(threads);
  }
  cv.notify_all();
  for (auto& t : ts) if (t.joinable()) t.join();
}

static uint32_t pow2ceil(uint32_t v) { uint32_t p = 1; while (p < v) p <<= 1; return p; }

DaemonLauncher::~DaemonLauncher() {
  {
    std::lock_guard<std::mutex> l(mu);
    stop = true;
    cv.notify_all();
  }
  if (observer.joinable()) observer.join();
  if (backend == dfcclBackendCuda) {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(device);
    if (stream) { cudaStreamSynchronize(stream); cudaStreamDestroy(stream); }
    if (devTable) cudaFree(devTable);
    (void)cudaGetLastError();
    cudaSetDevice(prev);
  } else {
    ::free(devTable);
  }
}

static void wakeLauncher(DaemonLauncher* L) {
  std::lock_guard<std::mutex> l(L->mu);
  L->wake = true;
  L->cv.notify_all();
}

// Launches (and relaunches) the daemon: the reference's observer thread.
static void observerMain(DaemonLauncher* L) {
  if (L->backend == dfcclBackendCuda) cudaSetDevice(L->device);
  std::unique_lock<std::mutex> lk(L->mu);
  for (;;) {
    L->cv.wait(lk, [&] { return L->wake || L->stop; });
    if (L->stop) break;
    L->wake = false;
    std::vector<ofcclRankCtx*> members = L->members;
    std::vector<ofcclRankCtx*> everyone = L->members;       // the launch table also names retired ranks
    everyone.insert(everyone.end(), L->retired.begin(), L->retired.end());
    lk.unlock();
    // the previous instance must be completely gone: its blocks park state the next one restores
    if (L->backend == dfcclBackendCuda) {
      cudaError_t e = cudaStreamSynchronize(L->stream);
      if (e != cudaSuccess) {
        DF_WARN("daemon kernel failed: %s", cudaGetErrorString(e));
        for (auto* m : members) m->asyncError = ncclUnhandledCudaError;
        lk.lock();
        break;
      }
    }
    bool work = false, dead = false;
    for (auto* m : members) {
      if ((ctl_load(&m->ctl->hold) ? m->remaining.load() : m->remaining.load() - m->untriggered.load()) - m->netPending.load() > 0 && !ctl_load(&m->ctl->finalQuit)) work = true;
      if (ctl_load(&m->ctl->abortFlag)) dead = true;
    }
    if (work && !dead) {
      for (auto* m : everyone) { ctl_store(&m->ctl->alive, 1); m->ctl->launches = m->ctl->launches + 1; }
      std::atomic_thread_fence(std::memory_order_seq_cst);
      ++L->launches;
      DF_TRACE(SUB_DAEMON, "daemon launch #%llu (%zu ranks x %d blocks x %d threads)", (unsigned long long)L->launches, members.size(), L->blocks, L->threads);
      if (L->backend == dfcclBackendCuda) {
        ncclResult_t r = launchDaemonCuda(L->devTable, L->expected, L->blocks, L->threads, L->stream);
        if (r != ncclSuccess) for (auto* m : members) m->asyncError = r;
      } else {
        runDaemonHost(L->devTable, L->expected, L->blocks);     // returns when every block has left
        for (auto* m : members) if (m->remaining.load() - m->untriggered.load() - m->netPending.load() > 0 && !ctl_load(&m->ctl->finalQuit) && !ctl_load(&m->ctl->abortFlag)) { lk.lock(); L->wake = true; lk.unlock(); break; }
      }
    }
    lk.lock();
  }
}

static void deliver(ofcclRankCtx* ctx, uint64_t entry) {
  const int coll = (int)cqeColl(entry);
  CallbackFunc cb = nullptr;
  void* args = nullptr;
  {
    std::lock_guard<std::mutex> l(ctx->mu);
    CollEntry* e = coll >= 0 && coll < (int)ctx->byId.size() ? ctx->byId[coll] : nullptr;
    if (!e) { DF_WARN("completion for unknown collective %d", coll); return; }
    e->lastStatus = cqeStatus(entry);
    if (e->lastStatus != ST_OK && ctx->asyncError == ncclSuccess)
      ctx->asyncError = e->lastStatus == ST_TIMEOUT ? dfcclTimeout : e->lastStatus == ST_ABORTED ? dfcclAborted : ncclInternalError;
    cb = e->cb; args = e->cbArgs;
  }
  ctx->cqes++;
  if (ctx->faultFreezeMs > 0) std::this_thread::sleep_for(std::chrono::milliseconds(ctx->faultFreezeMs));
  if (cb) { cb(coll, args); ctx->cbs++; }
  {
    std::lock_guard<std::mutex> l(ctx->mu);
    { uint64_t* w = &ctx->byId[coll]->completed; __atomic_store_n(w, *w + 1, __ATOMIC_RELEASE); }   // also read lock-free by spinning waiters
    ctx->remaining--;
    if (ctx->remaining.load() == 0) ctl_store(&ctx->ctl->hold, 0);
  }
  ctx->doneCv.notify_all();
}

// Short waits are polled (yielding the CPU, dropping the lock between looks) before the caller is put to
// sleep on the condition variable: being woken costs tens of microseconds, a completion usually arrives sooner.
template <typename Quick, typename Pred>
static bool spinFirst(std::unique_lock<std::mutex>& l, Quick quick, Pred pred, int spins = 4000) {
  if (pred()) return true;
  l.unlock();                                   // `quick` reads atomics only: the poller is not slowed by lock traffic
  for (int i = 0; i < spins && !quick(); ++i) sched_yield();
  l.lock();
  return pred();
}

// Turns completion entries into callbacks: the reference's poller thread.
static void pollerMain(ofcclRankCtx* ctx) {
  logSetRank(ctx->rank);
  // this thread may launch the daemon: bind it to the context's device once (switching devices back and forth around
  // a launch would make the runtime create a context on whatever device the thread started with)
  if (ctx->backend == dfcclBackendCuda) cudaSetDevice(ctx->device);
  int64_t empty = 0;
  int idleSpins = 0;
  while (!ctx->stopPoller.load()) {
    if (ctx->remaining.load() == 0) {
      // stay awake for a moment: a caller that submits again right away then finds nobody to wake (waking a
      // sleeping thread costs the submitter a system call)
      if (++idleSpins < 4000) { sched_yield(); continue; }
      std::unique_lock<std::mutex> l(ctx->mu);
      ctx->pollCv.wait_for(l, std::chrono::milliseconds(20), [&] { return ctx->remaining.load() > 0 || ctx->stopPoller.load(); });
      continue;
    }
    idleSpins = 0;
    if (ctx->untriggered.load() > 0) {          // stream-ordered submissions whose release has not been seen yet
      int fired = 0;
      std::unique_lock<std::mutex> l(ctx->mu, std::try_to_lock);     // never make a submitting thread wait for this scan
      if (l.owns_lock()) {
        auto& pt = ctx->pendingTrig;
        for (size_t i = 0; i < pt.size();) {
          if (__atomic_load_n((const uint64_t*)&ctx->hostTrig[pt[i].first], __ATOMIC_ACQUIRE) >= pt[i].second) { pt[i] = pt.back(); pt.pop_back(); ++fired; }
          else ++i;
        }
        l.unlock();
      }
      if (fired) {
        ctx->untriggered -= fired;
        if (!ctl_load(&ctx->ctl->alive) && !ctl_load(&ctx->ctl->abortFlag)) {
          // a released submission found the daemon parked: launch it from this thread (it is awake and has just seen
          // the release; handing over to the observer thread would add a thread wake-up to the collective's latency)
          if (ctx->backend == dfcclBackendCuda && ctx->launcher->expected == 1) { if (::launchFromCaller(ctx) != ncclSuccess) wakeLauncher(ctx->launcher.get()); }
          else wakeLauncher(ctx->launcher.get());
        }
      }
    }
    const uint64_t slot = ctx->cqHead & (ctx->cqCap - 1);
    const uint64_t e = __atomic_load_n((const uint64_t*)&ctx->hostCq[slot], __ATOMIC_ACQUIRE);
    if (cqeGen(e) == (uint32_t)(ctx->cqHead / ctx->cqCap) + 1u) {
      ++ctx->cqHead;
      empty = 0;
      deliver(ctx, e);
      continue;
    }
    // nothing new: if the daemon left while work is outstanding, have it launched again
    if (++empty % ctx->checkInterval == 0 || (empty & 63) == 0) {
      const int64_t ready = (ctl_load(&ctx->ctl->hold) ? ctx->remaining.load() : ctx->remaining.load() - ctx->untriggered.load()) - ctx->netPending.load();
      if (!ctl_load(&ctx->ctl->alive) && ready > 0 && !ctl_load(&ctx->ctl->abortFlag)) wakeLauncher(ctx->launcher.get());
    }
    if (empty > 2000) std::this_thread::sleep_for(std::chrono::microseconds(20)); else sched_yield();
  }
}

static ncclResult_t checkInfo(const dfcclCollInfo* info, ncclComm* comm) {
  if (!info || !comm) { DF_WARN("null argument"); return ncclInvalidArgument; }
  if (info->kind < 0 || info->kind >= dfcclCollNumKinds) { DF_WARN("invalid collective kind %d", info->kind); return ncclInvalidArgument; }
  if ((int)info->inType < 0 || (int)info->inType >= ncclNumTypes || (int)info->outType < 0 || (int)info->outType >= ncclNumTypes) { DF_WARN("invalid datatype"); return ncclInvalidArgument; }
  if (info->root < 0 || info->root >= comm->nranks) { DF_WARN("invalid root %d", info->root); return ncclInvalidArgument; }
  const bool reduces = info->kind == dfcclCollAllReduce || info->kind == dfcclCollReduce || info->kind == dfcclCollReduceScatter;
  if (!reduces && info->inType != info->outType) { DF_WARN("only reducing collectives can cast"); return ncclInvalidArgument; }
  return ncclSuccess;
}

}  // namespace dfccl

// ------------------------------------------------------------------ life cycle

DF_API ncclResult_t dfcclInitRankCtxOnDevice(ofcclRankCtx_t* out, int rank, int device) {
  if (!out) return ncclInvalidArgument;
  auto* ctx = new ofcclRankCtx();
  ctx->rank = rank; ctx->device = device; ctx->deviceChosen = device >= 0;
  ctx->backend = defaultBackend();
  *out = ctx;
  return ncclSuccess;
}
DF_API ncclResult_t dfcclSetDaemonGeometry(ofcclRankCtx_t ctx, int blocks, int threads) {
  if (!ctx || ctx->finalized) return ncclInvalidUsage;
  if (blocks < 0 || blocks > DF_MAX_BLOCKS || threads < 0 || threads > 512 || (threads % 32) != 0) return ncclInvalidArgument;
  ctx->wantBlocks = blocks; ctx->wantThreads = threads;
  return ncclSuccess;
}
DF_API ncclResult_t ofcclInitRankCtx(ofcclRankCtx_t* out, int rank) { return dfcclInitRankCtxOnDevice(out, rank, -1); }

DF_API ncclResult_t dfcclPrepare(const dfcclCollInfo* info, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) {
  if (!ctx) return ncclInvalidArgument;
  DFCHECK(checkInfo(info, comm));
  std::lock_guard<std::mutex> l(ctx->mu);
  if (ctx->finalized) { DF_WARN("collective %d registered after the context was finalized", collId); return ncclInvalidUsage; }
  if (collId < 0 || collId >= DF_MAX_COLLS) { DF_WARN("collective id %d outside [0, %d)", collId, DF_MAX_COLLS); return ncclInvalidArgument; }
  if (ctx->colls.count(collId)) { DF_WARN("collective id %d registered twice", collId); return ncclInvalidUsage; }
  if (!ctx->colls.empty() && ctx->colls.begin()->second.comm->backend != comm->backend) { DF_WARN("all collectives of a context must use one backend"); return ncclInvalidUsage; }
  if (!ctx->colls.empty() && ctx->colls.begin()->second.comm->device != comm->device) { DF_WARN("all collectives of a context must use communicators of one device"); return ncclInvalidUsage; }
  CollEntry e;
  e.info = *info;
  e.comm = comm;
  int devOp = OP_SUM;
  double scale = 1.0;
  int postDiv = 0;
  const bool reduces = info->kind == dfcclCollAllReduce || info->kind == dfcclCollReduce || info->kind == dfcclCollReduceScatter;
  if (reduces) DFCHECK(resolveRedOp(comm, info->op, info->inType, comm->nranks, &devOp, &scale, &postDiv));
  if (info->scale != 0.f && info->scale != 1.f) scale *= (double)info->scale;
  if (reduces && !reduceSupported(info->inType, info->outType, devOp)) { DF_WARN("no kernel for type %d -> %d with operator %d", (int)info->inType, (int)info->outType, (int)info->op); return ncclInvalidArgument; }
  CollStatic& cs = e.cs;
  memset(&cs, 0, sizeof(cs));
  cs.kind = info->kind; cs.inType = info->inType; cs.outType = info->outType; cs.op = devOp;
  cs.nranks = comm->nranks; cs.rank = comm->rank; cs.root = info->root; cs.count = info->count;
  cs.scale = scale; cs.postDiv = postDiv;
  ctx->colls[collId] = e;
  ctx->maxCollId = std::max(ctx->maxCollId, collId);
  if (paramI64("SHOW_ALL_PREPARED_COLL", 0)) DF_WARN("prepared coll %d kind %d count %zu type %d->%d", collId, info->kind, info->count, (int)info->inType, (int)info->outType);
  return ncclSuccess;
}

// ---- fused tensor-parallel operators: one zeroed heap block per member, laid out alike on all of them
struct FusedLayout { uint64_t arrive, done, doneCount, epochCounter, flags, big, bytes; };
static FusedLayout fusedLayout(const dfcclFusedInfo& f, int n) {
  FusedLayout L{};
  L.arrive = 0; L.done = 8ull * n; L.doneCount = 16ull * n; L.epochCounter = 16ull * n + 8;
  L.flags = (16ull * n + 16 + 63) & ~63ull;
  const uint64_t m = (uint64_t)f.rowsPerRank * n;
  // all-gather -> GEMM: one counter per 128-row block of the gathered operand, then the operand itself [M, k];
  // GEMM -> reduce-scatter: one flag per (source rank, tile of my rows), then the receive areas [n][rowsPerRank, N]
  const uint64_t nFlags = f.kind == dfcclFusedAllGatherGemm ? m / GEMM_BM : (uint64_t)n * (f.rowsPerRank / GEMM_BM) * (f.n / GEMM_BN);
  L.big = (L.flags + 4 * nFlags + 1023) & ~1023ull;
  L.bytes = L.big + (f.kind == dfcclFusedAllGatherGemm ? m * f.k * 2 : (uint64_t)n * f.rowsPerRank * f.n * 2);
  return L;
}

DF_API ncclResult_t dfcclPrepareFusedGemm(const dfcclFusedInfo* info, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) {
  if (!ctx || !info || !comm) return ncclInvalidArgument;
  if (info->kind != dfcclFusedAllGatherGemm && info->kind != dfcclFusedGemmReduceScatter) { DF_WARN("unknown fused operator kind %d", info->kind); return ncclInvalidArgument; }
  if (info->rowsPerRank <= 0 || info->k <= 0 || info->n <= 0 || info->rowsPerRank % GEMM_BM || info->k % GEMM_BK || info->n % GEMM_BN) {
    DF_WARN("fused operator %d: rows per rank, k and n must be positive multiples of %d, %d and %d (got %d, %d, %d)", collId, GEMM_BM, GEMM_BK, GEMM_BN, info->rowsPerRank, info->k, info->n);
    return ncclInvalidArgument;
  }
  if (comm->nranks > 8) { DF_WARN("fused operators serve communicators of up to 8 ranks"); return ncclInvalidArgument; }
  if (comm->netMode || comm->shmMode) { DF_WARN("fused operators need peer memory: not available on communicators that go through host memory"); return ncclInvalidUsage; }
  std::lock_guard<std::mutex> l(ctx->mu);
  if (ctx->finalized) { DF_WARN("operator %d registered after the context was finalized", collId); return ncclInvalidUsage; }
  if (collId < 0 || collId >= DF_MAX_COLLS) return ncclInvalidArgument;
  if (ctx->colls.count(collId)) { DF_WARN("collective id %d registered twice", collId); return ncclInvalidUsage; }
  if (!ctx->colls.empty() && ctx->colls.begin()->second.comm->backend != comm->backend) return ncclInvalidUsage;
  if (!ctx->colls.empty() && ctx->colls.begin()->second.comm->device != comm->device) return ncclInvalidUsage;
  CollEntry e;
  e.comm = comm;
  e.fused = *info;
  memset(&e.cs, 0, sizeof(e.cs));
  // the registration check at finalize compares these fields across the members
  e.cs.kind = 100 + info->kind; e.cs.count = (uint64_t)info->rowsPerRank; e.cs.inType = info->k; e.cs.outType = info->n;
  e.cs.nranks = comm->nranks; e.cs.rank = comm->rank;
  ctx->colls[collId] = e;
  ctx->maxCollId = std::max(ctx->maxCollId, collId);
  return ncclSuccess;
}

struct FinalizeMsg { int32_t collId, nBlocks, algo, kind, inType, outType, pad0, pad1; uint64_t count, flagsOff, pushOff; };

DF_API ncclResult_t ofcclFinalizeRankCtx7StartHostThrds(ofcclRankCtx_t ctx) {
  if (!ctx) return ncclInvalidArgument;
  NvtxRange range("dfccl:finalize");
  if (ctx->finalized) { DF_WARN("context finalized twice"); return ncclInvalidUsage; }
  if (ctx->colls.empty()) { DF_WARN("no collective registered"); return ncclInvalidUsage; }
  ncclComm* first = ctx->colls.begin()->second.comm;
  ctx->backend = first->backend;
  ctx->device = first->device;
  const dfcclBackend_t be = ctx->backend;
  int prevDev = 0;
  if (be == dfcclBackendCuda) { cudaGetDevice(&prevDev); CUDACHECK(cudaSetDevice(ctx->device)); }
  logSetRank(ctx->rank);
  ctx->nBlocks = ctx->wantBlocks > 0 ? std::min(ctx->wantBlocks, DF_MAX_BLOCKS) : daemonBlocks(be);
  ctx->checkInterval = std::max<int64_t>(1, paramI64("CHECK_REMAINING_SQE_INTERVAL", 10000));
  const Topology* topo = nullptr;
  DFCHECK(topoGet(&topo));

  // 1. schedule + flag words of every collective
  for (auto& kv : ctx->colls) {
    CollEntry& e = kv.second;
    if (e.comm->netMode) continue;               // runs on the host over its own ring (created in step 2)
    if (e.fused.kind) {                          // rendezvous words, counters and receive areas of a fused operator
      e.fusedBytes = fusedLayout(e.fused, e.comm->nranks).bytes;
      DFCHECK(e.comm->heap->alloc(e.fusedBytes, &e.fusedOff, true));
      e.flagsOff = e.fusedOff;
      continue;
    }
    const size_t bytes = e.info.count * (size_t)dtypeSize(e.info.inType);
    bool nv = nvlsEligible(e.comm, e.cs.kind, e.cs.inType, e.cs.outType, e.cs.op, e.cs.postDiv, e.cs.count);
    TunerChoice ch = tunerChoose(*topo, e.info.kind, bytes, e.comm->nranks, ctx->nBlocks, nv, e.info.algo, e.info.nBlocks);
    // reduce-scatter, all-gather and broadcast take the multimem schedule only when it is pinned at registration
    if (e.info.algo == dfcclAlgoNvls && nvlsEligibleRsAg(e.comm, e.cs.kind, e.cs.inType, e.cs.outType, e.cs.op, e.cs.postDiv, e.cs.count)) ch.algo = dfcclAlgoNvls;
    if (ch.algo == dfcclAlgoNvls) {
      // staging slots in the arena; every member walks its collectives in id order, so the offsets agree.
      // (the output of a reduce-scatter and the input of an all-gather or broadcast are local to the rank and need no slot)
      NvlsArena* a = e.comm->nvls;
      const bool inPlace = (e.info.flags & DFCCL_COLL_ARENA_BUFFERS) != 0;      // the caller's buffers are arena memory: no slots
      const size_t inB = e.cs.kind == dfcclCollAllGather || e.cs.kind == dfcclCollBroadcast || inPlace ? 0 : sendBytes(&e.cs);
      const size_t outB = e.cs.kind == dfcclCollReduceScatter || inPlace ? 0 : recvBytes(&e.cs);
      uint64_t in = 0, out = 0;
      if ((inB == 0 || a->alloc(inB, &in) == ncclSuccess) && (outB == 0 || a->alloc(outB, &out) == ncclSuccess)) {
        e.cs.mcHeap = a->mc; e.cs.nvlsPeers = a->peersDev; e.cs.nvlsIn = in; e.cs.nvlsOut = out;
        e.cs.stagingSendOff = (uint64_t)(a->uc + in - e.comm->heap->base());
        e.cs.stagingRecvOff = (uint64_t)(a->uc + out - e.comm->heap->base());
      } else {
        DF_INFO(SUB_TUNING, "collective %d: NVLS arena full, using peer loads and stores", kv.first);
        ch = tunerChoose(*topo, e.info.kind, bytes, e.comm->nranks, ctx->nBlocks, false, e.info.algo == dfcclAlgoNvls ? dfcclAlgoAuto : e.info.algo, e.info.nBlocks);
      }
    }
    e.cs.algo = ch.algo; e.cs.nBlocks = ch.nBlocks;
    // collectives too small for every block start at different blocks, so that their fixed costs (flag round trips,
    // completion) spread over the daemon instead of queueing on its first blocks
    e.cs.blockBase = ch.nBlocks < ctx->nBlocks ? (int32_t)((((uint32_t)kv.first * 0x9E3779B1u) >> 16) % (uint32_t)ctx->nBlocks) : 0;
    if (ch.algo != dfcclAlgoNvls && pushEligible(e.comm, e.cs.kind, bytes, e.info.algo)) {
      // small all-reduce, all-gather or reduce-scatter: one hop through slots at the peers ([2 parities][n writers]
      // [piece + 16 bytes: a reduce-scatter chunk keeps its misalignment]); a pure function of what every member
      // registered, so all members decide alike
      e.cs.algo = dfcclAlgoPush;
      e.cs.pushSlotBytes = (bytes + 16 + 511) & ~(size_t)511;
      e.pushBytes = 2 * (size_t)e.comm->nranks * e.cs.pushSlotBytes;
      DFCHECK(e.comm->heap->alloc(e.pushBytes, &e.pushOff, false));
    }
    e.flagsBytes = sizeof(FlagSlot) * (size_t)ch.nBlocks * e.comm->nranks;
    DFCHECK(e.comm->heap->alloc(e.flagsBytes, &e.flagsOff, true));
  }
  // 2. exchange, communicator by communicator in an order all ranks agree on (smallest id first)
  std::vector<std::pair<int, ncclComm*>> order;
  for (auto& kv : ctx->colls) {
    bool seen = false;
    for (auto& o : order) if (o.second == kv.second.comm) seen = true;
    if (!seen) order.push_back({kv.first, kv.second.comm});
  }
  for (auto& oc : order) {
    ncclComm* comm = oc.second;
    std::vector<int> ids;
    for (auto& kv : ctx->colls) if (kv.second.comm == comm) ids.push_back(kv.first);
    const int n = comm->nranks;
    std::vector<int32_t> cnt(n, 0);
    cnt[comm->rank] = (int32_t)ids.size();
    DFCHECK(comm->boot->allGather(cnt.data(), sizeof(int32_t)));
    for (int j = 0; j < n; ++j) if (cnt[j] != (int32_t)ids.size()) { DF_WARN("rank %d registered %d collectives on this communicator, rank %d registered %zu", j, cnt[j], comm->rank, ids.size()); return ncclInvalidUsage; }
    if (comm->netMode) {
      // one ring of connections per collective (ascending id on every member): collectives submitted in
      // different orders on different ranks then never meet in one FIFO
      for (int id : ids) {
        std::unique_ptr<NetRing> ring;
        DFCHECK(NetRing::create(comm->boot.get(), &ring));
        ctx->colls[id].ring = std::shared_ptr<NetRing>(ring.release());
        ctx->colls[id].cs.valid = 0;             // the daemon never sees it
      }
      continue;
    }
    std::vector<FinalizeMsg> all((size_t)n * ids.size());
    for (size_t i = 0; i < ids.size(); ++i) {
      CollEntry& e = ctx->colls[ids[i]];
      all[(size_t)comm->rank * ids.size() + i] = {ids[i], e.cs.nBlocks, e.cs.algo, e.cs.kind, e.cs.inType, e.cs.outType, 0, 0, e.cs.count, e.flagsOff, e.pushOff};
    }
    DFCHECK(comm->boot->allGather(all.data(), sizeof(FinalizeMsg) * ids.size()));
    for (size_t i = 0; i < ids.size(); ++i) {
      CollEntry& e = ctx->colls[ids[i]];
      e.cs.myFlags = (FlagSlot*)(comm->heap->base() + e.flagsOff);
      for (int j = 0; j < n; ++j) {
        const FinalizeMsg& m = all[(size_t)j * ids.size() + i];
        if (m.collId != ids[i] || m.kind != e.cs.kind || m.count != e.cs.count || m.inType != e.cs.inType || m.outType != e.cs.outType || m.nBlocks != e.cs.nBlocks || m.algo != e.cs.algo) {
          DF_WARN("collective %d is registered differently on rank %d", ids[i], j);
          return ncclInvalidUsage;
        }
        e.cs.peerHeap[j] = comm->peerHeap[j];
        e.cs.peerFlags[j] = (FlagSlot*)(comm->peerHeap[j] + m.flagsOff);
        e.cs.peerPush[j] = e.pushBytes ? comm->peerHeap[j] + m.pushOff : nullptr;
        e.peerFusedOff[j] = m.flagsOff;
      }
      e.cs.valid = e.fused.kind ? 0 : 1;         // fused operators are stream kernels: the daemon never sees their ids
    }
  }
  if (be == dfcclBackendCuda)
    for (auto& kv : ctx->colls) if (kv.second.fused.kind) { gemmReserveSmsAtLeast(ctx->nBlocks); break; }   // all CTAs of a fused launch must be resident beside the daemon
  // 3. queues and device tables
  const uint32_t maxColls = (uint32_t)ctx->maxCollId + 1;
  ctx->byId.assign(maxColls, nullptr);
  for (auto& kv : ctx->colls) ctx->byId[kv.first] = &kv.second;
  ctx->sqCap = pow2ceil(std::max<uint32_t>(64, 2 * (uint32_t)ctx->colls.size() + 2));
  ctx->cqCap = pow2ceil(std::max<uint32_t>(64, 2 * (uint32_t)ctx->colls.size() + 2));
  DFCHECK(pinnedAlloc(be, (void**)&ctx->hostFrontier, sizeof(uint64_t) * ctx->nBlocks));
  DFCHECK(pinnedAlloc(be, (void**)&ctx->hostCq, sizeof(uint64_t) * ctx->cqCap));
  DFCHECK(pinnedAlloc(be, (void**)&ctx->ctl, sizeof(DaemonCtl)));
  DFCHECK(pinnedAlloc(be, (void**)&ctx->hostTrig, sizeof(uint64_t) * ((size_t)ctx->maxCollId + 1)));
  RankDev& rd = ctx->rdHost;
  memset(&rd, 0, sizeof(rd));
  rd.hostFrontier = ctx->hostFrontier;
  if (be == dfcclBackendCuda) { DFCHECK(devAlloc(be, (void**)&ctx->devAbort, 64)); rd.abortWord = ctx->devAbort; }
  else rd.abortWord = &ctx->ctl->abortFlag;
  rd.hostCq = ctx->hostCq; rd.ctl = ctx->ctl;
  rd.sqCap = ctx->sqCap; rd.cqCap = ctx->cqCap; rd.nBlocks = (uint32_t)ctx->nBlocks; rd.maxColls = maxColls;
  DFCHECK(devAlloc(be, (void**)&rd.devSq, sizeof(Sqe) * ctx->sqCap));
  DFCHECK(devAlloc(be, (void**)&rd.colls, sizeof(CollStatic) * maxColls));
  DFCHECK(devAlloc(be, (void**)&rd.dyn, sizeof(CollDyn) * (size_t)maxColls * ctx->nBlocks));
  DFCHECK(devAlloc(be, (void**)&rd.doneCount, sizeof(uint32_t) * maxColls));
  DFCHECK(devAlloc(be, (void**)&rd.failCount, sizeof(uint32_t) * maxColls));
  DFCHECK(devAlloc(be, (void**)&rd.doneEpoch, sizeof(uint64_t) * maxColls));
  DFCHECK(devAlloc(be, (void**)&rd.trigger, sizeof(uint64_t) * maxColls));
  DFCHECK(devAlloc(be, (void**)&rd.saved, sizeof(BlockSaved) * ctx->nBlocks));
  DFCHECK(devAlloc(be, (void**)&rd.stats, sizeof(DevStats) * ctx->nBlocks));
  if (paramI64("TRACE", 0)) {
    rd.traceCap = pow2ceil((uint32_t)paramI64("TRACE_EVENTS", 1 << 16));
    DFCHECK(devAlloc(be, (void**)&rd.trace, sizeof(TraceEvent) * rd.traceCap));
  }
  // tunables; the un-prefixed names are the reference's (src/enqueue_ofccl.cc:1287-1297)
  rd.spinBudget = (uint32_t)std::max<int64_t>(1, paramI64("BASE_CTX_SWITCH_THRESHOLD", 32));
  rd.headTries = (uint32_t)std::max<int64_t>(1, paramI64("NUM_TRY_TASKQ_HEAD", 5));
  rd.recvSuccessFactor = (uint32_t)paramI64("RECV_SUCCESS_FACTOR", 5);
  const int64_t tolerant = paramI64("TOLERANT_UNPROGRESSED_CNT", 0);     // polls in the reference; here ~1 us each
  rd.idleQuitNs = (uint64_t)paramI64("IDLE_QUIT_US", tolerant ? tolerant : 1000) * 1000ull;
  rd.stallQuitNs = (uint64_t)paramI64("STALL_QUIT_US", tolerant ? tolerant : 5000) * 1000ull;
  rd.trigQuitNs = (uint64_t)paramI64("TRIGGER_QUIT_US", (int64_t)(rd.idleQuitNs / 1000)) * 1000ull;
  rd.waitTimeoutNs = (uint64_t)paramI64("WAIT_TIMEOUT_MS", 0) * 1000000ull;
  rd.maxLifetimeNs = (uint64_t)paramI64("MAX_LIFETIME_MS", 2000) * 1000000ull;
  // a block's data phase is left after this many bytes when other work is queued (the reference parks a
  // collective at its 1 MiB slices: src/include/collectives.h:112-113)
  rd.sliceBytes = (uint64_t)std::max<int64_t>(0, paramI64("SLICE_BYTES", 1 << 20));
  std::vector<CollStatic> table(maxColls);
  memset(table.data(), 0, sizeof(CollStatic) * maxColls);
  for (auto& kv : ctx->colls) table[kv.first] = kv.second.cs;
  DFCHECK(devUpload(be, rd.colls, table.data(), sizeof(CollStatic) * maxColls));
  DFCHECK(devAlloc(be, (void**)&ctx->rdDev, sizeof(RankDev)));
  DFCHECK(devUpload(be, ctx->rdDev, &rd, sizeof(RankDev)));
  if (be == dfcclBackendCuda) {
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue64", &ctx->fnWrite64, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) ctx->fnWrite64 = nullptr;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue64", &ctx->fnWait64, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) ctx->fnWait64 = nullptr;
    (void)cudaGetLastError();
    if (paramI64("NO_STREAM_MEMOPS", 0)) ctx->fnWrite64 = ctx->fnWait64 = nullptr;
    if (cudaGetDriverEntryPoint("cuStreamBatchMemOp", &ctx->fnBatch, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) ctx->fnBatch = nullptr;
    (void)cudaGetLastError();
    if (!ctx->fnWrite64) ctx->fnBatch = nullptr;
    CUDACHECK(cudaStreamCreateWithFlags(&ctx->wakeStream, cudaStreamNonBlocking));
    { int lo = 0, hi = 0; cudaDeviceGetStreamPriorityRange(&lo, &hi); CUDACHECK(cudaStreamCreateWithPriority(&ctx->sqStream, cudaStreamNonBlocking, hi)); }
    ctx->wakeEvents.resize(256);
    for (auto& e : ctx->wakeEvents) CUDACHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  }
  // 4. launcher: shared by the ranks of a loopback group, private otherwise
  std::shared_ptr<LoopGroup> loop = first->loop;
  {
    std::shared_ptr<DaemonLauncher> L;
    if (loop) {
      std::lock_guard<std::mutex> l(loop->mu);
      if (!loop->launcher) { loop->launcher = std::make_shared<DaemonLauncher>(); loop->launcher->expected = loop->nranks; }
      L = loop->launcher;
    } else {
      L = std::make_shared<DaemonLauncher>();
      L->expected = 1;
    }
    std::lock_guard<std::mutex> l(L->mu);
    L->backend = be; L->device = ctx->device; L->blocks = ctx->nBlocks;
    L->threads = (be == dfcclBackendCuda && ctx->wantThreads > 0) ? ctx->wantThreads : daemonThreads(be);
    ctx->launcherSlot = (int)L->members.size();
    L->members.push_back(ctx);
    ctx->launcher = L;
    if ((int)L->members.size() == L->expected) {
      std::vector<RankDev*> tab;
      for (auto* m : L->members) tab.push_back(m->rdDev);
      if (be == dfcclBackendCuda) {
        int lo = 0, hi = 0;
        cudaDeviceGetStreamPriorityRange(&lo, &hi);
        CUDACHECK(cudaStreamCreateWithPriority(&L->stream, cudaStreamNonBlocking, hi));
        CUDACHECK(cudaMalloc((void**)&L->devTable, sizeof(RankDev*) * tab.size()));
        CUDACHECK(cudaMemcpy(L->devTable, tab.data(), sizeof(RankDev*) * tab.size(), cudaMemcpyHostToDevice));
        if (L->expected > 1) {
          int maxb = 0;
          DFCHECK(daemonMaxResidentBlocks(ctx->device, L->threads, &maxb));
          if (L->expected * L->blocks > maxb) { DF_WARN("%d ranks x %d blocks do not fit on device %d together (%d resident blocks); lower DFCCL_DAEMON_BLOCKS", L->expected, L->blocks, ctx->device, maxb); return ncclInvalidUsage; }
        }
      } else {
        L->devTable = (RankDev**)malloc(sizeof(RankDev*) * tab.size());
        memcpy(L->devTable, tab.data(), sizeof(RankDev*) * tab.size());
      }
      if (be == dfcclBackendCuda) {
        // First launch now, while nothing depends on the daemon.  CUDA loads kernels lazily and the
        // first launch of this one grows the context's local-memory pool, which needs an idle
        // device: done later, with a user stream already blocked on a flag only the daemon sets,
        // that launch (and every launch queued behind it) would never start.  With no submission
        // pending every block leaves after the idle limit.
        DFCHECK(warmRuntimeKernels());
        cudaFuncAttributes fa;
        CUDACHECK(cudaFuncGetAttributes(&fa, dfcclWriteWordKernel));
        for (auto* m : L->members) ctl_store(&m->ctl->alive, 1);
        DFCHECK(launchDaemonCuda(L->devTable, L->expected, L->blocks, L->threads, L->stream));
        CUDACHECK(cudaStreamSynchronize(L->stream));
        for (auto* m : L->members) ctl_store(&m->ctl->alive, 0);
      }
      L->started = true;
      L->observer = std::thread(observerMain, L.get());
    }
  }
  ctx->poller = std::thread(pollerMain, ctx);
  ctx->finalized = true;
  if (be == dfcclBackendCuda) { CUDACHECK(cudaDeviceSynchronize()); cudaSetDevice(prevDev); }
  DF_INFO(SUB_INIT, "rank context %d finalized: %zu collectives, %d daemon blocks", ctx->rank, ctx->colls.size(), ctx->nBlocks);
  return ncclSuccess;
}

DF_API ncclResult_t ofcclPrepareDone(ofcclRankCtx_t ctx) {
  DFCHECK(ofcclFinalizeRankCtx7StartHostThrds(ctx));
  return ncclSuccess;          // the daemon starts with the first submission; an idle daemon would only hold SMs
}

// ------------------------------------------------------------------ submit

// How a submission is released to the daemon.
enum SubmitMode {
  SUBMIT_HOST = 0,        // at once
  SUBMIT_STREAM = 1,      // by a stream memory operation enqueued now, after the work already in `stream`
  SUBMIT_DEFERRED = 2,    // by a later dfcclTriggerOnStream (or by the replay of a graph that captured one)
};

static ncclResult_t submit(ofcclRankCtx* ctx, const void* send, void* recv, int collId, CallbackFunc cb, void* cbArgs,
                           SubmitMode mode, cudaStream_t stream) {
  if (!ctx || !ctx->finalized || ctx->destroyed) { DF_WARN("context is not ready for submissions"); return ncclInvalidUsage; }
  const bool onStream = mode != SUBMIT_HOST;
  NvtxRange range(onStream ? "dfccl:submit(stream)" : "dfccl:submit");
  if (ctl_load(&ctx->ctl->abortFlag)) return dfcclAborted;
  if (ctx->faultDelayUs > 0) std::this_thread::sleep_for(std::chrono::microseconds(ctx->faultDelayUs));
  Sqe q;
  memset(&q, 0, sizeof(q));
  uint64_t trig = 0;
  // A stream-ordered release normally also writes a host-visible mirror of the trigger word, which the poller
  // watches to launch a parked daemon.  While an instance is running and held resident (a stream is parked on one
  // of this context's completions) nobody needs that wake-up: the release is then a single write to device memory -
  // every stream memory operation is preceded by a system-wide fence, so the second write costs as much as the first.
  const bool deferWake = onStream && ctx->backend == dfcclBackendCuda &&
                         !(mode == SUBMIT_STREAM && ctl_load(&ctx->ctl->hold) && ctl_load(&ctx->ctl->alive) && ctx->fnWrite64);
  {
    std::unique_lock<std::mutex> l(ctx->mu);
    CollEntry* ep = collId >= 0 && collId < (int)ctx->byId.size() ? ctx->byId[collId] : nullptr;
    if (!ep) { DF_WARN("collective %d was never prepared", collId); return ncclInvalidArgument; }
    CollEntry& e = *ep;
    if (e.fused.kind) { DF_WARN("id %d is a fused operator: run it with dfcclRunFusedGemm", collId); return ncclInvalidUsage; }
    if (e.submitted != e.completed) {
      if (!onStream) { DF_WARN("collective %d submitted again before its callback ran", collId); return ncclInvalidUsage; }
      // Stream-ordered callers enqueue ahead of the GPU: the previous submission of this id is
      // already ordered before this one on the device, so the host only has to wait for it.
      auto prevDone = [&] { return e.submitted == e.completed || ctl_load(&ctx->ctl->abortFlag); };
      uint64_t* completedWord = &e.completed;
      const uint64_t wantDone = e.submitted;
      const bool ok = spinFirst(l, [&] { return __atomic_load_n(completedWord, __ATOMIC_ACQUIRE) >= wantDone || ctl_load(&ctx->ctl->abortFlag); }, prevDone) ||
                      ctx->doneCv.wait_for(l, std::chrono::seconds(120), prevDone);
      if (!ok) { DF_WARN("collective %d: previous submission did not complete within 120 s", collId); return dfcclTimeout; }
      if (ctl_load(&ctx->ctl->abortFlag)) return dfcclAborted;
    }
    const CollStatic& cs = e.cs;
    const bool needSend = !(cs.kind == dfcclCollBroadcast && cs.rank != cs.root);
    const bool needRecv = !(cs.kind == dfcclCollReduce && cs.rank != cs.root);
    if ((needSend && !send) || (needRecv && !recv)) { DF_WARN("null buffer for collective %d", collId); return ncclInvalidArgument; }
    if (e.comm->netMode) {
      if (onStream) { DF_WARN("collective %d: stream-ordered submission is not available on communicators that go through the network path", collId); return ncclInvalidUsage; }
      NetCollDesc d{cs.kind, cs.inType, cs.outType, cs.op, cs.root, cs.postDiv, cs.scale, (size_t)cs.count};
      ncclComm* comm = e.comm;
      std::shared_ptr<NetRing> ring = e.ring;
      CallbackFunc prevCb = e.cb;
      void* prevArgs = e.cbArgs;
      e.cb = cb; e.cbArgs = cbArgs;
      e.submitted++;
      ctx->remaining++;
      ctx->netPending++;
      ctx->sqes++;
      const bool posted = ctx->netWorkers.post([ctx, comm, ring, d, send, recv, collId] {
        logSetRank(ctx->rank);
        ncclResult_t r = netStagedCollective(comm, ring.get(), d, send, recv, nullptr);
        const uint32_t st = r == ncclSuccess ? ST_OK : r == dfcclAborted ? ST_ABORTED : r == dfcclTimeout ? ST_TIMEOUT : ST_BAD_ARG;
        ctx->netPending--;
        deliver(ctx, ((uint64_t)st << 24) | (uint64_t)(uint32_t)collId);
      });
      if (!posted) {                        // no thread to run it on: undo the bookkeeping, the caller may try again
        e.cb = prevCb; e.cbArgs = prevArgs;
        e.submitted--; ctx->remaining--; ctx->netPending--; ctx->sqes--;
        DF_WARN("collective %d: no worker thread could be created for the network path", collId);
        return ncclSystemError;
      }
      ctx->pollCv.notify_one();
      return ncclSuccess;
    }
    Heap* heap = e.comm->heap;
    const size_t sB = sendBytes(&cs), rB = recvBytes(&cs);
    q.collId = collId;
    const bool viaArena = cs.algo == dfcclAlgoNvls || cs.algo == dfcclAlgoPush;
    if (cs.algo == dfcclAlgoPush) {          // the user's buffers are touched by this rank only: used where they are
      if (heap->contains(send, sB)) q.send = heap->offsetOf(send); else { q.flags |= SQE_SEND_STAGED; q.send = (uint64_t)(uintptr_t)send; }
      if (heap->contains(recv, rB)) q.recv = heap->offsetOf(recv); else { q.flags |= SQE_RECV_STAGED; q.recv = (uint64_t)(uintptr_t)recv; }
    } else if (viaArena) {          // in place when the buffer lives in the arena, else through this collective's slots
      NvlsArena* a = e.comm->nvls;
      if (rawSend(&cs)) { if (heap->contains(send, sB)) q.send = heap->offsetOf(send); else { q.flags |= SQE_SEND_STAGED; q.send = (uint64_t)(uintptr_t)send; } }
      else if (a->contains(send, sB)) q.send = (uint64_t)((const char*)send - a->uc);
      else if (e.info.flags & DFCCL_COLL_ARENA_BUFFERS) { DF_WARN("collective %d was registered for buffers in the multicast arena; this send buffer is not", collId); return ncclInvalidArgument; }
      else { q.flags |= SQE_SEND_STAGED; q.send = (uint64_t)(uintptr_t)send; }
      if (rawRecv(&cs)) { if (heap->contains(recv, rB)) q.recv = heap->offsetOf(recv); else { q.flags |= SQE_RECV_STAGED; q.recv = (uint64_t)(uintptr_t)recv; } }
      else if (a->contains(recv, rB)) q.recv = (uint64_t)((char*)recv - a->uc);
      else if (e.info.flags & DFCCL_COLL_ARENA_BUFFERS) { DF_WARN("collective %d was registered for buffers in the multicast arena; this receive buffer is not", collId); return ncclInvalidArgument; }
      else { q.flags |= SQE_RECV_STAGED; q.recv = (uint64_t)(uintptr_t)recv; }
    }
    bool stageSend = !viaArena && needSend && !heap->contains(send, sB);
    if (needSend && cs.kind == dfcclCollAllReduce && cs.algo == dfcclAlgoOneShot && send == recv && cs.nranks > 1) stageSend = true;
    bool stageRecv = !viaArena && needRecv && !heap->contains(recv, rB);
    // staging areas are created on first need; the static table on the device learns their offsets
    bool tableDirty = false;
    if (stageSend && e.stagingBytes[0] < sB) { if (e.stagingBytes[0]) heap->free(e.stagingOff[0]); DFCHECK(heap->alloc(sB, &e.stagingOff[0], false)); e.stagingBytes[0] = sB; e.cs.stagingSendOff = e.stagingOff[0]; tableDirty = true; }
    if (stageRecv && e.stagingBytes[1] < rB) { if (e.stagingBytes[1]) heap->free(e.stagingOff[1]); DFCHECK(heap->alloc(rB, &e.stagingOff[1], false)); e.stagingBytes[1] = rB; e.cs.stagingRecvOff = e.stagingOff[1]; tableDirty = true; }
    if (tableDirty) DFCHECK(devUpload(ctx->backend, &ctx->rdHost.colls[collId], &e.cs, sizeof(CollStatic)));
    if (!viaArena) {
      if (stageSend) { q.flags |= SQE_SEND_STAGED; q.send = (uint64_t)(uintptr_t)send; } else if (needSend) q.send = heap->offsetOf(send);
      if (stageRecv) { q.flags |= SQE_RECV_STAGED; q.recv = (uint64_t)(uintptr_t)recv; } else if (needRecv) q.recv = heap->offsetOf(recv);
    }
    if (onStream) { q.flags |= SQE_TRIGGERED; q.trigger = trig = ++e.triggerSeq; }
    // flow control: never overwrite an entry some block has not consumed yet
    while (ctx->sqTail - ctx->sqMinFrontier >= ctx->sqCap && (ctx->sqMinFrontier = minFrontier(ctx), ctx->sqTail - ctx->sqMinFrontier >= ctx->sqCap)) {
      ctx->sqFull++;
      l.unlock();
      if (!ctl_load(&ctx->ctl->alive)) wakeLauncher(ctx->launcher.get());
      sched_yield();
      l.lock();
    }
    e.cb = cb; e.cbArgs = cbArgs;
    e.submitted++;
    ctx->remaining++;
    ctx->sqes++;
    if (deferWake) {                   // the poller watches the trigger's host mirror and wakes a parked daemon
      ctx->pendingTrig.emplace_back(collId, trig);
      ctx->untriggered++;
    }
    if (ctx->faultDrop > 0) {          // accepted, counted, never published
      --ctx->faultDrop;
    } else {
      DFCHECK(pushSqe(ctx, q));
    }
  }
  ctx->pollCv.notify_one();
  if (!deferWake && !ctl_load(&ctx->ctl->alive)) wakeLauncher(ctx->launcher.get());
  if (mode == SUBMIT_STREAM) {
    volatile uint64_t* word = ctx->rdHost.trigger + collId;
    if (ctx->backend == dfcclBackendCuda) {
      volatile uint64_t* mirror = ctx->hostTrig + collId;
      if (!deferWake && ctx->fnWrite64) {
        typedef CUresult (*Fn)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);
        CUresult r = ((Fn)ctx->fnWrite64)((CUstream)stream, (CUdeviceptr)(uintptr_t)word, trig, 0);
        if (r != CUDA_SUCCESS) { DF_WARN("cuStreamWriteValue64 failed (%d)", (int)r); return ncclUnhandledCudaError; }
      } else if (ctx->fnBatch) {
        // device trigger word and its host mirror in one driver call
        typedef CUresult (*Fn)(CUstream, unsigned int, CUstreamBatchMemOpParams*, unsigned int);
        CUstreamBatchMemOpParams ops[2];
        memset(ops, 0, sizeof(ops));
        ops[0].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_64;
        ops[0].writeValue.address = (CUdeviceptr)(uintptr_t)word;
        ops[0].writeValue.value64 = trig;
        ops[1].writeValue.operation = CU_STREAM_MEM_OP_WRITE_VALUE_64;
        ops[1].writeValue.address = (CUdeviceptr)(uintptr_t)mirror;
        ops[1].writeValue.value64 = trig;
        CUresult r = ((Fn)ctx->fnBatch)((CUstream)stream, 2, ops, 0);
        if (r != CUDA_SUCCESS) { DF_WARN("cuStreamBatchMemOp failed (%d)", (int)r); return ncclUnhandledCudaError; }
      } else if (ctx->fnWrite64) {
        typedef CUresult (*Fn)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);
        CUresult r = ((Fn)ctx->fnWrite64)((CUstream)stream, (CUdeviceptr)(uintptr_t)word, trig, 0);
        if (r == CUDA_SUCCESS) r = ((Fn)ctx->fnWrite64)((CUstream)stream, (CUdeviceptr)(uintptr_t)mirror, trig, 0);
        if (r != CUDA_SUCCESS) { DF_WARN("cuStreamWriteValue64 failed (%d)", (int)r); return ncclUnhandledCudaError; }
      } else {
        // no stream memory operations: a one-thread kernel writes the word, a host function (on a side
        // stream, so that the caller's stream never waits for a CPU thread) publishes the mirror
        dfcclWriteWordKernel<<<1, 1, 0, stream>>>(word, trig);
        CUDACHECK(cudaGetLastError());
        cudaEvent_t ev;
        { std::lock_guard<std::mutex> l(ctx->mu); ev = ctx->wakeEvents[ctx->wakeTurn++ % ctx->wakeEvents.size()]; }
        CUDACHECK(cudaEventRecord(ev, stream));
        CUDACHECK(cudaStreamWaitEvent(ctx->wakeStream, ev, 0));
        CUDACHECK(cudaLaunchHostFunc(ctx->wakeStream, triggerReached, new std::pair<ofcclRankCtx*, std::pair<int, uint64_t>>(ctx, {collId, trig})));
      }
    } else {
      __atomic_store_n((uint64_t*)word, trig, __ATOMIC_RELEASE);
    }
  }
  return ncclSuccess;
}

DF_API ncclResult_t dfcclRun(const void* s, void* r, int collId, CallbackFunc cb, void* args, ofcclRankCtx_t ctx) {
  return submit(ctx, s, r, collId, cb, args, SUBMIT_HOST, nullptr);
}
DF_API ncclResult_t dfcclRunOnStream(const void* s, void* r, int collId, cudaStream_t stream, CallbackFunc cb, void* args, ofcclRankCtx_t ctx) {
  return submit(ctx, s, r, collId, cb, args, SUBMIT_STREAM, stream);
}
DF_API ncclResult_t dfcclRunDeferred(const void* s, void* r, int collId, CallbackFunc cb, void* args, ofcclRankCtx_t ctx) {
  return submit(ctx, s, r, collId, cb, args, SUBMIT_DEFERRED, nullptr);
}

// Release, in stream order, the oldest submission of `collId` that dfcclRunDeferred published (or will publish: the
// trigger word counts releases, so the order of the two calls does not matter).  The release is a one-thread kernel
// and may be captured in a CUDA graph; every replay releases one more submission.
DF_API ncclResult_t dfcclTriggerOnStream(int collId, cudaStream_t stream, ofcclRankCtx_t ctx) {
  if (!ctx || !ctx->finalized || ctx->destroyed) return ncclInvalidUsage;
  if (collId < 0 || collId >= (int)ctx->byId.size() || !ctx->byId[collId]) return ncclInvalidArgument;
  if (ctx->byId[collId]->comm->netMode || ctx->byId[collId]->fused.kind) return ncclInvalidUsage;
  volatile uint64_t* word = ctx->rdHost.trigger + collId;
  if (ctx->backend == dfcclBackendCuda) {
    dfcclBumpWordKernel<<<1, 1, 0, stream>>>(word, ctx->hostTrig + collId);
    CUDACHECK(cudaGetLastError());
  } else {
    __atomic_fetch_add((uint64_t*)word, 1, __ATOMIC_ACQ_REL);
  }
  return ncclSuccess;
}

DF_API ncclResult_t dfcclWait(int collId, int timeoutMs, ofcclRankCtx_t ctx) {
  if (!ctx || !ctx->finalized) return ncclInvalidUsage;
  std::unique_lock<std::mutex> l(ctx->mu);
  auto it = ctx->colls.find(collId);
  if (it == ctx->colls.end()) return ncclInvalidArgument;
  CollEntry& e = it->second;
  auto pred = [&] { return e.completed == e.submitted || ctl_load(&ctx->ctl->abortFlag); };
  uint64_t* completedWord = &e.completed;
  const uint64_t wantDone = e.submitted;
  if (spinFirst(l, [&] { return __atomic_load_n(completedWord, __ATOMIC_ACQUIRE) >= wantDone || ctl_load(&ctx->ctl->abortFlag); }, pred)) {}
  else if (timeoutMs < 0) ctx->doneCv.wait(l, pred);
  else if (!ctx->doneCv.wait_for(l, std::chrono::milliseconds(timeoutMs), pred)) return dfcclTimeout;
  if (ctl_load(&ctx->ctl->abortFlag) && e.completed != e.submitted) return dfcclAborted;
  return e.lastStatus == ST_OK ? ncclSuccess : e.lastStatus == ST_TIMEOUT ? dfcclTimeout : e.lastStatus == ST_ABORTED ? dfcclAborted : ncclInternalError;
}

DF_API ncclResult_t dfcclWaitAll(int timeoutMs, ofcclRankCtx_t ctx) {
  if (!ctx || !ctx->finalized) return ncclInvalidUsage;
  std::unique_lock<std::mutex> l(ctx->mu);
  auto pred = [&] { return ctx->remaining.load() == 0 || ctl_load(&ctx->ctl->abortFlag); };
  if (spinFirst(l, pred, pred)) {}
  else if (timeoutMs < 0) ctx->doneCv.wait(l, pred);
  else if (!ctx->doneCv.wait_for(l, std::chrono::milliseconds(timeoutMs), pred)) return dfcclTimeout;
  if (ctl_load(&ctx->ctl->abortFlag) && ctx->remaining.load()) return dfcclAborted;
  return ctx->asyncError;
}

// Launch an instance of the daemon from the calling thread (cuda backend).  Launches share one stream, so an
// instance that is still leaving is simply followed by this one; a surplus instance finds nothing and leaves.
static ncclResult_t launchFromCaller(ofcclRankCtx* ctx) {
  DaemonLauncher* L = ctx->launcher.get();
  std::vector<ofcclRankCtx*> everyone;
  {
    std::lock_guard<std::mutex> l(L->mu);
    if (L->stop || ctl_load(&ctx->ctl->alive) || ctl_load(&ctx->ctl->abortFlag) || ctl_load(&ctx->ctl->finalQuit)) return ncclSuccess;
    everyone = L->members;
    everyone.insert(everyone.end(), L->retired.begin(), L->retired.end());
    for (auto* m : everyone) { ctl_store(&m->ctl->alive, 1); m->ctl->launches = m->ctl->launches + 1; }
    ++L->launches;
  }
  std::atomic_thread_fence(std::memory_order_seq_cst);
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != L->device) cudaSetDevice(L->device);
  ncclResult_t r = launchDaemonCuda(L->devTable, L->expected, L->blocks, L->threads, L->stream);
  if (prev != L->device) cudaSetDevice(prev);
  return r;
}

DF_API ncclResult_t dfcclSetHoldOnWait(ofcclRankCtx_t ctx, int on) {
  if (!ctx) return ncclInvalidArgument;
  ctx->holdOnWait = on != 0;
  return ncclSuccess;
}

DF_API ncclResult_t dfcclStreamWait(int collId, cudaStream_t stream, ofcclRankCtx_t ctx) {
  if (!ctx || !ctx->finalized) return ncclInvalidUsage;
  uint64_t want;
  {
    std::lock_guard<std::mutex> l(ctx->mu);
    auto it = ctx->colls.find(collId);
    if (it == ctx->colls.end()) return ncclInvalidArgument;
    want = it->second.submitted;
  }
  if (ctx->backend == dfcclBackendCuda && ctx->fnWait64) {
    // The stream is about to park on a word only the daemon sets.  Outside a capture, make sure an instance is
    // queued BEFORE the wait in host order and that it stays until the work is done: the release of the stream
    // then never depends on another host thread getting a launch through while this one may be blocked in the
    // driver (full launch queue, module load).  Captured steps keep the poller-driven wake-up.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess) { (void)cudaGetLastError(); cap = cudaStreamCaptureStatusNone; }
    // (only where this context has the daemon launch to itself: ranks that share one launch - several ranks
    // of one process on one device - must keep leaving when stalled, or one rank's held blocks would keep the
    // shared kernel alive in front of the relaunch another rank is waiting for)
    if (ctx->holdOnWait && cap == cudaStreamCaptureStatusNone && ctx->remaining.load() > 0 && ctx->launcher && ctx->launcher->expected == 1) {
      ctl_store(&ctx->ctl->hold, 1);
      std::atomic_thread_fence(std::memory_order_seq_cst);
      if (!ctl_load(&ctx->ctl->alive)) DFCHECK(launchFromCaller(ctx));
    }
    typedef CUresult (*Fn)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);
    // the flag holds (status << 56 | epoch): any finished submission >= want satisfies >=
    CUresult r = ((Fn)ctx->fnWait64)((CUstream)stream, (CUdeviceptr)(uintptr_t)(ctx->rdHost.doneEpoch + collId), want, CU_STREAM_WAIT_VALUE_GEQ);
    if (r != CUDA_SUCCESS) { DF_WARN("cuStreamWaitValue64 failed (%d)", (int)r); return ncclUnhandledCudaError; }
    return ncclSuccess;
  }
  return dfcclWait(collId, -1, ctx);     // no stream memory operations: the host waits instead
}

DF_API ncclResult_t dfcclAbort(ofcclRankCtx_t ctx) {
  if (!ctx) return ncclInvalidArgument;
  if (ctx->ctl) ctl_store(&ctx->ctl->abortFlag, 1);
  if (ctx->devAbort && ctx->sqStream) {
    // the daemon polls a word in device memory; the write goes through the stream that fills the ring (a stream
    // memory operation needs no SM, so it lands whatever the kernels are doing)
    std::lock_guard<std::mutex> l(ctx->mu);
    typedef CUresult (*Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (!paramI64("NO_STREAM_MEMOPS", 0) && cudaGetDriverEntryPoint("cuStreamWriteValue32", &fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess && fn)
      ((Fn)fn)((CUstream)ctx->sqStream, (CUdeviceptr)(uintptr_t)ctx->devAbort, 1u, 0);
    else { uint32_t one = 1; cudaMemcpyAsync(ctx->devAbort, &one, sizeof(one), cudaMemcpyHostToDevice, ctx->sqStream); cudaStreamSynchronize(ctx->sqStream); }
    (void)cudaGetLastError();
  }
  ctx->doneCv.notify_all();
  return ncclSuccess;
}
DF_API ncclResult_t dfcclGetAsyncError(ofcclRankCtx_t ctx, ncclResult_t* e) {
  if (!ctx || !e) return ncclInvalidArgument;
  // a bounded wait that ran out inside a registered fused operator left its verdict in pinned memory
  if (ctx->asyncError == ncclSuccess && ctx->backend == dfcclBackendCuda && ctx->fusedLaunches.load() && gemmGaveUp()) ctx->asyncError = dfcclTimeout;
  *e = ctx->asyncError;
  return ncclSuccess;
}

// The counters that live in host memory only: safe to read while the device is busy or stuck.
DF_API ncclResult_t dfcclGetHostStats(ofcclRankCtx_t ctx, dfcclStats* s) {
  if (!ctx || !s) return ncclInvalidArgument;
  memset(s, 0, sizeof(*s));
  s->sqesSubmitted = ctx->sqes; s->cqesDelivered = ctx->cqes; s->callbacksRun = ctx->cbs; s->sqFullRetries = ctx->sqFull;
  if (!ctx->finalized) return ncclSuccess;
  s->daemonLaunches = ctx->ctl->launches; s->daemonVoluntaryQuits = ctx->ctl->voluntaryQuits;
  s->deviceEvents = ctl_load(&ctx->ctl->alive);               // 1 while an instance of the daemon is (believed to be) running
  return ncclSuccess;
}

DF_API ncclResult_t dfcclGetStats(ofcclRankCtx_t ctx, dfcclStats* s) {
  if (!ctx || !s) return ncclInvalidArgument;
  memset(s, 0, sizeof(*s));
  s->sqesSubmitted = ctx->sqes; s->cqesDelivered = ctx->cqes; s->callbacksRun = ctx->cbs; s->sqFullRetries = ctx->sqFull;
  s->fusedLaunches = ctx->fusedLaunches;
  if (!ctx->finalized) return ncclSuccess;
  s->daemonLaunches = ctx->ctl->launches; s->daemonVoluntaryQuits = ctx->ctl->voluntaryQuits;
  std::vector<DevStats> d(ctx->nBlocks);
  if (ctx->backend == dfcclBackendCuda) { int prev; cudaGetDevice(&prev); cudaSetDevice(ctx->device); cudaError_t e = cudaMemcpy(d.data(), ctx->rdHost.stats, sizeof(DevStats) * ctx->nBlocks, cudaMemcpyDeviceToHost); cudaSetDevice(prev); if (e != cudaSuccess) { (void)cudaGetLastError(); return ncclUnhandledCudaError; } }
  else memcpy(d.data(), ctx->rdHost.stats, sizeof(DevStats) * ctx->nBlocks);
  for (auto& b : d) {
    s->ctxSwitches += b.ctxSwitches; s->ctxSaves += b.ctxSaves; s->ctxLoads += b.ctxLoads;
    s->waitPolls += b.waitPolls; s->waitTimeouts += b.waitTimeouts;
    s->bytesReduced += b.bytesReduced; s->bytesCopied += b.bytesCopied; s->totalSwitchNs += b.totalSwitchNs;
    s->maxSwitchNs = std::max<uint64_t>(s->maxSwitchNs, b.maxSwitchNs);
    s->dataYields += b.yields; s->schedulerPasses += b.passes;
    s->nsTriggers += b.nsTriggers; s->nsWalk += b.nsWalk; s->nsQueues += b.nsQueues;
  }
  if (ctx->rdHost.trace) {
    uint64_t head = 0;
    devDownload(ctx->backend, &head, (char*)ctx->rdDev + offsetof(RankDev, traceHead), sizeof(head));
    s->deviceEvents = head;
  }
  return ncclSuccess;
}

DF_API ncclResult_t dfcclTraceDump(ofcclRankCtx_t ctx, const char* path) {
  if (!ctx || !path || !ctx->finalized) return ncclInvalidArgument;
  if (!ctx->rdHost.trace) { DF_WARN("tracing is off (set DFCCL_TRACE=1 before finalizing)"); return ncclInvalidUsage; }
  uint64_t head = 0;
  DFCHECK(devDownload(ctx->backend, &head, (char*)ctx->rdDev + offsetof(RankDev, traceHead), sizeof(head)));
  const uint32_t cap = ctx->rdHost.traceCap;
  std::vector<TraceEvent> ev(cap);
  DFCHECK(devDownload(ctx->backend, ev.data(), ctx->rdHost.trace, sizeof(TraceEvent) * cap));
  std::ofstream o(path);
  if (!o) return ncclSystemError;
  static const char* names[] = {"?", "sqe", "start", "stall", "arrived", "data_begin", "data_end", "done", "quit", "launch", "peers_done", "yield"};
  o.setf(std::ios::fixed);
  o.precision(3);                 // microseconds with nanosecond resolution; the default would round the absolute stamps
  o << "{\"traceEvents\":[\n";
  uint64_t n = std::min<uint64_t>(head, cap), first = head - n;
  for (uint64_t i = 0; i < n; ++i) {
    const TraceEvent& e = ev[(first + i) & (cap - 1)];
    const char* ph = e.event == TR_DATA_BEGIN ? "B" : e.event == TR_DATA_END ? "E" : "i";
    o << (i ? ",\n" : "") << "{\"name\":\"" << (e.event == TR_DATA_BEGIN || e.event == TR_DATA_END ? "data" : names[e.event < 12 ? e.event : 0])
      << "\",\"ph\":\"" << ph << "\",\"ts\":" << (double)e.ns / 1000.0 << ",\"pid\":" << ctx->rank << ",\"tid\":" << e.block
      << ",\"args\":{\"coll\":" << e.collId << "}}";
  }
  o << "\n]}\n";
  return ncclSuccess;
}

DF_API ncclResult_t dfcclInjectFault(ofcclRankCtx_t ctx, dfcclFault_t fault, int64_t arg) {
  if (!ctx) return ncclInvalidArgument;
  std::lock_guard<std::mutex> l(ctx->mu);
  switch (fault) {
    case dfcclFaultNone: ctx->faultDrop = ctx->faultDelayUs = ctx->faultFreezeMs = 0; break;
    case dfcclFaultDropSqe: ctx->faultDrop = arg; break;
    case dfcclFaultDelaySqeUs: ctx->faultDelayUs = arg; break;
    case dfcclFaultFreezePoller: ctx->faultFreezeMs = arg; break;
    default: return ncclInvalidArgument;
  }
  return ncclSuccess;
}

// Heap pieces go back at destroy time (the communicators they came from may be destroyed right
// after); nobody writes them any more: this rank completed every submission, which needed every
// peer's last flag.
static void releaseHeapParts(ofcclRankCtx* ctx) {
  // arena slots were taken in ascending id order; giving them back in descending order unwinds the bump allocator
  for (auto it = ctx->colls.rbegin(); it != ctx->colls.rend(); ++it) {
    CollEntry& e = it->second;
    if (e.cs.algo == dfcclAlgoNvls && e.comm && e.comm->nvls && !(e.info.flags & DFCCL_COLL_ARENA_BUFFERS)) {
      if (e.cs.kind != dfcclCollReduceScatter) e.comm->nvls->release(e.cs.nvlsOut);
      if (e.cs.kind != dfcclCollAllGather) e.comm->nvls->release(e.cs.nvlsIn);
    }
  }
  for (auto& kv : ctx->colls) {
    CollEntry& e = kv.second;
    e.ring.reset();
    if (e.flagsBytes) e.comm->heap->free(e.flagsOff);
    if (e.fusedBytes) e.comm->heap->free(e.fusedOff);
    if (e.pushBytes) e.comm->heap->free(e.pushOff);
    for (int k = 0; k < 2; ++k) if (e.stagingBytes[k]) e.comm->heap->free(e.stagingOff[k]);
    e.comm = nullptr;
  }
}

static void releaseCtx(ofcclRankCtx* ctx) {
  const dfcclBackend_t be = ctx->backend;
  if (ctx->wakeStream) { cudaStreamSynchronize(ctx->wakeStream); cudaStreamDestroy(ctx->wakeStream); }
  for (auto e : ctx->wakeEvents) cudaEventDestroy(e);
  RankDev& rd = ctx->rdHost;
  devFree(be, rd.devSq); devFree(be, rd.colls); devFree(be, rd.dyn); devFree(be, rd.doneCount); devFree(be, rd.failCount);
  devFree(be, (void*)rd.doneEpoch); devFree(be, (void*)rd.trigger); devFree(be, rd.saved); devFree(be, rd.stats); devFree(be, rd.trace);
  devFree(be, ctx->rdDev);
  pinnedFree(be, (void*)ctx->hostFrontier);
  if (ctx->sqStream) { cudaStreamSynchronize(ctx->sqStream); cudaStreamDestroy(ctx->sqStream); }
  if (ctx->devAbort) devFree(be, ctx->devAbort);
  pinnedFree(be, (void*)ctx->hostCq); pinnedFree(be, ctx->ctl); pinnedFree(be, (void*)ctx->hostTrig);
  delete ctx;
}

DF_API ncclResult_t ofcclDestroy(ofcclRankCtx_t ctx) {
  if (!ctx) return ncclSuccess;
  if (!ctx->finalized) { delete ctx; return ncclSuccess; }
  const dfcclBackend_t be = ctx->backend;
  int prev = 0;
  if (be == dfcclBackendCuda) { cudaGetDevice(&prev); cudaSetDevice(ctx->device); }
  ctx->destroyed = true;
  // quit entry: a running daemon's blocks of this rank leave for good; a parked daemon is not launched for it again
  {
    std::lock_guard<std::mutex> l(ctx->mu);
    Sqe q;
    memset(&q, 0, sizeof(q));
    q.collId = -1; q.flags = SQE_QUIT;
    (void)pushSqe(ctx, q);
  }
  if (ctx->sqStream) cudaStreamSynchronize(ctx->sqStream);         // the quit entry is in the ring
  if (ctx->wakeStream) cudaStreamSynchronize(ctx->wakeStream);     // no wake-up callback may outlive the context
  ctx->stopPoller = true;
  ctx->pollCv.notify_all();
  ctx->netWorkers.shutdown();          // jobs already posted still run to their completion entry
  if (ctx->poller.joinable()) ctx->poller.join();
  std::shared_ptr<DaemonLauncher> L = ctx->launcher;
  ctx->launcher.reset();
  std::shared_ptr<LoopGroup> loop = ctx->colls.begin()->second.comm->loop;
  // my blocks must have seen the quit entry (or be parked) before the flag words are reused
  for (int i = 0; i < 50000 && ctl_load(&ctx->ctl->alive) && !ctl_load(&ctx->ctl->finalQuit); ++i) std::this_thread::sleep_for(std::chrono::microseconds(100));
  releaseHeapParts(ctx);
  bool last = false;
  {
    std::lock_guard<std::mutex> l(L->mu);
    L->members.erase(std::remove(L->members.begin(), L->members.end(), ctx), L->members.end());
    last = L->members.empty();
    // A shared daemon keeps serving the other ranks and its launch table still names this
    // rank's device state, so that state lives on (its blocks leave at once on the quit entry)
    // until the last rank of the group is destroyed.  From here on this thread no longer
    // touches ctx: the last rank's thread may free it at any time.
    if (!last) L->retired.push_back(ctx);
  }
  if (last) {
    if (loop) { std::lock_guard<std::mutex> l(loop->mu); if (loop->launcher == L) loop->launcher.reset(); }
    std::vector<ofcclRankCtx*> retired;
    { std::lock_guard<std::mutex> l(L->mu); retired.swap(L->retired); }
    L.reset();                      // joins the observer, drains the stream, frees the launch table
    for (auto* z : retired) releaseCtx(z);
    releaseCtx(ctx);
  }
  if (be == dfcclBackendCuda) cudaSetDevice(prev);
  return ncclSuccess;
}

// ------------------------------------------------------------------ registered fused operators

static CollEntry* fusedEntry(ofcclRankCtx* ctx, int collId) {
  if (!ctx || !ctx->finalized || ctx->destroyed || collId < 0 || collId >= (int)ctx->byId.size()) return nullptr;
  CollEntry* e = ctx->byId[collId];
  return e && e->fused.kind ? e : nullptr;
}

DF_API ncclResult_t dfcclFusedGemmOperand(int collId, ofcclRankCtx_t ctx, void** shard, void** gathered) {
  CollEntry* e = fusedEntry(ctx, collId);
  if (!e || e->fused.kind != dfcclFusedAllGatherGemm) return ncclInvalidArgument;
  const FusedLayout L = fusedLayout(e->fused, e->comm->nranks);
  char* g = e->comm->heap->base() + e->fusedOff + L.big;
  if (gathered) *gathered = g;
  if (shard) *shard = g + (size_t)e->comm->rank * e->fused.rowsPerRank * e->fused.k * 2;
  return ncclSuccess;
}

// Host backend: the operator's arithmetic with the library's own collectives around a plain loop nest, rounding where
// the kernel rounds (bf16 operands, fp32 accumulation, partial tiles of the reduce-scatter stored as bf16).
static float bf16ToF(uint16_t b) { uint32_t u = (uint32_t)b << 16; float f; memcpy(&f, &u, 4); return f; }
static uint16_t fToBf16(float f) { uint32_t u; memcpy(&u, &f, 4); u += 0x7fffu + ((u >> 16) & 1u); return (uint16_t)(u >> 16); }
static void hostGemmNt(const uint16_t* a, const uint16_t* b, uint16_t* c, int M, int N, int K) {
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc += bf16ToF(a[(size_t)i * K + k]) * bf16ToF(b[(size_t)j * K + k]);
      c[(size_t)i * N + j] = fToBf16(acc);
    }
}

static ncclResult_t runFused(int collId, const void* x, const void* w, void* out, int wT, cudaStream_t stream, ofcclRankCtx_t ctx);
DF_API ncclResult_t dfcclRunFusedGemm(int collId, const void* x, const void* w, void* out, cudaStream_t stream, ofcclRankCtx_t ctx) {
  return runFused(collId, x, w, out, 0, stream, ctx);
}
// The same with the weight stored transposed, [k, n] row-major: the backward pass runs these operators on W^T and hands
// over W as it is stored (the tensor cores read it as an MN-major operand, no transposed copy).
DF_API ncclResult_t dfcclRunFusedGemmT(int collId, const void* x, const void* wT, void* out, cudaStream_t stream, ofcclRankCtx_t ctx) {
  return runFused(collId, x, wT, out, 1, stream, ctx);
}

static void hostTranspose(const uint16_t* src, uint16_t* dst, int rows, int cols) {        // dst[cols, rows] = src[rows, cols]^T
  for (int i = 0; i < rows; ++i) for (int j = 0; j < cols; ++j) dst[(size_t)j * rows + i] = src[(size_t)i * cols + j];
}

static ncclResult_t runFused(int collId, const void* x, const void* w, void* out, int wT, cudaStream_t stream, ofcclRankCtx_t ctx) {
  CollEntry* e = fusedEntry(ctx, collId);
  if (!e) { DF_WARN("id %d is not a registered fused operator of a finalized context", collId); return ncclInvalidArgument; }
  if (!x || !w || !out) return ncclInvalidArgument;
  if (ctl_load(&ctx->ctl->abortFlag)) return dfcclAborted;
  NvtxRange range(e->fused.kind == dfcclFusedAllGatherGemm ? "dfccl:AllGatherGemm" : "dfccl:GemmReduceScatter");
  ncclComm* comm = e->comm;
  const int n = comm->nranks, me = comm->rank, rows = e->fused.rowsPerRank, K = e->fused.k, N = e->fused.n, M = rows * n;
  const FusedLayout L = fusedLayout(e->fused, n);
  char* mine = comm->heap->base() + e->fusedOff;
  ctx->fusedLaunches++;
  if (ctx->backend != dfcclBackendCuda) {
    std::vector<uint16_t> wn;
    if (wT) { wn.resize((size_t)N * K); hostTranspose((const uint16_t*)w, wn.data(), K, N); w = wn.data(); }
    if (e->fused.kind == dfcclFusedAllGatherGemm) {
      DFCHECK(commCollective(comm, dfcclCollAllGather, x, mine + L.big, (size_t)rows * K, ncclBfloat16, ncclSum, 0, stream));
      hostGemmNt((const uint16_t*)(mine + L.big), (const uint16_t*)w, (uint16_t*)out, M, N, K);
    } else {
      std::vector<uint16_t> partial((size_t)M * N);
      hostGemmNt((const uint16_t*)x, (const uint16_t*)w, partial.data(), M, N, K);
      DFCHECK(commCollective(comm, dfcclCollReduceScatter, partial.data(), out, (size_t)rows * N, ncclBfloat16, ncclSum, 0, stream));
    }
    return ncclSuccess;
  }
  if (gemmGaveUp()) { ctx->asyncError = dfcclTimeout; DF_WARN("an earlier fused operator on this device gave up on a bounded wait"); return dfcclTimeout; }
  int prev = 0;
  cudaGetDevice(&prev);
  if (prev != comm->device) cudaSetDevice(comm->device);
  ncclResult_t res = ncclSuccess;
  FusedArgs f;
  memset(&f, 0, sizeof(f));
  f.nranks = n; f.rank = me; f.rowsPerRank = rows;
  f.arrive = (volatile uint64_t*)(mine + L.arrive); f.done = (volatile uint64_t*)(mine + L.done);
  f.doneCount = (uint32_t*)(mine + L.doneCount); f.epochCounter = (uint64_t*)(mine + L.epochCounter);
  for (int j = 0; j < n; ++j) {
    char* theirs = comm->peerHeap[j] + e->peerFusedOff[j];
    f.peerArrive[j] = (volatile uint64_t*)(theirs + L.arrive) + me;
    f.peerDone[j] = (volatile uint64_t*)(theirs + L.done) + me;
  }
  if (e->fused.kind == dfcclFusedAllGatherGemm) {
    char* gathered = mine + L.big;
    char* shard = gathered + (size_t)me * rows * K * 2;
    if ((const char*)x != shard) {
      cudaError_t ce = cudaMemcpyAsync(shard, x, (size_t)rows * K * 2, cudaMemcpyDeviceToDevice, stream);
      if (ce != cudaSuccess) { DF_WARN("fused operator %d: copy of the input rows failed: %s", collId, cudaGetErrorString(ce)); res = ncclUnhandledCudaError; }
    }
    f.mode = 1;
    f.gathered = (__nv_bfloat16*)gathered; f.blockReady = (uint32_t*)(mine + L.flags);
    for (int j = 0; j < n; ++j) f.peerA[j] = (const __nv_bfloat16*)(comm->peerHeap[j] + e->peerFusedOff[j] + L.big + (size_t)j * rows * K * 2);
    if (res == ncclSuccess) res = gemmLaunch(gathered, w, out, M, N, K, n == 1 ? nullptr : &f, stream, 0, wT);
  } else {
    f.mode = 2;
    const uint64_t tiles = (uint64_t)(rows / GEMM_BM) * (N / GEMM_BN);
    f.mySlots = (const __nv_bfloat16*)(mine + L.big); f.myTileFlags = (const uint32_t*)(mine + L.flags);
    f.reduced = (__nv_bfloat16*)out;
    for (int j = 0; j < n; ++j) {
      char* theirs = comm->peerHeap[j] + e->peerFusedOff[j];
      f.slot[j] = (__nv_bfloat16*)(theirs + L.big + (size_t)me * rows * N * 2);       // my partial tiles at owner j
      f.tileFlag[j] = (uint32_t*)(theirs + L.flags);
    }
    (void)tiles;
    res = gemmLaunch(x, w, out, M, N, K, n == 1 ? nullptr : &f, stream, 0, wT);
  }
  if (prev != comm->device) cudaSetDevice(prev);
  return res;
}

// ------------------------------------------------------------------ per-collective wrappers

static ncclResult_t prep(int kind, size_t count, ncclDataType_t t, ncclRedOp_t op, int root, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) {
  dfcclCollInfo i;
  memset(&i, 0, sizeof(i));
  i.kind = kind; i.count = count; i.inType = i.outType = t; i.op = op; i.root = root; i.scale = 1.f;
  return dfcclPrepare(&i, comm, collId, ctx);
}
DF_API ncclResult_t ofcclPrepareAllReduce(size_t count, ncclDataType_t t, ncclRedOp_t op, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) { return prep(dfcclCollAllReduce, count, t, op, 0, comm, collId, ctx); }
DF_API ncclResult_t ofcclPrepareReduce(size_t count, ncclDataType_t t, ncclRedOp_t op, int root, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) { return prep(dfcclCollReduce, count, t, op, root, comm, collId, ctx); }
DF_API ncclResult_t ofcclPrepareReduceScatter(size_t recvcount, ncclDataType_t t, ncclRedOp_t op, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) { return prep(dfcclCollReduceScatter, recvcount, t, op, 0, comm, collId, ctx); }
DF_API ncclResult_t ofcclPrepareAllGather(size_t sendcount, ncclDataType_t t, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) { return prep(dfcclCollAllGather, sendcount, t, ncclSum, 0, comm, collId, ctx); }
DF_API ncclResult_t ofcclPrepareBroadcast(size_t count, ncclDataType_t t, int root, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) { return prep(dfcclCollBroadcast, count, t, ncclSum, root, comm, collId, ctx); }
DF_API ncclResult_t ofcclPrepareBcast(size_t count, ncclDataType_t t, int root, ncclComm_t comm, int collId, ofcclRankCtx_t ctx) { return prep(dfcclCollBroadcast, count, t, ncclSum, root, comm, collId, ctx); }

DF_API ncclResult_t ofcclRunAllReduce(const void* s, void* r, int collId, CallbackFunc cb, void* a, ofcclRankCtx_t ctx) { return dfcclRun(s, r, collId, cb, a, ctx); }
DF_API ncclResult_t ofcclRunReduce(const void* s, void* r, int collId, CallbackFunc cb, void* a, ofcclRankCtx_t ctx) { return dfcclRun(s, r, collId, cb, a, ctx); }
DF_API ncclResult_t ofcclRunReduceScatter(const void* s, void* r, int collId, CallbackFunc cb, void* a, ofcclRankCtx_t ctx) { return dfcclRun(s, r, collId, cb, a, ctx); }
DF_API ncclResult_t ofcclRunAllGather(const void* s, void* r, int collId, CallbackFunc cb, void* a, ofcclRankCtx_t ctx) { return dfcclRun(s, r, collId, cb, a, ctx); }
DF_API ncclResult_t ofcclRunBroadcast(const void* s, void* r, int collId, CallbackFunc cb, void* a, ofcclRankCtx_t ctx) { return dfcclRun(s, r, collId, cb, a, ctx); }
DF_API ncclResult_t ofcclRunBcast(void* b, int collId, CallbackFunc cb, void* a, ofcclRankCtx_t ctx) { return dfcclRun(b, b, collId, cb, a, ctx); }

#define DF_ALIAS(name, params, args) DF_API ncclResult_t p##name params { return name args; }
DF_ALIAS(ofcclInitRankCtx, (ofcclRankCtx_t* c, int r), (c, r))
DF_ALIAS(ofcclFinalizeRankCtx7StartHostThrds, (ofcclRankCtx_t c), (c))
DF_ALIAS(ofcclPrepareDone, (ofcclRankCtx_t c), (c))
DF_ALIAS(ofcclDestroy, (ofcclRankCtx_t c), (c))
DF_ALIAS(ofcclPrepareAllReduce, (size_t n, ncclDataType_t t, ncclRedOp_t o, ncclComm_t c, int i, ofcclRankCtx_t x), (n, t, o, c, i, x))
DF_ALIAS(ofcclPrepareReduce, (size_t n, ncclDataType_t t, ncclRedOp_t o, int r, ncclComm_t c, int i, ofcclRankCtx_t x), (n, t, o, r, c, i, x))
DF_ALIAS(ofcclPrepareReduceScatter, (size_t n, ncclDataType_t t, ncclRedOp_t o, ncclComm_t c, int i, ofcclRankCtx_t x), (n, t, o, c, i, x))
DF_ALIAS(ofcclPrepareAllGather, (size_t n, ncclDataType_t t, ncclComm_t c, int i, ofcclRankCtx_t x), (n, t, c, i, x))
DF_ALIAS(ofcclPrepareBroadcast, (size_t n, ncclDataType_t t, int r, ncclComm_t c, int i, ofcclRankCtx_t x), (n, t, r, c, i, x))
DF_ALIAS(ofcclPrepareBcast, (size_t n, ncclDataType_t t, int r, ncclComm_t c, int i, ofcclRankCtx_t x), (n, t, r, c, i, x))
DF_ALIAS(ofcclRunAllReduce, (const void* s, void* r, int i, CallbackFunc cb, void* a, ofcclRankCtx_t x), (s, r, i, cb, a, x))
DF_ALIAS(ofcclRunReduce, (const void* s, void* r, int i, CallbackFunc cb, void* a, ofcclRankCtx_t x), (s, r, i, cb, a, x))
DF_ALIAS(ofcclRunReduceScatter, (const void* s, void* r, int i, CallbackFunc cb, void* a, ofcclRankCtx_t x), (s, r, i, cb, a, x))
DF_ALIAS(ofcclRunAllGather, (const void* s, void* r, int i, CallbackFunc cb, void* a, ofcclRankCtx_t x), (s, r, i, cb, a, x))
DF_ALIAS(ofcclRunBroadcast, (const void* s, void* r, int i, CallbackFunc cb, void* a, ofcclRankCtx_t x), (s, r, i, cb, a, x))
DF_ALIAS(ofcclRunBcast, (void* b, int i, CallbackFunc cb, void* a, ofcclRankCtx_t x), (b, i, cb, a, x))
