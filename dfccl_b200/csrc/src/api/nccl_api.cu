// Exported nccl* entry points (communicator management and stream-ordered
// collectives).  Argument conventions follow the reference's wrappers
// (src/collectives/*.cc, src/init.cc:93-1123, src/misc/argcheck.cc:10-91,
// src/enqueue.cc:1445-1498 for user reduction ops, src/group.cc:96-105 for
// groups); every call also exists under a p-prefixed profiling alias, as with the
// reference's PROFAPI build (src/include/core.h:17-31).
#include "../comm/comm.h"
#include "../common/log.h"
#include "../common/param.h"
#include "../topo/topo.h"
#include "p2p.h"
#include <algorithm>
#include <atomic>
#include <cstring>
#include <thread>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

using namespace dfccl;

#define DF_API extern "C" __attribute__((visibility("default")))

DF_API ncclResult_t ncclGetVersion(int* version) {
  if (!version) return ncclInvalidArgument;
  *version = NCCL_VERSION_CODE;
  return ncclSuccess;
}

DF_API ncclResult_t ncclGetUniqueId(ncclUniqueId* id) {
  if (!id) return ncclInvalidArgument;
  return bootstrapGetUniqueId(id);
}

static int groupDepth();
static void groupRecordInit(ncclComm_t* out, int nranks, const ncclUniqueId& id, int rank, dfcclBackend_t be, int dev);

DF_API ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId commId, int rank) {
  if (!comm) return ncclInvalidArgument;
  if (nranks < 1 || rank < 0 || rank >= nranks) { DF_WARN("invalid rank %d of %d", rank, nranks); return ncclInvalidArgument; }
  dfcclBackend_t be = defaultBackend();
  int dev = 0;
  if (be == dfcclBackendCuda) CUDACHECK(cudaGetDevice(&dev));
  if (groupDepth() > 0) {               // inside a group: recorded for the device that is current now, created at ncclGroupEnd
    *comm = nullptr;
    groupRecordInit(comm, nranks, commId, rank, be, dev);
    return ncclSuccess;
  }
  std::unique_ptr<Bootstrap> b;
  DFCHECK(bootstrapCreateTcp(commId, rank, nranks, &b));
  return commCreate(std::shared_ptr<Bootstrap>(std::move(b)), be, dev, false, nullptr, comm);
}

static ncclResult_t initGroup(ncclComm_t* comms, int n, const int* devs, bool privateHeaps, dfcclBackend_t be) {
  auto boots = bootstrapCreateLocal(n);
  auto loop = std::make_shared<LoopGroup>();
  loop->nranks = n; loop->backend = be; loop->device = devs ? devs[0] : 0;
  std::vector<ncclResult_t> res(n, ncclSuccess);
  std::vector<std::thread> ts;
  for (int r = 0; r < n; ++r) {
    std::shared_ptr<Bootstrap> b(std::move(boots[r]));
    int dev = devs ? devs[r] : r;
    ts.emplace_back([=, &res] { res[r] = commCreate(b, be, dev, privateHeaps, privateHeaps ? loop : nullptr, &comms[r]); });
  }
  for (auto& t : ts) t.join();
  for (auto r : res) if (r != ncclSuccess) return r;
  return ncclSuccess;
}

DF_API ncclResult_t ncclCommInitAll(ncclComm_t* comms, int ndev, const int* devlist) {
  if (!comms || ndev < 1) return ncclInvalidArgument;
  dfcclBackend_t be = defaultBackend();
  if (be == dfcclBackendCuda) {
    int have = 0;
    CUDACHECK(cudaGetDeviceCount(&have));
    for (int i = 0; i < ndev; ++i) {
      int d = devlist ? devlist[i] : i;
      if (d < 0 || d >= have) { DF_WARN("device %d does not exist", d); return ncclInvalidArgument; }
      for (int j = 0; j < i; ++j) if ((devlist ? devlist[j] : j) == d) { DF_WARN("device %d listed twice; use dfcclCommInitLoopback for several ranks on one device", d); return ncclInvalidArgument; }
    }
  }
  // the host backend has no devices to tell heaps apart: one private heap per rank
  return initGroup(comms, ndev, devlist, be == dfcclBackendHost, be);
}

DF_API ncclResult_t dfcclCommInitLoopback(ncclComm_t* comms, int nranks, int device) {
  if (!comms || nranks < 1 || nranks > DF_MAX_RANKS) return ncclInvalidArgument;
  std::vector<int> devs(nranks, device);
  return initGroup(comms, nranks, devs.data(), true, defaultBackend());
}

DF_API ncclResult_t dfcclCommSplit(ncclComm_t comm, int color, int key, ncclComm_t* newcomm) {
  if (!comm || !newcomm) return ncclInvalidArgument;
  struct CK { int color, key, rank; };
  std::vector<CK> all(comm->nranks);
  all[comm->rank] = {color, key, comm->rank};
  DFCHECK(comm->boot->allGather(all.data(), sizeof(CK)));
  if (color < 0) { *newcomm = nullptr; return ncclSuccess; }
  std::vector<CK> mine;
  for (auto& e : all) if (e.color == color) mine.push_back(e);
  std::stable_sort(mine.begin(), mine.end(), [](const CK& a, const CK& b) { return a.key < b.key; });
  std::vector<int> members;
  for (auto& e : mine) members.push_back(e.rank);
  // every member calls split the same number of times, so the count names this split on all of them
  int tagBase = (int)(((comm->splitCount++ & 0x3f) + 1) << 24) | ((color & 0x3f) << 18);
  std::unique_ptr<Bootstrap> sub;
  DFCHECK(bootstrapCreateSub(comm->boot, members, tagBase, &sub));
  return commCreate(std::shared_ptr<Bootstrap>(std::move(sub)), comm->backend, comm->device, false, comm->loop, newcomm, comm->heap);
}

DF_API ncclResult_t ncclCommDestroy(ncclComm_t comm) { return commDestroy(comm); }

DF_API ncclResult_t ncclCommAbort(ncclComm_t comm) {
  if (!comm) return ncclSuccess;
  // The abort word goes up before anything that waits: kernels of this communicator (and host-backend calls running
  // in other threads) look at it every few hundred polls and leave, so the device synchronisation inside the
  // destroy below returns promptly instead of after the kernels' wait limit.
  comm->ctl->abortFlag = 1;
  comm->aborted = true;
  { std::lock_guard<std::mutex> l(comm->mu); }      // a call of another thread that is still inside the communicator has left
  return commDestroy(comm);
}

DF_API const char* ncclGetErrorString(ncclResult_t r) { return resultString(r); }

DF_API ncclResult_t ncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* asyncError) {
  if (!comm || !asyncError) return ncclInvalidArgument;
  if (comm->asyncError == ncclSuccess && comm->ctl->pad)
    comm->asyncError = comm->ctl->pad == ST_TIMEOUT ? dfcclTimeout : comm->ctl->pad == ST_ABORTED ? dfcclAborted : ncclInternalError;
  *asyncError = comm->asyncError;
  return ncclSuccess;
}
DF_API ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) {
  if (!comm || !count) return ncclInvalidArgument;
  *count = comm->nranks;
  return ncclSuccess;
}
DF_API ncclResult_t ncclCommCuDevice(const ncclComm_t comm, int* device) {
  if (!comm || !device) return ncclInvalidArgument;
  *device = comm->device;
  return ncclSuccess;
}
DF_API ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) {
  if (!comm || !rank) return ncclInvalidArgument;
  *rank = comm->rank;
  return ncclSuccess;
}

DF_API ncclResult_t ncclRedOpCreatePreMulSum(ncclRedOp_t* op, void* scalar, ncclDataType_t datatype,
                                             ncclScalarResidence_t residence, ncclComm_t comm) {
  if (!op || !scalar || !comm) return ncclInvalidArgument;
  unsigned char raw[8] = {0};
  size_t sz = datatype == ncclFloat16 || datatype == ncclBfloat16 ? 2 : datatype == ncclFloat32 ? 4 : datatype == ncclFloat64 ? 8 : 0;
  if (sz == 0) { DF_WARN("PreMulSum supports floating types only"); return ncclInvalidArgument; }
  if (residence == ncclScalarHostImmediate || comm->backend == dfcclBackendHost) memcpy(raw, scalar, sz);
  else CUDACHECK(cudaMemcpy(raw, scalar, sz, cudaMemcpyDefault));   // read now: the scalar is folded into the registration
  double v = 1.0;
  if (datatype == ncclFloat32) { float f; memcpy(&f, raw, 4); v = f; }
  else if (datatype == ncclFloat64) memcpy(&v, raw, 8);
  else if (datatype == ncclFloat16) { __half h; memcpy(&h, raw, 2); v = __half2float(h); }
  else { __nv_bfloat16 h; memcpy(&h, raw, 2); v = __bfloat162float(h); }
  std::lock_guard<std::mutex> l(comm->mu);
  size_t i = 0;
  for (; i < comm->userOps.size(); ++i) if (!comm->userOps[i].live) break;
  if (i == comm->userOps.size()) comm->userOps.emplace_back();
  comm->userOps[i].live = true;
  comm->userOps[i].scalar = v;
  *op = (ncclRedOp_t)((int)ncclNumOps + (int)i);
  return ncclSuccess;
}
DF_API ncclResult_t ncclRedOpDestroy(ncclRedOp_t op, ncclComm_t comm) {
  if (!comm) return ncclInvalidArgument;
  int i = (int)op - (int)ncclNumOps;
  std::lock_guard<std::mutex> l(comm->mu);
  if (i < 0 || i >= (int)comm->userOps.size() || !comm->userOps[i].live) { DF_WARN("operator %d was not created by ncclRedOpCreatePreMulSum", (int)op); return ncclInvalidArgument; }
  comm->userOps[i].live = false;
  return ncclSuccess;
}

// ---- groups (reference: src/group.cc:96-105,150-422).  Inside ncclGroupStart / ncclGroupEnd nothing blocks and nothing
// waits for a peer: communicator initialisations and collectives are recorded, and ncclGroupEnd runs them - the
// initialisations on threads of their own (one thread may create the communicators of all its GPUs, each of which
// waits for the others), then the collectives (launched back to back on the GPU; on the host backend, where a
// collective is a blocking call, each communicator's calls on a thread of their own so that one thread may hold
// several ranks), then the send / recv calls fused into one kernel per communicator and stream.
static thread_local int t_groupDepth = 0;
namespace {
struct GroupInit { ncclComm_t* out; int nranks, rank, device; ncclUniqueId id; dfcclBackend_t be; };
struct GroupColl { ncclComm* comm; int kind; const void* send; void* recv; size_t count; ncclDataType_t type; ncclRedOp_t op; int root; cudaStream_t stream; };
thread_local std::vector<GroupInit> t_groupInits;
thread_local std::vector<GroupColl> t_groupColls;

ncclResult_t initRankNow(ncclComm_t* comm, int nranks, const ncclUniqueId& commId, int rank, dfcclBackend_t be, int dev) {
  if (be == dfcclBackendCuda) CUDACHECK(cudaSetDevice(dev));
  std::unique_ptr<Bootstrap> b;
  DFCHECK(bootstrapCreateTcp(commId, rank, nranks, &b));
  return commCreate(std::shared_ptr<Bootstrap>(std::move(b)), be, dev, false, nullptr, comm);
}

ncclResult_t groupCollective(ncclComm* c, int kind, const void* s, void* r, size_t count, ncclDataType_t t, ncclRedOp_t op, int root, cudaStream_t st) {
  if (t_groupDepth > 0 && c) { t_groupColls.push_back({c, kind, s, r, count, t, op, root, st}); return ncclSuccess; }
  return commCollective(c, kind, s, r, count, t, op, root, st);
}

ncclResult_t groupFlush() {
  ncclResult_t res = ncclSuccess;
  std::vector<GroupInit> inits;
  std::vector<GroupColl> colls;
  inits.swap(t_groupInits);
  colls.swap(t_groupColls);
  if (!inits.empty()) {                                   // every member of a communicator waits for the others: one thread each
    std::vector<ncclResult_t> rs(inits.size(), ncclSuccess);
    std::vector<std::thread> ts;
    for (size_t i = 0; i < inits.size(); ++i)
      ts.emplace_back([&, i] { rs[i] = initRankNow(inits[i].out, inits[i].nranks, inits[i].id, inits[i].rank, inits[i].be, inits[i].device); });
    for (auto& t : ts) t.join();
    for (auto r : rs) if (r != ncclSuccess && res == ncclSuccess) res = r;
  }
  if (!colls.empty() && res == ncclSuccess) {
    bool host = false;
    for (auto& g : colls) if (g.comm->backend != dfcclBackendCuda) host = true;
    if (!host) {
      for (auto& g : colls) {                             // asynchronous launches: program order per communicator is kept
        ncclResult_t r = commCollective(g.comm, g.kind, g.send, g.recv, g.count, g.type, g.op, g.root, g.stream);
        if (r != ncclSuccess && res == ncclSuccess) res = r;
      }
    } else {
      std::vector<ncclComm*> order;                       // communicators in order of first appearance
      for (auto& g : colls) if (std::find(order.begin(), order.end(), g.comm) == order.end()) order.push_back(g.comm);
      std::vector<ncclResult_t> rs(order.size(), ncclSuccess);
      std::vector<std::thread> ts;
      for (size_t i = 0; i < order.size(); ++i)
        ts.emplace_back([&, i] {
          for (auto& g : colls) {
            if (g.comm != order[i]) continue;
            ncclResult_t r = commCollective(g.comm, g.kind, g.send, g.recv, g.count, g.type, g.op, g.root, g.stream);
            if (r != ncclSuccess && rs[i] == ncclSuccess) rs[i] = r;
          }
        });
      for (auto& t : ts) t.join();
      for (auto r : rs) if (r != ncclSuccess && res == ncclSuccess) res = r;
    }
  }
  ncclResult_t p = p2pFlush();
  return res != ncclSuccess ? res : p;
}
}  // namespace

static int groupDepth() { return t_groupDepth; }
static void groupRecordInit(ncclComm_t* out, int nranks, const ncclUniqueId& id, int rank, dfcclBackend_t be, int dev) {
  t_groupInits.push_back({out, nranks, rank, dev, id, be});
}

DF_API ncclResult_t ncclGroupStart(void) { ++t_groupDepth; return ncclSuccess; }
DF_API ncclResult_t ncclGroupEnd(void) {
  if (t_groupDepth == 0) { DF_WARN("ncclGroupEnd without ncclGroupStart"); return ncclInvalidUsage; }
  if (--t_groupDepth > 0) return ncclSuccess;
  return groupFlush();
}

DF_API ncclResult_t ncclAllReduce(const void* s, void* r, size_t count, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return groupCollective(c, dfcclCollAllReduce, s, r, count, t, op, 0, st);
}
DF_API ncclResult_t ncclReduce(const void* s, void* r, size_t count, ncclDataType_t t, ncclRedOp_t op, int root, ncclComm_t c, cudaStream_t st) {
  return groupCollective(c, dfcclCollReduce, s, r, count, t, op, root, st);
}
DF_API ncclResult_t ncclBroadcast(const void* s, void* r, size_t count, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st) {
  return groupCollective(c, dfcclCollBroadcast, s, r, count, t, ncclSum, root, st);
}
DF_API ncclResult_t ncclBcast(void* buff, size_t count, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st) {
  return groupCollective(c, dfcclCollBroadcast, buff, buff, count, t, ncclSum, root, st);
}
DF_API ncclResult_t ncclReduceScatter(const void* s, void* r, size_t recvcount, ncclDataType_t t, ncclRedOp_t op, ncclComm_t c, cudaStream_t st) {
  return groupCollective(c, dfcclCollReduceScatter, s, r, recvcount, t, op, 0, st);
}
DF_API ncclResult_t ncclAllGather(const void* s, void* r, size_t sendcount, ncclDataType_t t, ncclComm_t c, cudaStream_t st) {
  return groupCollective(c, dfcclCollAllGather, s, r, sendcount, t, ncclSum, 0, st);
}
DF_API ncclResult_t ncclSend(const void* s, size_t count, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t st) {
  DFCHECK(p2pEnqueue(c, true, (void*)s, count, t, peer, st));
  return t_groupDepth ? ncclSuccess : p2pFlush();
}
DF_API ncclResult_t ncclRecv(void* r, size_t count, ncclDataType_t t, int peer, ncclComm_t c, cudaStream_t st) {
  DFCHECK(p2pEnqueue(c, false, r, count, t, peer, st));
  return t_groupDepth ? ncclSuccess : p2pFlush();
}

// ---- extensions that belong to the communicator
DF_API ncclResult_t dfcclSetBackend(dfcclBackend_t b) {
  if (b != dfcclBackendCuda && b != dfcclBackendHost) return ncclInvalidArgument;
  setDefaultBackend(b);
  return ncclSuccess;
}
DF_API ncclResult_t dfcclGetBackend(dfcclBackend_t* b) {
  if (!b) return ncclInvalidArgument;
  *b = defaultBackend();
  return ncclSuccess;
}
DF_API ncclResult_t dfcclMemAlloc(void** ptr, size_t bytes, ncclComm_t comm) {
  if (!ptr || !comm) return ncclInvalidArgument;
  uint64_t off;
  DFCHECK(comm->heap->alloc(bytes, &off, true));
  *ptr = comm->heap->base() + off;
  return ncclSuccess;
}
DF_API ncclResult_t dfcclMemFree(void* ptr, ncclComm_t comm) {
  if (!comm) return ncclInvalidArgument;
  if (!ptr) return ncclSuccess;
  if (!comm->heap->contains(ptr)) { DF_WARN("dfcclMemFree: pointer is not from the symmetric heap"); return ncclInvalidArgument; }
  return comm->heap->free(comm->heap->offsetOf(ptr));
}
DF_API ncclResult_t dfcclNvlsInit(ncclComm_t comm, size_t bytes, int* available) {
  if (!comm) return ncclInvalidArgument;
  // members that do not (or may not) map one another's memory get no multicast arena either
  if (!comm->nvls && comm->nranks > 1 && !comm->netMode && !comm->shmMode && (!comm->loop || comm->backend != dfcclBackendCuda)) DFCHECK(nvlsArenaCreate(comm, bytes ? bytes : (size_t)(512u << 20), &comm->nvls));
  if (available) *available = comm->nvls ? 1 : 0;
  return ncclSuccess;
}
DF_API ncclResult_t dfcclNvlsAlloc(void** ptr, size_t bytes, ncclComm_t comm) {
  if (!comm || !ptr) return ncclInvalidArgument;
  if (!comm->nvls) { DF_WARN("this communicator has no NVLS arena"); return ncclInvalidUsage; }
  uint64_t off = 0;
  ncclResult_t r = comm->nvls->alloc(bytes, &off);
  if (r != ncclSuccess) { DF_WARN("NVLS arena exhausted: %zu bytes requested, %zu of %zu in use (raise DFCCL_NVLS_BYTES)", bytes, comm->nvls->bump, comm->nvls->bytes); return r; }
  *ptr = comm->nvls->uc + off;
  return ncclSuccess;
}
DF_API ncclResult_t dfcclNvlsInfo(ncclComm_t comm, void** uc, void** mc, size_t* bytes, size_t* used) {
  if (!comm) return ncclInvalidArgument;
  dfccl::NvlsArena* a = comm->nvls;
  if (uc) *uc = a ? a->uc : nullptr;
  if (mc) *mc = a ? a->mc : nullptr;
  if (bytes) *bytes = a ? a->bytes : 0;
  if (used) *used = a ? a->bump : 0;
  return ncclSuccess;
}
DF_API ncclResult_t dfcclHeapInfo(ncclComm_t comm, void** base, size_t* bytes, size_t* used) {
  if (!comm) return ncclInvalidArgument;
  if (base) *base = comm->heap->base();
  if (bytes) *bytes = comm->heap->bytes();
  if (used) *used = comm->heap->used();
  return ncclSuccess;
}

// ---- profiling aliases
#define DF_ALIAS(ret, name, params, args) DF_API ret p##name params { return name args; }
DF_ALIAS(ncclResult_t, ncclGetVersion, (int* v), (v))
DF_ALIAS(ncclResult_t, ncclGetUniqueId, (ncclUniqueId* i), (i))
DF_ALIAS(ncclResult_t, ncclCommInitRank, (ncclComm_t* c, int n, ncclUniqueId i, int r), (c, n, i, r))
DF_ALIAS(ncclResult_t, ncclCommInitAll, (ncclComm_t* c, int n, const int* d), (c, n, d))
DF_ALIAS(ncclResult_t, ncclCommDestroy, (ncclComm_t c), (c))
DF_ALIAS(ncclResult_t, ncclCommAbort, (ncclComm_t c), (c))
DF_ALIAS(const char*, ncclGetErrorString, (ncclResult_t r), (r))
DF_ALIAS(ncclResult_t, ncclCommGetAsyncError, (ncclComm_t c, ncclResult_t* e), (c, e))
DF_ALIAS(ncclResult_t, ncclCommCount, (const ncclComm_t c, int* n), (c, n))
DF_ALIAS(ncclResult_t, ncclCommCuDevice, (const ncclComm_t c, int* n), (c, n))
DF_ALIAS(ncclResult_t, ncclCommUserRank, (const ncclComm_t c, int* n), (c, n))
DF_ALIAS(ncclResult_t, ncclRedOpCreatePreMulSum, (ncclRedOp_t* o, void* s, ncclDataType_t t, ncclScalarResidence_t r, ncclComm_t c), (o, s, t, r, c))
DF_ALIAS(ncclResult_t, ncclRedOpDestroy, (ncclRedOp_t o, ncclComm_t c), (o, c))
DF_ALIAS(ncclResult_t, ncclGroupStart, (void), ())
DF_ALIAS(ncclResult_t, ncclGroupEnd, (void), ())
DF_ALIAS(ncclResult_t, ncclAllReduce, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t o, ncclComm_t c, cudaStream_t st), (s, r, n, t, o, c, st))
DF_ALIAS(ncclResult_t, ncclReduce, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t o, int root, ncclComm_t c, cudaStream_t st), (s, r, n, t, o, root, c, st))
DF_ALIAS(ncclResult_t, ncclBroadcast, (const void* s, void* r, size_t n, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st), (s, r, n, t, root, c, st))
DF_ALIAS(ncclResult_t, ncclBcast, (void* b, size_t n, ncclDataType_t t, int root, ncclComm_t c, cudaStream_t st), (b, n, t, root, c, st))
DF_ALIAS(ncclResult_t, ncclReduceScatter, (const void* s, void* r, size_t n, ncclDataType_t t, ncclRedOp_t o, ncclComm_t c, cudaStream_t st), (s, r, n, t, o, c, st))
DF_ALIAS(ncclResult_t, ncclAllGather, (const void* s, void* r, size_t n, ncclDataType_t t, ncclComm_t c, cudaStream_t st), (s, r, n, t, c, st))
DF_ALIAS(ncclResult_t, ncclSend, (const void* s, size_t n, ncclDataType_t t, int p, ncclComm_t c, cudaStream_t st), (s, n, t, p, c, st))
DF_ALIAS(ncclResult_t, ncclRecv, (void* r, size_t n, ncclDataType_t t, int p, ncclComm_t c, cudaStream_t st), (r, n, t, p, c, st))
