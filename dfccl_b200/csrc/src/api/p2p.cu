#include "p2p.h"
#include "../common/log.h"
#include "../device/p2p_impl.h"
#include <cstring>
#include <map>
#include <memory>
#include <thread>
#include <vector>

namespace dfccl {

__global__ void __launch_bounds__(512, 1) dfcclP2pKernel(RankDev* rd, const P2pList* lists) {
  __shared__ P2pShared sh;
  p2pBlockMain(rd, &lists[blockIdx.x / DF_P2P_CHANNELS], blockIdx.x % DF_P2P_CHANNELS, &sh);
}

namespace {
struct Pending { ncclComm* comm; bool isSend; void* buf; size_t bytes; int peer; cudaStream_t stream; };
thread_local std::vector<Pending> t_pending;

// Staging pieces of receives into buffers outside the heap go back to the heap once the kernel that used them has
// run: from a host function enqueued behind the kernel (cuda backend), never by making the caller wait.
struct FreeLater { Heap* heap; std::vector<uint64_t> offs; };
void CUDART_CB freeStaging(void* arg) {
  FreeLater* f = (FreeLater*)arg;
  for (auto off : f->offs) f->heap->free(off);      // host bookkeeping only: no CUDA call in here
  delete f;
}

// What one (communicator, stream) of a flush has started on the host backend and not yet waited for.
struct NetRecv { int peer, tag; void* buf; size_t bytes; };
struct HostLaunch {
  ncclComm* comm = nullptr;
  std::shared_ptr<std::vector<P2pList>> lists;
  std::vector<std::thread> threads;
  std::vector<uint64_t> temps;
  // network path: receives still to be done by the flushing thread, and the verdicts of the sending threads
  std::vector<NetRecv> netRecvs;
  cudaStream_t stream = nullptr;
  std::shared_ptr<std::vector<ncclResult_t>> sendResults;
};

// Messages of one (source, destination) pair match in program order: the tag carries the pair's sequence number.
inline int netP2pTag(uint32_t seq) { return 0x8000 | (int)(seq & 0x7FFF); }   // below 0x10000: a sub-group adds its own base above that

// Network path (members that cannot map one another's memory): a send is a message over the out-of-band connection
// of the communicator, staged through host memory; it goes out from a thread of its own so that two ranks that send
// to each other before receiving cannot block one another.  The receives of the whole flush follow once every send
// has been started (netFinish).  The stream is drained first and the call returns with the data in place, like the
// collectives of this path.
ncclResult_t netLaunchFor(ncclComm* c, cudaStream_t stream, const std::vector<Pending>& ops, HostLaunch* host) {
  host->comm = c; host->stream = stream;
  const bool cuda = c->backend == dfcclBackendCuda;
  if (cuda) {
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != c->device) cudaSetDevice(c->device);
    cudaError_t e = cudaStreamSynchronize(stream);
    if (prev != c->device) cudaSetDevice(prev);
    if (e != cudaSuccess) { DF_WARN("send / recv over the network path: %s", cudaGetErrorString(e)); return ncclUnhandledCudaError; }
  }
  std::lock_guard<std::mutex> l(c->mu);
  size_t nSend = 0;
  for (auto& p : ops) if (p.isSend) ++nSend;
  host->sendResults = std::make_shared<std::vector<ncclResult_t>>(nSend, ncclSuccess);
  size_t k = 0;
  for (auto& p : ops) {
    if (!p.isSend) { host->netRecvs.push_back({p.peer, netP2pTag(++c->recvSeq[p.peer]), p.buf, p.bytes}); continue; }
    auto data = std::make_shared<std::vector<char>>(p.bytes);
    if (cuda) { CUDACHECK(cudaMemcpy(data->data(), p.buf, p.bytes, cudaMemcpyDeviceToHost)); }
    else memcpy(data->data(), p.buf, p.bytes);
    const int tag = netP2pTag(++c->sendSeq[p.peer]), peer = p.peer;
    auto boot = c->boot;
    auto results = host->sendResults;
    const size_t slot = k++;
    host->threads.emplace_back([boot, data, tag, peer, results, slot] { (*results)[slot] = boot->send(peer, tag, data->data(), data->size()); });
  }
  return ncclSuccess;
}

ncclResult_t netFinish(HostLaunch* h) {
  ncclResult_t res = ncclSuccess;
  ncclComm* c = h->comm;
  for (auto& r : h->netRecvs) {
    if (res != ncclSuccess) break;
    if (c->backend == dfcclBackendCuda) {
      std::vector<char> tmp(r.bytes);
      res = c->boot->recv(r.peer, r.tag, tmp.data(), r.bytes);
      if (res == ncclSuccess && cudaMemcpy(r.buf, tmp.data(), r.bytes, cudaMemcpyHostToDevice) != cudaSuccess) { (void)cudaGetLastError(); res = ncclUnhandledCudaError; }
    } else {
      res = c->boot->recv(r.peer, r.tag, r.buf, r.bytes);
    }
  }
  for (auto& t : h->threads) t.join();
  h->threads.clear();
  if (h->sendResults) for (auto r : *h->sendResults) if (res == ncclSuccess && r != ncclSuccess) res = r;
  return res;
}

ncclResult_t launchFor(ncclComm* c, cudaStream_t stream, const std::vector<Pending>& ops, HostLaunch* host) {
  if (c->netMode) return netLaunchFor(c, stream, ops, host);
  // lists keyed by (direction, peer), operations in program order
  std::map<std::pair<int, int>, std::vector<const Pending*>> by;
  for (auto& p : ops) by[{p.isSend ? 1 : 0, p.peer}].push_back(&p);
  std::vector<P2pList> lists;
  std::vector<uint64_t> temps;         // staging areas to release after the launch has run
  std::lock_guard<std::mutex> l(c->mu);
  for (auto& kv : by) {
    const int isSend = kv.first.first, peer = kv.first.second;
    size_t done = 0;
    while (done < kv.second.size()) {
      P2pList L;
      memset(&L, 0, sizeof(L));
      L.isSend = isSend; L.peer = peer;
      // my slots: [dir][peer][chan]; dir 0 = "receiver ready" words (read by senders), dir 1 = "data done" words (read by receivers)
      FlagSlot* mineBase = (FlagSlot*)(c->heap->base() + c->p2pFlagsOff);
      FlagSlot* theirBase = (FlagSlot*)(c->peerHeap[peer] + c->peerP2pFlagsOff[peer]);
      const int n = c->nranks;
      L.mine = mineBase + ((isSend ? 0 : 1) * n + peer) * DF_P2P_CHANNELS;
      L.theirs = theirBase + ((isSend ? 1 : 0) * n + c->rank) * DF_P2P_CHANNELS;
      L.peerHeap = c->peerHeap[peer]; L.myHeap = c->heap->base();
      size_t maxBytes = 0;
      while (done < kv.second.size() && L.nOps < DF_P2P_MAX_OPS) {
        const Pending* p = kv.second[done++];
        P2pOp& o = L.ops[L.nOps++];
        o.buf = (uint64_t)(uintptr_t)p->buf; o.bytes = p->bytes;
        o.seq = isSend ? ++c->sendSeq[peer] : ++c->recvSeq[peer];
        if (!isSend) {
          if (c->heap->contains(p->buf, p->bytes)) o.stagingOff = c->heap->offsetOf(p->buf);
          else { DFCHECK(c->heap->alloc(p->bytes, &o.stagingOff, false)); o.staged = 1; temps.push_back(o.stagingOff); }
        }
        maxBytes = std::max(maxBytes, p->bytes);
      }
      L.channels = (int)std::min<size_t>(DF_P2P_CHANNELS, std::max<size_t>(1, maxBytes / (256u << 10)));
      lists.push_back(L);
    }
  }
  if (lists.empty()) return ncclSuccess;
  // both sides must agree on the channel count of a transfer: it is a function of the byte count only
  if (c->backend == dfcclBackendCuda) {
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != c->device) cudaSetDevice(c->device);
    P2pList* dl = nullptr;
    CUDACHECK(cudaMallocAsync((void**)&dl, sizeof(P2pList) * lists.size(), stream));
    CUDACHECK(cudaMemcpyAsync(dl, lists.data(), sizeof(P2pList) * lists.size(), cudaMemcpyHostToDevice, stream));
    dfcclP2pKernel<<<(unsigned)(lists.size() * DF_P2P_CHANNELS), 512, 0, stream>>>(c->saRd, dl);
    CUDACHECK(cudaGetLastError());
    CUDACHECK(cudaFreeAsync(dl, stream));
    if (!temps.empty()) CUDACHECK(cudaLaunchHostFunc(stream, freeStaging, new FreeLater{c->heap, temps}));
    if (prev != c->device) cudaSetDevice(prev);
  } else {
    // the "kernels" of every communicator of the flush are started before any of them is waited for (p2pFlush): one
    // thread may hold both ends of a transfer (ncclCommInitAll, then a group with send / recv on every communicator)
    host->comm = c;
    host->lists = std::make_shared<std::vector<P2pList>>(lists);
    host->temps = temps;
    auto shared = host->lists;
    RankDev* rd = c->saRd;
    for (size_t i = 0; i < shared->size(); ++i)
      for (int ch = 0; ch < DF_P2P_CHANNELS; ++ch)
        host->threads.emplace_back([shared, rd, i, ch] { P2pShared sh; p2pBlockMain(rd, &(*shared)[i], ch, &sh); });
  }
  return ncclSuccess;
}
}  // namespace

ncclResult_t p2pEnqueue(ncclComm* comm, bool isSend, void* buf, size_t count, ncclDataType_t type, int peer, cudaStream_t stream) {
  if (!comm) return ncclInvalidArgument;
  if (peer < 0 || peer >= comm->nranks) { DF_WARN("invalid peer %d", peer); return ncclInvalidArgument; }
  if ((int)type < 0 || (int)type >= ncclNumTypes) return ncclInvalidArgument;
  if (count && !buf) return ncclInvalidArgument;
  if (peer == comm->rank) { DF_WARN("send / recv to self is not supported"); return ncclInvalidUsage; }
  t_pending.push_back({comm, isSend, buf, count * (size_t)dtypeSize(type), peer, stream});
  return ncclSuccess;
}

ncclResult_t p2pFlush() {
  std::vector<Pending> all;
  all.swap(t_pending);
  std::map<std::pair<ncclComm*, cudaStream_t>, std::vector<Pending>> by;
  for (auto& p : all) by[{p.comm, p.stream}].push_back(p);
  // launch everything first: a kernel of one communicator may be the partner of a kernel of another one in this very
  // flush, so nothing here waits between two launches
  std::vector<HostLaunch> started(by.size());
  ncclResult_t res = ncclSuccess;
  size_t k = 0;
  for (auto& kv : by) {
    res = launchFor(kv.first.first, kv.first.second, kv.second, &started[k++]);
    if (res != ncclSuccess) break;
  }
  for (auto& h : started) {
    if (h.comm && h.comm->netMode) { ncclResult_t r = netFinish(&h); if (res == ncclSuccess) res = r; continue; }
    for (auto& t : h.threads) t.join();
    for (auto off : h.temps) h.comm->heap->free(off);
  }
  return res;
}

}  // namespace dfccl
