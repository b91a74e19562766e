// Rings of network connections and the host-staged collective algorithms that run over them.
// (A .cu file only because it uses the library's reduce / copy data path, which is one source
// for device and host; everything here runs on the CPU.)
#include "net.h"
#include "../common/log.h"
#include "../device/datapath.h"
#include <algorithm>
#include <cstring>
#include <sched.h>
#include <vector>

namespace dfccl {

ncclResult_t NetRing::create(Bootstrap* boot, std::unique_ptr<NetRing>* out) {
  std::unique_ptr<NetRing> r(new NetRing());
  r->net_ = netGet();
  r->rank_ = boot->rank();
  r->n_ = boot->nranks();
  if (r->n_ > 1) {
    std::vector<char> handles((size_t)r->n_ * DFCCL_NET_HANDLE_BYTES, 0);
    DFCHECK((ncclResult_t)r->net_->listen(0, handles.data() + (size_t)r->rank_ * DFCCL_NET_HANDLE_BYTES, &r->listen_));
    DFCHECK(boot->allGather(handles.data(), DFCCL_NET_HANDLE_BYTES));
    const int next = (r->rank_ + 1) % r->n_;
    DFCHECK((ncclResult_t)r->net_->connect(0, handles.data() + (size_t)next * DFCCL_NET_HANDLE_BYTES, &r->send_));
    DFCHECK((ncclResult_t)r->net_->accept(r->listen_, &r->recv_));
    DFCHECK(boot->barrier());                 // nobody closes its listener before every neighbour is through
  }
  *out = std::move(r);
  return ncclSuccess;
}

NetRing::~NetRing() {
  if (send_) net_->closeSend(send_);
  if (recv_) net_->closeRecv(recv_);
  if (listen_) net_->closeListen(listen_);
}

ncclResult_t NetRing::exchange(const void* send, size_t sbytes, void* recv, size_t rbytes, volatile uint32_t* abortFlag) {
  void *rs = nullptr, *rr = nullptr;
  if (recv) DFCHECK((ncclResult_t)net_->irecv(recv_, recv, rbytes, &rr));
  if (send) DFCHECK((ncclResult_t)net_->isend(send_, send, sbytes, &rs));
  ncclResult_t res = ncclSuccess;
  while (rs || rr) {
    int done = 0;
    size_t got = 0;
    if (rs) { ncclResult_t t = (ncclResult_t)net_->test(rs, &done, &got); if (t != ncclSuccess) { res = t; rs = nullptr; } else if (done) rs = nullptr; }
    if (rr) {
      ncclResult_t t = (ncclResult_t)net_->test(rr, &done, &got);
      if (t != ncclSuccess) { res = t; rr = nullptr; }
      else if (done) { rr = nullptr; if (got != rbytes) { DF_WARN("net: received %zu bytes, expected %zu", got, rbytes); res = ncclInternalError; } }
    }
    if (abortFlag && *abortFlag) return dfcclAborted;      // pending requests are released when the ring is closed
    if (rs || rr) sched_yield();
  }
  return res;
}

namespace {

// dst = cast<outType>(scale * (a (op) b)); b may be null (then it is a scaled / cast copy)
ncclResult_t hostReduce(int inType, int outType, int op, const void* a, const void* b, void* dst, size_t n, double scale, int postDiv) {
  if (n == 0) return ncclSuccess;
  DataArgs args;
  memset(&args, 0, sizeof(args));
  args.src[0] = (const char*)a; args.nsrc = 1;
  if (b) { args.src[1] = (const char*)b; args.nsrc = 2; }
  args.dst[0] = (char*)dst; args.ndst = 1;
  args.n = n; args.scale = scale; args.postDiv = postDiv;
  if (!reduce_dispatch(inType, outType, op, &args)) { DF_WARN("net: no host kernel for type %d -> %d, operator %d", inType, outType, op); return ncclInvalidArgument; }
  return ncclSuccess;
}

struct Chunks {
  size_t count; int n;
  size_t beg(int c) const { size_t per = (count + n - 1) / n; return std::min(count, per * (size_t)c); }
  size_t len(int c) const { return beg(c + 1) - beg(c); }
};
inline int mod(int a, int n) { return ((a % n) + n) % n; }

}  // namespace

ncclResult_t netCollective(NetRing* ring, const NetCollDesc& d, const void* send, void* recv, volatile uint32_t* abortFlag) {
  const int n = ring->nranks(), me = ring->rank();
  const size_t es = (size_t)dtypeSize(d.inType), eo = (size_t)dtypeSize(d.outType);
  const char* in = (const char*)send;
  char* out = (char*)recv;
  switch (d.kind) {
    case dfcclCollAllReduce:
    case dfcclCollReduceScatter: {
      // ring reduce-scatter in the input type: after n-1 steps chunk `me` is complete here
      const bool rs = d.kind == dfcclCollReduceScatter;
      const size_t total = rs ? d.count * n : d.count;
      Chunks ch{total, n};
      if (rs) { ch.count = total; }                       // chunk c = block of rank c (count elements each)
      std::vector<char> acc(in, in + total * es), tmp(((total + n - 1) / n) * es);
      auto cbeg = [&](int c) { return rs ? d.count * (size_t)c : ch.beg(c); };
      auto clen = [&](int c) { return rs ? d.count : ch.len(c); };
      for (int s = 0; s < n - 1; ++s) {
        const int sc = mod(me - s - 1, n), rc = mod(me - s - 2, n);
        DFCHECK(ring->exchange(acc.data() + cbeg(sc) * es, clen(sc) * es, tmp.data(), clen(rc) * es, abortFlag));
        DFCHECK(hostReduce(d.inType, d.inType, d.op, acc.data() + cbeg(rc) * es, tmp.data(), acc.data() + cbeg(rc) * es, clen(rc), 1.0, 0));
      }
      if (rs) return hostReduce(d.inType, d.outType, d.op, acc.data() + cbeg(me) * es, nullptr, out, d.count, d.scale, d.postDiv);
      // scale / cast my chunk into the output, then circulate the finished chunks
      DFCHECK(hostReduce(d.inType, d.outType, d.op, acc.data() + cbeg(me) * es, nullptr, out + cbeg(me) * eo, clen(me), d.scale, d.postDiv));
      for (int s = 0; s < n - 1; ++s) {
        const int sc = mod(me - s, n), rc = mod(me - s - 1, n);
        DFCHECK(ring->exchange(out + cbeg(sc) * eo, clen(sc) * eo, out + cbeg(rc) * eo, clen(rc) * eo, abortFlag));
      }
      return ncclSuccess;
    }
    case dfcclCollAllGather: {
      const size_t bytes = d.count * es;
      if (out + (size_t)me * bytes != in) memcpy(out + (size_t)me * bytes, in, bytes);
      for (int s = 0; s < n - 1; ++s) {
        const int sc = mod(me - s, n), rc = mod(me - s - 1, n);
        DFCHECK(ring->exchange(out + (size_t)sc * bytes, bytes, out + (size_t)rc * bytes, bytes, abortFlag));
      }
      return ncclSuccess;
    }
    case dfcclCollBroadcast: {
      const size_t bytes = d.count * es;
      const int pos = mod(me - d.root, n);                // distance from the root along the ring
      if (pos == 0) { if (out != in) memcpy(out, in, bytes); }
      else DFCHECK(ring->exchange(nullptr, 0, out, bytes, abortFlag));
      if (pos < n - 1) DFCHECK(ring->exchange(out, bytes, nullptr, 0, abortFlag));
      return ncclSuccess;
    }
    case dfcclCollReduce: {
      // a chain that starts after the root and ends at it
      const int pos = mod(me - d.root - 1, n);
      if (n == 1) return hostReduce(d.inType, d.outType, d.op, in, nullptr, out, d.count, d.scale, d.postDiv);
      std::vector<char> acc(d.count * es), tmp;
      if (pos == 0) return ring->exchange(in, d.count * es, nullptr, 0, abortFlag);
      tmp.resize(d.count * es);
      DFCHECK(ring->exchange(nullptr, 0, tmp.data(), d.count * es, abortFlag));
      if (pos == n - 1) return hostReduce(d.inType, d.outType, d.op, tmp.data(), in, out, d.count, d.scale, d.postDiv);
      DFCHECK(hostReduce(d.inType, d.inType, d.op, tmp.data(), in, acc.data(), d.count, 1.0, 0));
      return ring->exchange(acc.data(), d.count * es, nullptr, 0, abortFlag);
    }
    default: break;
  }
  return ncclInvalidArgument;
}

}  // namespace dfccl
