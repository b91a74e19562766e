#include "bootstrap.h"
#include "../common/log.h"
#include "../common/param.h"
#include "../common/socket.h"
#include <algorithm>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <poll.h>
#include <random>
#include <sys/socket.h>
#include <thread>
#include <tuple>
#include <unistd.h>

namespace dfccl {
namespace {

constexpr uint64_t kMagic = 0xdfcc1b200b007ull;

struct IdBlob {            // what the 128 opaque bytes hold
  uint64_t magic;
  uint64_t nonce;
  SockAddr root;
};
static_assert(sizeof(IdBlob) <= NCCL_UNIQUE_ID_BYTES, "unique id too large");

struct Hello {             // rank -> root
  uint64_t magic, nonce;
  int32_t rank, nranks;
  SockAddr listen;
};

enum ConnKind : int32_t { CONN_RING = 1, CONN_MSG = 2 };
struct ConnHeader { int32_t kind, src, tag; uint64_t bytes; };

// Root service: wait for `nranks` hellos, answer each with the full table.
void rootMain(Socket* lsock, uint64_t nonce) {
  std::unique_ptr<Socket> listenSock(lsock);
  std::vector<Socket> conns;
  std::vector<SockAddr> table;
  int n = -1, seen = 0;
  while (n < 0 || seen < n) {
    Socket c;
    ncclResult_t r = listenSock->accept(&c, 600000);
    if (r != ncclSuccess) { DF_WARN("bootstrap root: gave up waiting for ranks (%d/%d joined)", seen, n); return; }
    Hello h;
    if (c.recv(&h, sizeof(h)) != ncclSuccess) continue;
    if (h.magic != kMagic || h.nonce != nonce) { DF_WARN("bootstrap root: stray connection ignored"); continue; }
    if (n < 0) { n = h.nranks; conns.resize(n); table.resize(n); }
    if (h.nranks != n || h.rank < 0 || h.rank >= n) { DF_WARN("bootstrap root: rank %d/%d does not fit job of %d", h.rank, h.nranks, n); continue; }
    if (conns[h.rank].fd >= 0) { DF_WARN("bootstrap root: rank %d joined twice", h.rank); continue; }
    table[h.rank] = h.listen;
    conns[h.rank] = std::move(c);
    ++seen;
  }
  for (int i = 0; i < n; ++i) conns[i].send(table.data(), sizeof(SockAddr) * n);
  DF_INFO(SUB_BOOT, "bootstrap root: %d ranks joined", n);
}

ncclResult_t startRoot(SockAddr* addr, uint64_t nonce) {
  auto* ls = new Socket();
  ncclResult_t r = ls->listen(addr);
  if (r != ncclSuccess) { delete ls; return r; }
  std::thread(rootMain, ls, nonce).detach();
  return ncclSuccess;
}

class TcpBootstrap final : public Bootstrap {
 public:
  TcpBootstrap(int rank, int nranks) : rank_(rank), n_(nranks) {}
  int rank() const override { return rank_; }
  int nranks() const override { return n_; }
  void setAbortFlag(volatile uint32_t* f) override { abort_ = f; listen_.abortFlag = f; next_.abortFlag = f; prev_.abortFlag = f; }

  ncclResult_t init(const IdBlob& id) {
    SockAddr mine;
    DFCHECK(pickLocalAddr(&mine));
    if (mine.sa.sa_family == AF_INET) mine.sin.sin_port = 0; else mine.sin6.sin6_port = 0;
    DFCHECK(listen_.listen(&mine));
    Socket root;
    DFCHECK(root.connect(id.root, (int)paramI64("BOOTSTRAP_TIMEOUT_MS", 120000)));
    Hello h{kMagic, id.nonce, rank_, n_, mine};
    DFCHECK(root.send(&h, sizeof(h)));
    table_.resize(n_);
    DFCHECK(root.recv(table_.data(), sizeof(SockAddr) * n_));
    if (n_ > 1) {
      DFCHECK(next_.connect(table_[(rank_ + 1) % n_]));
      ConnHeader ch{CONN_RING, rank_, 0, 0};
      DFCHECK(next_.send(&ch, sizeof(ch)));
      while (prev_.fd < 0) DFCHECK(acceptOne(-1, -1));
    }
    next_.abortFlag = prev_.abortFlag = abort_;
    DF_INFO(SUB_BOOT, "bootstrap rank %d/%d up, listening on %s", rank_, n_, addrToString(mine).c_str());
    return ncclSuccess;
  }

  ncclResult_t allGather(void* data, size_t bytes) override {
    std::lock_guard<std::mutex> l(mu_);
    char* d = (char*)data;
    for (int i = 0; i < n_ - 1; ++i) {
      int sIdx = (rank_ - i + n_) % n_, rIdx = (rank_ - i - 1 + n_) % n_;
      DFCHECK(sendRecv(d + sIdx * bytes, d + rIdx * bytes, bytes));
    }
    return ncclSuccess;
  }

  ncclResult_t barrier() override {
    std::vector<char> b(n_, 0);
    return allGather(b.data(), 1);
  }

  ncclResult_t send(int peer, int tag, const void* data, size_t bytes) override {
    Socket s;
    s.abortFlag = abort_;
    DFCHECK(s.connect(table_[peer]));
    ConnHeader ch{CONN_MSG, rank_, tag, bytes};
    DFCHECK(s.send(&ch, sizeof(ch)));
    DFCHECK(s.send(data, bytes));
    // No acknowledgement: an orderly close delivers buffered payload before the FIN, and two ranks
    // that send to each other before receiving must not wait on one another here.
    return ncclSuccess;
  }

  ncclResult_t recv(int peer, int tag, void* data, size_t bytes) override {
    std::lock_guard<std::mutex> l(mu_);
    for (;;) {
      for (auto it = unexpected_.begin(); it != unexpected_.end(); ++it) {
        if (it->src == peer && it->tag == tag) {
          if (it->data.size() != bytes) { DF_WARN("bootstrap recv: size mismatch from %d tag %d (%zu vs %zu)", peer, tag, it->data.size(), bytes); return ncclInternalError; }
          memcpy(data, it->data.data(), bytes);
          unexpected_.erase(it);
          return ncclSuccess;
        }
      }
      DFCHECK(acceptOne(peer, tag));
    }
  }

 private:
  struct Unexpected { int src, tag; std::vector<char> data; };

  // Accept one connection: ring link from prev, or a message (always parked in unexpected_).
  ncclResult_t acceptOne(int, int) {
    Socket c;
    DFCHECK(listen_.accept(&c, (int)paramI64("BOOTSTRAP_TIMEOUT_MS", 120000)));
    ConnHeader ch;
    DFCHECK(c.recv(&ch, sizeof(ch)));
    if (ch.kind == CONN_RING) {
      if (ch.src != (rank_ - 1 + n_) % n_) { DF_WARN("bootstrap: ring link from unexpected rank %d", ch.src); return ncclInternalError; }
      prev_ = std::move(c);
      return ncclSuccess;
    }
    Unexpected u{ch.src, ch.tag, std::vector<char>(ch.bytes)};
    DFCHECK(c.recv(u.data.data(), ch.bytes));
    unexpected_.push_back(std::move(u));
    return ncclSuccess;
  }

  // Full-duplex step of the ring: push to next while pulling from prev.
  ncclResult_t sendRecv(const char* sbuf, char* rbuf, size_t bytes) {
    size_t sent = 0, got = 0;
    while (sent < bytes || got < bytes) {
      pollfd pf[2] = {{next_.fd, (short)(sent < bytes ? POLLOUT : 0), 0}, {prev_.fd, (short)(got < bytes ? POLLIN : 0), 0}};
      int r = ::poll(pf, 2, 100);
      if (abort_ && *abort_) return dfcclAborted;
      if (r < 0) { if (errno == EINTR) continue; return ncclSystemError; }
      if (pf[0].revents & (POLLOUT | POLLERR | POLLHUP)) {
        ssize_t k = ::send(next_.fd, sbuf + sent, bytes - sent, MSG_NOSIGNAL | MSG_DONTWAIT);
        if (k < 0 && errno != EAGAIN && errno != EINTR) { DF_WARN("bootstrap ring send: %s", strerror(errno)); return ncclSystemError; }
        if (k > 0) sent += (size_t)k;
      }
      if (pf[1].revents & (POLLIN | POLLERR | POLLHUP)) {
        ssize_t k = ::recv(prev_.fd, rbuf + got, bytes - got, MSG_DONTWAIT);
        if (k == 0) { DF_WARN("bootstrap ring: previous rank closed the link"); return ncclSystemError; }
        if (k < 0 && errno != EAGAIN && errno != EINTR) { DF_WARN("bootstrap ring recv: %s", strerror(errno)); return ncclSystemError; }
        if (k > 0) got += (size_t)k;
      }
    }
    return ncclSuccess;
  }

  int rank_, n_;
  Socket listen_, next_, prev_;
  std::vector<SockAddr> table_;
  std::deque<Unexpected> unexpected_;
  std::mutex mu_;
  volatile uint32_t* abort_ = nullptr;
};

// ------------------------------------------------------------------ in-process
struct LocalShared {
  int n;
  std::mutex mu;
  std::condition_variable cv;
  std::vector<char> buf;
  int arrived = 0, departed = 0;
  uint64_t gen = 0;
  std::map<std::tuple<int, int, int>, std::deque<std::vector<char>>> mail;  // (src,dst,tag)
};

class LocalBootstrap final : public Bootstrap {
 public:
  LocalBootstrap(std::shared_ptr<LocalShared> s, int rank) : s_(std::move(s)), rank_(rank) {}
  int rank() const override { return rank_; }
  int nranks() const override { return s_->n; }
  void setAbortFlag(volatile uint32_t* f) override { abort_ = f; }

  ncclResult_t allGather(void* data, size_t bytes) override {
    std::unique_lock<std::mutex> l(s_->mu);
    // wait until the previous round has been fully read out
    if (!waitFor(l, [&] { return s_->departed == 0 || s_->arrived < s_->n; })) return dfcclAborted;
    if (s_->arrived == 0) s_->buf.assign(bytes * s_->n, 0);
    if (s_->buf.size() != bytes * s_->n) { DF_WARN("local allGather: ranks disagree on the slice size"); return ncclInternalError; }
    memcpy(s_->buf.data() + rank_ * bytes, (char*)data + rank_ * bytes, bytes);
    uint64_t myGen = s_->gen;
    if (++s_->arrived == s_->n) { s_->departed = 0; ++s_->gen; s_->cv.notify_all(); }
    else if (!waitFor(l, [&] { return s_->gen != myGen; })) return dfcclAborted;
    memcpy(data, s_->buf.data(), bytes * s_->n);
    if (++s_->departed == s_->n) { s_->arrived = 0; s_->departed = 0; s_->cv.notify_all(); }
    return ncclSuccess;
  }
  ncclResult_t barrier() override { std::vector<char> b(s_->n, 0); return allGather(b.data(), 1); }
  ncclResult_t send(int peer, int tag, const void* data, size_t bytes) override {
    std::lock_guard<std::mutex> l(s_->mu);
    s_->mail[{rank_, peer, tag}].emplace_back((const char*)data, (const char*)data + bytes);
    s_->cv.notify_all();
    return ncclSuccess;
  }
  ncclResult_t recv(int peer, int tag, void* data, size_t bytes) override {
    std::unique_lock<std::mutex> l(s_->mu);
    auto key = std::make_tuple(peer, rank_, tag);
    if (!waitFor(l, [&] { auto it = s_->mail.find(key); return it != s_->mail.end() && !it->second.empty(); })) return dfcclAborted;
    auto& q = s_->mail[key];
    if (q.front().size() != bytes) return ncclInternalError;
    memcpy(data, q.front().data(), bytes);
    q.pop_front();
    return ncclSuccess;
  }

 private:
  template <class Pred>
  bool waitFor(std::unique_lock<std::mutex>& l, Pred p) {
    while (!p()) {
      s_->cv.wait_for(l, std::chrono::milliseconds(50));
      if (abort_ && *abort_) return false;
    }
    return true;
  }
  std::shared_ptr<LocalShared> s_;
  int rank_;
  volatile uint32_t* abort_ = nullptr;
};

// ------------------------------------------------------------------ sub-group view
class SubBootstrap final : public Bootstrap {
 public:
  SubBootstrap(std::shared_ptr<Bootstrap> p, std::vector<int> members, int tagBase)
      : p_(std::move(p)), m_(std::move(members)), tag_(tagBase) {
    rank_ = (int)(std::find(m_.begin(), m_.end(), p_->rank()) - m_.begin());
  }
  int rank() const override { return rank_; }
  int nranks() const override { return (int)m_.size(); }
  void setAbortFlag(volatile uint32_t* f) override { p_->setAbortFlag(f); }
  ncclResult_t allGather(void* data, size_t bytes) override {
    char* d = (char*)data;
    int n = nranks();
    uint32_t seq = seq_++;
    int tag = tag_ + (int)(seq & 0xffff);
    for (int i = 1; i < n; ++i) DFCHECK(p_->send(m_[(rank_ + i) % n], tag, d + rank_ * bytes, bytes));
    for (int i = 1; i < n; ++i) { int src = (rank_ - i + n) % n; DFCHECK(p_->recv(m_[src], tag, d + src * bytes, bytes)); }
    return ncclSuccess;
  }
  ncclResult_t barrier() override { std::vector<char> b(nranks(), 0); return allGather(b.data(), 1); }
  ncclResult_t send(int peer, int tag, const void* data, size_t bytes) override { return p_->send(m_[peer], tag_ + 0x10000 + tag, data, bytes); }
  ncclResult_t recv(int peer, int tag, void* data, size_t bytes) override { return p_->recv(m_[peer], tag_ + 0x10000 + tag, data, bytes); }

 private:
  std::shared_ptr<Bootstrap> p_;
  std::vector<int> m_;
  int tag_, rank_;
  uint32_t seq_ = 0;
};

}  // namespace

ncclResult_t bootstrapGetUniqueId(ncclUniqueId* id) {
  IdBlob b{};
  b.magic = kMagic;
  std::random_device rd;
  b.nonce = ((uint64_t)rd() << 32) ^ rd() ^ (uint64_t)getpid();
  std::string commId = paramStr("COMM_ID", "");
  if (!commId.empty()) {
    // every rank derives the same id from the environment; rank 0 starts the root in bootstrapCreateTcp
    DFCHECK(addrFromString(commId.c_str(), &b.root));
    b.nonce = 0;
  } else {
    DFCHECK(pickLocalAddr(&b.root));
    DFCHECK(startRoot(&b.root, b.nonce));
  }
  memset(id, 0, sizeof(*id));
  memcpy(id->internal, &b, sizeof(b));
  return ncclSuccess;
}

ncclResult_t bootstrapCreateTcp(const ncclUniqueId& id, int rank, int nranks, std::unique_ptr<Bootstrap>* out) {
  IdBlob b;
  memcpy(&b, id.internal, sizeof(b));
  if (b.magic != kMagic) { DF_WARN("unique id was not produced by ncclGetUniqueId"); return ncclInvalidArgument; }
  if (b.nonce == 0 && rank == 0) {          // COMM_ID mode: rank 0 hosts the root at the agreed address
    SockAddr a = b.root;
    DFCHECK(startRoot(&a, 0));
  }
  auto t = std::make_unique<TcpBootstrap>(rank, nranks);
  DFCHECK(t->init(b));
  *out = std::move(t);
  return ncclSuccess;
}

std::vector<std::unique_ptr<Bootstrap>> bootstrapCreateLocal(int nranks) {
  auto s = std::make_shared<LocalShared>();
  s->n = nranks;
  std::vector<std::unique_ptr<Bootstrap>> v;
  for (int r = 0; r < nranks; ++r) v.emplace_back(new LocalBootstrap(s, r));
  return v;
}

ncclResult_t bootstrapCreateSub(std::shared_ptr<Bootstrap> parent, const std::vector<int>& members, int tagBase,
                                std::unique_ptr<Bootstrap>* out) {
  if (std::find(members.begin(), members.end(), parent->rank()) == members.end()) return ncclInvalidArgument;
  out->reset(new SubBootstrap(std::move(parent), members, tagBase));
  return ncclSuccess;
}

}  // namespace dfccl
