// Built-in TCP implementation of the network interface, and the plugin loader.
// One worker thread per connection end executes the posted requests in order; a message is an
// 8-byte length followed by the payload.
#include "net.h"
#include "../common/log.h"
#include "../common/param.h"
#include "../common/socket.h"
#include <atomic>
#include <condition_variable>
#include <cstring>
#include <deque>
#include <dlfcn.h>
#include <mutex>
#include <thread>

namespace dfccl {
namespace {

struct Request {
  void* data = nullptr;
  size_t bytes = 0, got = 0;
  std::atomic<int> done{0};
  ncclResult_t result = ncclSuccess;
};

struct Conn {                       // one end of a connection with its worker
  Socket sock;
  bool sender = false;
  std::thread worker;
  std::mutex mu;
  std::condition_variable cv;
  std::deque<Request*> q;
  bool stop = false;
  volatile uint32_t abortWord = 0;

  void run() {
    for (;;) {
      Request* r = nullptr;
      {
        std::unique_lock<std::mutex> l(mu);
        cv.wait(l, [&] { return stop || !q.empty(); });
        if (q.empty()) return;      // stop requested and nothing left to do
        r = q.front();
        q.pop_front();
      }
      uint64_t len = r->bytes;
      ncclResult_t res;
      if (sender) {
        res = sock.send(&len, sizeof(len));
        if (res == ncclSuccess && r->bytes) res = sock.send(r->data, r->bytes);
        r->got = r->bytes;
      } else {
        res = sock.recv(&len, sizeof(len));
        if (res == ncclSuccess && len > r->bytes) { DF_WARN("net: message of %llu bytes for a buffer of %zu", (unsigned long long)len, r->bytes); res = ncclInternalError; }
        if (res == ncclSuccess && len) res = sock.recv(r->data, (size_t)len);
        r->got = (size_t)len;
      }
      r->result = res;
      r->done.store(1, std::memory_order_release);
    }
  }
  void start() { sock.abortFlag = &abortWord; worker = std::thread([this] { run(); }); }
  void shutdown() {
    { std::lock_guard<std::mutex> l(mu); stop = true; }
    abortWord = 1;                  // a worker blocked in the socket leaves at its next poll
    cv.notify_all();
    if (worker.joinable()) worker.join();
    for (Request* r : q) { r->result = ncclInternalError; r->done.store(1); }
    q.clear();
    sock.close();
  }
};

struct Listener { Socket sock; };

int s_init() { return ncclSuccess; }
int s_devices(int* n) { *n = 1; return ncclSuccess; }
int s_props(int dev, dfcclNetProperties_v1_t* p) {
  if (dev != 0 || !p) return ncclInvalidArgument;
  p->name = "tcp"; p->speedMbps = 10000; p->maxComms = 65536;
  return ncclSuccess;
}
int s_listen(int dev, void* handle, void** out) {
  if (dev != 0) return ncclInvalidArgument;
  auto* L = new Listener();
  SockAddr a;
  ncclResult_t r = pickLocalAddr(&a);
  if (r == ncclSuccess) r = L->sock.listen(&a);
  if (r != ncclSuccess) { delete L; return r; }
  static_assert(sizeof(SockAddr) <= DFCCL_NET_HANDLE_BYTES, "handle too small");
  memset(handle, 0, DFCCL_NET_HANDLE_BYTES);
  memcpy(handle, &a, sizeof(a));
  *out = L;
  return ncclSuccess;
}
int s_connect(int dev, const void* handle, void** out) {
  if (dev != 0) return ncclInvalidArgument;
  SockAddr a;
  memcpy(&a, handle, sizeof(a));
  auto* c = new Conn();
  c->sender = true;
  ncclResult_t r = c->sock.connect(a);
  if (r != ncclSuccess) { delete c; return r; }
  c->start();
  *out = c;
  return ncclSuccess;
}
int s_accept(void* listenComm, void** out) {
  auto* L = (Listener*)listenComm;
  auto* c = new Conn();
  ncclResult_t r = L->sock.accept(&c->sock, 60000);
  if (r != ncclSuccess) { delete c; return r; }
  c->start();
  *out = c;
  return ncclSuccess;
}
int post(void* comm, void* data, size_t bytes, void** request) {
  auto* c = (Conn*)comm;
  auto* r = new Request();
  r->data = data; r->bytes = bytes;
  { std::lock_guard<std::mutex> l(c->mu); c->q.push_back(r); }
  c->cv.notify_one();
  *request = r;
  return ncclSuccess;
}
int s_isend(void* comm, const void* data, size_t bytes, void** request) { return post(comm, (void*)data, bytes, request); }
int s_irecv(void* comm, void* data, size_t bytes, void** request) { return post(comm, data, bytes, request); }
int s_test(void* request, int* done, size_t* bytes) {
  auto* r = (Request*)request;
  if (!r->done.load(std::memory_order_acquire)) { *done = 0; return ncclSuccess; }
  *done = 1;
  if (bytes) *bytes = r->got;
  ncclResult_t res = r->result;
  delete r;
  return res;
}
int s_closeConn(void* comm) { auto* c = (Conn*)comm; c->shutdown(); delete c; return ncclSuccess; }
int s_closeListen(void* l) { delete (Listener*)l; return ncclSuccess; }

}  // namespace

const dfcclNet_v1_t netSocket = {"socket", s_init, s_devices, s_props, s_listen, s_connect, s_accept,
                                 s_isend, s_irecv, s_test, s_closeConn, s_closeConn, s_closeListen};

const dfcclNet_v1_t* netGet() {
  static const dfcclNet_v1_t* chosen = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    chosen = &netSocket;
    std::string name = paramStr("NET_PLUGIN", "libdfccl-net.so");
    void* h = dlopen(name.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) { DF_INFO(SUB_NET, "no external network plugin (%s): using the built-in sockets", name.c_str()); return; }
    auto* t = (const dfcclNet_v1_t*)dlsym(h, "dfcclNetPlugin_v1");
    int ndev = 0;
    if (!t) DF_INFO(SUB_NET, "%s exports no dfcclNetPlugin_v1: using the built-in sockets", name.c_str());
    else if (t->init() != 0 || t->devices(&ndev) != 0 || ndev < 1)
      DF_INFO(SUB_NET, "network plugin %s (%s) offers no device: using the built-in sockets", name.c_str(), t->name);
    else { chosen = t; DF_INFO(SUB_NET, "network plugin %s: %d device(s)", t->name, ndev); }
  });
  return chosen;
}

}  // namespace dfccl
