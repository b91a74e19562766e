// Blocking TCP helpers for the out-of-band control plane.
//
// Role of the reference's src/misc/socket.cc + src/include/socket.h: interface
// selection (SOCKET_IFNAME with ^ and = prefixes), listen / connect with retry,
// exact-length send / recv that poll an abort flag.  Re-done on poll(2) with a
// deadline instead of busy retry loops.
#pragma once
#include <cstddef>
#include <cstdint>
#include <netinet/in.h>
#include <string>
#include "dfccl.h"

namespace dfccl {

union SockAddr {
  sockaddr sa;
  sockaddr_in sin;
  sockaddr_in6 sin6;
};

std::string addrToString(const SockAddr& a);
ncclResult_t addrFromString(const char* hostPort, SockAddr* out);   // "ip:port" or "[v6]:port" or "host:port"
// Pick the local address the control plane binds to: SOCKET_IFNAME if set
// (prefix "^" excludes, "=" exact match), else the loopback interface.
ncclResult_t pickLocalAddr(SockAddr* out);

struct Socket {
  int fd = -1;
  volatile uint32_t* abortFlag = nullptr;   // polled inside every blocking call
  ~Socket() { close(); }
  Socket() = default;
  Socket(const Socket&) = delete;
  Socket& operator=(const Socket&) = delete;
  Socket(Socket&& o) noexcept : fd(o.fd), abortFlag(o.abortFlag) { o.fd = -1; }
  Socket& operator=(Socket&& o) noexcept { close(); fd = o.fd; abortFlag = o.abortFlag; o.fd = -1; return *this; }
  void close();
  ncclResult_t listen(SockAddr* addr);                      // binds addr (port 0 = any), fills the real port
  ncclResult_t accept(Socket* out, int timeoutMs = -1);
  ncclResult_t connect(const SockAddr& addr, int timeoutMs = 30000);
  ncclResult_t send(const void* p, size_t n);
  ncclResult_t recv(void* p, size_t n);
};

}  // namespace dfccl
