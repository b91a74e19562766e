#include "socket.h"
#include "log.h"
#include "param.h"
#include <arpa/inet.h>
#include <cerrno>
#include <cstring>
#include <ifaddrs.h>
#include <net/if.h>
#include <netdb.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <chrono>
#include <thread>
#include <unistd.h>

namespace dfccl {

std::string addrToString(const SockAddr& a) {
  char host[NI_MAXHOST] = "?", serv[NI_MAXSERV] = "?";
  socklen_t len = a.sa.sa_family == AF_INET6 ? sizeof(sockaddr_in6) : sizeof(sockaddr_in);
  getnameinfo(&a.sa, len, host, sizeof(host), serv, sizeof(serv), NI_NUMERICHOST | NI_NUMERICSERV);
  return std::string(host) + ":" + serv;
}

ncclResult_t addrFromString(const char* hostPort, SockAddr* out) {
  std::string s(hostPort), host, port;
  if (!s.empty() && s[0] == '[') {
    size_t rb = s.find(']');
    if (rb == std::string::npos || rb + 1 >= s.size() || s[rb + 1] != ':') return ncclInvalidArgument;
    host = s.substr(1, rb - 1); port = s.substr(rb + 2);
  } else {
    size_t c = s.rfind(':');
    if (c == std::string::npos) return ncclInvalidArgument;
    host = s.substr(0, c); port = s.substr(c + 1);
  }
  addrinfo hints{}, *res = nullptr;
  hints.ai_family = AF_UNSPEC; hints.ai_socktype = SOCK_STREAM;
  if (getaddrinfo(host.c_str(), port.c_str(), &hints, &res) != 0 || !res) {
    DF_WARN("cannot resolve '%s'", hostPort);
    return ncclInvalidArgument;
  }
  memset(out, 0, sizeof(*out));
  memcpy(out, res->ai_addr, res->ai_addrlen);
  freeaddrinfo(res);
  return ncclSuccess;
}

ncclResult_t pickLocalAddr(SockAddr* out) {
  memset(out, 0, sizeof(*out));
  std::string want = paramStr("SOCKET_IFNAME", "");
  bool exclude = false, exact = false;
  if (!want.empty() && want[0] == '^') { exclude = true; want.erase(0, 1); }
  if (!want.empty() && want[0] == '=') { exact = true; want.erase(0, 1); }
  ifaddrs* ifs = nullptr;
  if (!want.empty() && getifaddrs(&ifs) == 0) {
    for (ifaddrs* i = ifs; i; i = i->ifa_next) {
      if (!i->ifa_addr || !(i->ifa_flags & IFF_UP)) continue;
      int fam = i->ifa_addr->sa_family;
      if (fam != AF_INET && fam != AF_INET6) continue;
      bool match = exact ? want == i->ifa_name : strncmp(i->ifa_name, want.c_str(), want.size()) == 0;
      if (match == exclude) continue;
      if (exclude && (i->ifa_flags & IFF_LOOPBACK)) continue;
      memcpy(out, i->ifa_addr, fam == AF_INET ? sizeof(sockaddr_in) : sizeof(sockaddr_in6));
      DF_INFO(SUB_BOOT, "control plane on interface %s (%s)", i->ifa_name, addrToString(*out).c_str());
      freeifaddrs(ifs);
      return ncclSuccess;
    }
    freeifaddrs(ifs);
    DF_WARN("no interface matches SOCKET_IFNAME=%s", paramStr("SOCKET_IFNAME", "").c_str());
    return ncclSystemError;
  }
  out->sin.sin_family = AF_INET;
  out->sin.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  return ncclSuccess;
}

void Socket::close() { if (fd >= 0) { ::close(fd); fd = -1; } }

ncclResult_t Socket::listen(SockAddr* addr) {
  int fam = addr->sa.sa_family ? addr->sa.sa_family : AF_INET;
  fd = ::socket(fam, SOCK_STREAM, 0);
  if (fd < 0) { DF_WARN("socket(): %s", strerror(errno)); return ncclSystemError; }
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  socklen_t len = fam == AF_INET6 ? sizeof(sockaddr_in6) : sizeof(sockaddr_in);
  if (::bind(fd, &addr->sa, len) != 0) { DF_WARN("bind(%s): %s", addrToString(*addr).c_str(), strerror(errno)); close(); return ncclSystemError; }
  if (getsockname(fd, &addr->sa, &len) != 0) { close(); return ncclSystemError; }
  if (::listen(fd, 16384) != 0) { DF_WARN("listen(): %s", strerror(errno)); close(); return ncclSystemError; }
  return ncclSuccess;
}

ncclResult_t Socket::accept(Socket* out, int timeoutMs) {
  int waited = 0;
  for (;;) {
    pollfd p{fd, POLLIN, 0};
    int r = ::poll(&p, 1, 100);
    if (abortFlag && *abortFlag) return dfcclAborted;
    if (r < 0 && errno != EINTR) { DF_WARN("poll(): %s", strerror(errno)); return ncclSystemError; }
    if (r > 0) break;
    waited += 100;
    if (timeoutMs >= 0 && waited >= timeoutMs) return dfcclTimeout;
  }
  int c = ::accept(fd, nullptr, nullptr);
  if (c < 0) { DF_WARN("accept(): %s", strerror(errno)); return ncclSystemError; }
  int one = 1;
  setsockopt(c, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  out->close();
  out->fd = c;
  out->abortFlag = abortFlag;
  return ncclSuccess;
}

ncclResult_t Socket::connect(const SockAddr& addr, int timeoutMs) {
  auto t0 = std::chrono::steady_clock::now();
  for (;;) {
    fd = ::socket(addr.sa.sa_family, SOCK_STREAM, 0);
    if (fd < 0) { DF_WARN("socket(): %s", strerror(errno)); return ncclSystemError; }
    socklen_t len = addr.sa.sa_family == AF_INET6 ? sizeof(sockaddr_in6) : sizeof(sockaddr_in);
    if (::connect(fd, &addr.sa, len) == 0) break;
    int e = errno;
    close();
    if (abortFlag && *abortFlag) return dfcclAborted;
    auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
    if ((e != ECONNREFUSED && e != ETIMEDOUT && e != EINTR) || ms > timeoutMs) {
      DF_WARN("connect(%s): %s", addrToString(addr).c_str(), strerror(e));
      return ncclSystemError;
    }
    std::this_thread::sleep_for(std::chrono::milliseconds(2));
  }
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  return ncclSuccess;
}

static ncclResult_t xfer(Socket* s, bool isSend, char* p, size_t n) {
  size_t done = 0;
  while (done < n) {
    pollfd pf{s->fd, (short)(isSend ? POLLOUT : POLLIN), 0};
    int r = ::poll(&pf, 1, 100);
    if (s->abortFlag && *s->abortFlag) return dfcclAborted;
    if (r < 0) { if (errno == EINTR) continue; return ncclSystemError; }
    if (r == 0) continue;
    ssize_t k = isSend ? ::send(s->fd, p + done, n - done, MSG_NOSIGNAL) : ::recv(s->fd, p + done, n - done, 0);
    if (k == 0 && !isSend) { DF_WARN("peer closed the control connection"); return ncclSystemError; }
    if (k < 0) { if (errno == EINTR || errno == EAGAIN) continue; DF_WARN("socket %s: %s", isSend ? "send" : "recv", strerror(errno)); return ncclSystemError; }
    done += (size_t)k;
  }
  return ncclSuccess;
}
ncclResult_t Socket::send(const void* p, size_t n) { return xfer(this, true, (char*)p, n); }
ncclResult_t Socket::recv(void* p, size_t n) { return xfer(this, false, (char*)p, n); }

}  // namespace dfccl
