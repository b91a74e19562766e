// Network path: transport selection (external plugin or built-in TCP), a ring of connections
// per collective, and the host-staged collective algorithms that run over it.
//
// Used by communicators whose members cannot map each other's memory.  What the reference does
// with its NET transport, proxy threads and ring algorithms over receiver-side FIFOs
// (reference: src/transport/net.cc:774-1134, src/transport/net_socket.cc:38-630, src/proxy.cc:609-652)
// is reduced here to: copy the operands to host memory, run the ring algorithm of the collective
// over point-to-point connections with the reduction on the CPU (the library's own data path,
// compiled for the host), copy the result back.  Every registered collective gets its own ring of
// connections, so collectives issued in different orders on different ranks never share a FIFO.
#pragma once
#include <memory>
#include <vector>
#include "dfccl.h"
#include "dfccl_net.h"
#include "../bootstrap/bootstrap.h"

namespace dfccl {

// The transport in use (plugin if one loaded and has devices, else the built-in sockets).
const dfcclNet_v1_t* netGet();
extern const dfcclNet_v1_t netSocket;

// One ring: a sending connection to rank+1 and a receiving one from rank-1.
class NetRing {
 public:
  // Collective over the bootstrap: every member calls it, in the same order relative to other rings.
  static ncclResult_t create(Bootstrap* boot, std::unique_ptr<NetRing>* out);
  ~NetRing();
  int rank() const { return rank_; }
  int nranks() const { return n_; }
  // send `sbytes` to the next rank and receive `rbytes` from the previous one, concurrently
  ncclResult_t exchange(const void* send, size_t sbytes, void* recv, size_t rbytes, volatile uint32_t* abortFlag);

 private:
  NetRing() = default;
  const dfcclNet_v1_t* net_ = nullptr;
  int rank_ = 0, n_ = 1;
  void *listen_ = nullptr, *send_ = nullptr, *recv_ = nullptr;
};

// Host-memory collective over a ring; `send` / `recv` are host buffers laid out as for the device
// collectives (NCCL conventions for counts).  `scale` / `postDiv` as in CollStatic.
struct NetCollDesc {
  int kind, inType, outType, op, root, postDiv;
  double scale;
  size_t count;
};
ncclResult_t netCollective(NetRing* ring, const NetCollDesc& d, const void* send, void* recv, volatile uint32_t* abortFlag);

}  // namespace dfccl
