// Out-of-band rendezvous and small-message control plane of a communicator.
//
// Capabilities of the reference's bootstrap (src/bootstrap.cc:92-434,
// src/include/bootstrap.h:13-23): a 128-byte unique id that names the root's
// listening address (or comes from COMM_ID), a root thread that hands every rank
// the addresses it needs, allGather, barrier, tagged send / recv with a queue of
// unexpected messages, intra-node allGather.  Differences: the root returns the
// whole address table rather than only the ring successor, so send / recv connect
// directly; an in-process implementation (LocalBootstrap) serves communicators
// whose ranks are threads of one process (ncclCommInitAll, loopback groups).
#pragma once
#include <cstdint>
#include <memory>
#include <vector>
#include "dfccl.h"

namespace dfccl {

class Bootstrap {
 public:
  virtual ~Bootstrap() = default;
  virtual int rank() const = 0;
  virtual int nranks() const = 0;
  // data holds nranks slices of `bytes`; slice [rank] is the input, all are filled on return.
  virtual ncclResult_t allGather(void* data, size_t bytes) = 0;
  virtual ncclResult_t barrier() = 0;
  virtual ncclResult_t send(int peer, int tag, const void* data, size_t bytes) = 0;
  virtual ncclResult_t recv(int peer, int tag, void* data, size_t bytes) = 0;
  virtual void setAbortFlag(volatile uint32_t* flag) = 0;
};

// Fill `id` with a fresh unique id and start the root service for it in this process.
ncclResult_t bootstrapGetUniqueId(ncclUniqueId* id);
// TCP bootstrap: blocks until all nranks ranks have joined.
ncclResult_t bootstrapCreateTcp(const ncclUniqueId& id, int rank, int nranks, std::unique_ptr<Bootstrap>* out);
// In-process bootstrap for `nranks` threads; returns one object per rank.
std::vector<std::unique_ptr<Bootstrap>> bootstrapCreateLocal(int nranks);
// Sub-group view of a parent bootstrap (used by dfcclCommSplit): `members` lists
// parent ranks in new-rank order and must contain the caller.
ncclResult_t bootstrapCreateSub(std::shared_ptr<Bootstrap> parent, const std::vector<int>& members,
                                int tagBase, std::unique_ptr<Bootstrap>* out);

}  // namespace dfccl
