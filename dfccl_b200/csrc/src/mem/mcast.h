// NVLS arena: a region of every member's device memory bound to one NVLink-switch multicast
// object, mapped twice on every rank: a unicast view of the local part (ordinary loads and
// stores) and a multicast view (multimem.ld_reduce reads the element-wise reduction of all
// members' copies, computed in the switch; multimem.st writes all members' copies at once).
// Offsets are symmetric: byte `off` of the arena means the same logical word on every member,
// so the bump allocator must be driven identically on all of them.
//
// Creation is collective over the communicator and opt-in (DFCCL_NVLS=1 or dfcclNvlsInit).
// The multicast handle travels as a POSIX file descriptor that peers duplicate with
// pidfd_getfd(2).  On the host backend the arena is a block of the shared-memory heap and the
// "multicast" view is emulated by the engine with a loop over the members' blocks, which lets
// the schedule be tested without a GPU.
//
// The reference predates NVLS (NCCL 2.12); this replaces nothing in it.
#pragma once
#include <cstdint>
#include <mutex>
#include <vector>
#include "dfccl.h"

struct ncclComm;

namespace dfccl {

struct NvlsArena {
  size_t bytes = 0;
  size_t streamBytes = 0;          // [0, streamBytes): staging of the stream-ordered collectives (in | out halves)
  char* uc = nullptr;              // local part, unicast mapping
  char* mc = nullptr;              // multicast mapping (null on the host backend)
  char** peersDev = nullptr;       // host backend: every member's block, table readable by the engine
  std::vector<char*> peers;        // the same table on the host
  uint64_t heapOff = 0;            // host backend: where the block lives in my heap
  size_t bump = 0;                 // next free symmetric offset
  std::vector<uint64_t> marks;     // start offsets of the live allocations, in order
  std::mutex mu;
  // driver objects (cuda backend)
  unsigned long long mcHandle = 0, memHandle = 0;
  bool bound = false;
  int device = 0;
  dfcclBackend_t backend = dfcclBackendCuda;

  bool contains(const void* p, size_t n) const { return (const char*)p >= uc && (const char*)p + n <= uc + bytes; }
  // symmetric allocation, 512-byte aligned; ncclInvalidUsage when the arena is full
  ncclResult_t alloc(size_t n, uint64_t* off);
  // gives back the most recent allocation (a no-op for any other offset: the allocator is a stack)
  void release(uint64_t off);
};

// Collective.  ncclSuccess with *out == nullptr when the devices or the driver cannot do it.
ncclResult_t nvlsArenaCreate(ncclComm* comm, size_t bytes, NvlsArena** out);
void nvlsArenaDestroy(ncclComm* comm, NvlsArena* a);

}  // namespace dfccl
