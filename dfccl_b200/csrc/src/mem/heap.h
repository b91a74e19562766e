// Symmetric heap: one region per (process, device) that every peer of every
// communicator of the process maps, so kernels address a peer's buffer as
// peerBase + offset.  This is what replaces the reference's P2P transport with
// its receiver-side FIFOs (src/transport/p2p.cc:166-334) and its SHM transport
// (src/transport/shm.cc:58-167): user buffers that live in the heap are read and
// written in place by the peers, nothing is staged.
//   cuda backend : cudaMalloc + cudaIpcGetMemHandle / cudaIpcOpenMemHandle across
//                  processes, plain pointers (+ peer access) inside a process
//   host backend : POSIX shared memory, mmap'd by peers (threads or processes)
//   cuda backend, bounce mode : for GPUs of one host that cannot map each other's memory (no peer access, or
//                  P2P_DISABLE): the heap itself lives in POSIX shared memory registered with CUDA, so every
//                  GPU reaches every member's heap through host memory at PCIe speed and the same kernels run
#pragma once
#include <cstdint>
#include <map>
#include <mutex>
#include <string>
#include <vector>
#include "dfccl.h"

namespace dfccl {

struct HeapHandle {              // exchanged through the bootstrap, fixed size
  uint64_t hostHash;
  int32_t pid;
  int32_t device;
  int32_t backend;
  int32_t heapId;                // distinguishes several heaps of one process (loopback ranks)
  int32_t hostShm;               // cuda backend: the heap is a registered shared-memory segment (blob = its name)
  int32_t pad;
  uint64_t bytes;
  uint64_t base;                 // address in the owning process
  char blob[64];                 // cudaIpcMemHandle_t or shm name
};

class Heap {
 public:
  static ncclResult_t create(dfcclBackend_t backend, int device, size_t bytes, Heap** out, bool hostShm = false);
  bool hostShm() const { return hostShm_; }
  ~Heap();
  char* base() const { return base_; }
  size_t bytes() const { return bytes_; }
  size_t used() const { return used_; }
  bool contains(const void* p, size_t n = 1) const {
    return (const char*)p >= base_ && (const char*)p + n <= base_ + bytes_;
  }
  uint64_t offsetOf(const void* p) const { return (uint64_t)((const char*)p - base_); }
  // 512-byte aligned first-fit allocation; memory is zeroed when `zero`
  ncclResult_t alloc(size_t bytes, uint64_t* off, bool zero = true);
  ncclResult_t free(uint64_t off);
  void exportHandle(HeapHandle* h) const;
  // Map a peer's heap (cached per owner); returns its base in this process.
  ncclResult_t importPeer(const HeapHandle& h, char** base);
  dfcclBackend_t backend() const { return backend_; }
  int device() const { return device_; }

 private:
  Heap() = default;
  dfcclBackend_t backend_ = dfcclBackendCuda;
  int device_ = 0, heapId_ = 0;
  bool hostShm_ = false;         // cuda backend only: memory is host shared memory registered with CUDA
  char* base_ = nullptr;
  size_t bytes_ = 0, used_ = 0;
  std::string shmName_;
  std::mutex mu_;
  std::map<uint64_t, uint64_t> free_;     // offset -> length
  std::map<uint64_t, uint64_t> live_;     // offset -> length
  struct Import { char* base; bool ipc; size_t bytes; bool registered; };
  std::map<std::string, Import> imports_;
};

uint64_t hostHash();             // boot id + hostname (HOSTID env overrides, as in the reference)

// Backend-neutral small helpers for runtime tables.
ncclResult_t devAlloc(dfcclBackend_t be, void** p, size_t bytes);      // zeroed device (or host) memory
ncclResult_t devFree(dfcclBackend_t be, void* p);
ncclResult_t pinnedAlloc(dfcclBackend_t be, void** p, size_t bytes);   // zeroed, host + device visible
ncclResult_t pinnedFree(dfcclBackend_t be, void* p);
ncclResult_t devUpload(dfcclBackend_t be, void* dst, const void* src, size_t bytes);
ncclResult_t devDownload(dfcclBackend_t be, void* dst, const void* src, size_t bytes);
ncclResult_t devZero(dfcclBackend_t be, void* dst, size_t bytes);

}  // namespace dfccl
