#include "heap.h"
#include "../common/log.h"
#include "../common/param.h"
#include <atomic>
#include <cstring>
#include <dirent.h>
#include <fcntl.h>
#include <signal.h>
#include <fstream>
#include <sys/mman.h>
#include <unistd.h>

namespace dfccl {

uint64_t hostHash() {
  std::string s = paramStr("HOSTID", "");
  if (s.empty()) {
    char host[256] = {0};
    gethostname(host, sizeof(host) - 1);
    s = host;
    std::ifstream f("/proc/sys/kernel/random/boot_id");
    std::string boot;
    if (f && std::getline(f, boot)) s += boot;
  }
  uint64_t h = 1469598103934665603ull;          // FNV-1a
  for (unsigned char c : s) { h ^= c; h *= 1099511628211ull; }
  return h;
}

static std::atomic<int> g_heapSeq{0};

// ---- shared-memory segments of the host backend outlive a process that is killed (or that never destroys its
// process-wide heap).  Names carry the owner's pid, so (a) every live name of this process is unlinked at exit and
// (b) the first heap of a process removes segments whose owner no longer exists - otherwise a recycled pid would
// find "its" name taken.
static std::mutex g_namesMu;
static std::vector<std::string> g_liveNames;

static void unlinkLiveNames() {
  std::lock_guard<std::mutex> l(g_namesMu);
  for (auto& n : g_liveNames) shm_unlink(n.c_str());
  g_liveNames.clear();
}
static void rememberName(const std::string& n) {
  static std::once_flag once;
  std::call_once(once, [] { atexit(unlinkLiveNames); });
  std::lock_guard<std::mutex> l(g_namesMu);
  g_liveNames.push_back(n);
}
static void forgetName(const std::string& n) {
  std::lock_guard<std::mutex> l(g_namesMu);
  for (size_t i = 0; i < g_liveNames.size(); ++i) if (g_liveNames[i] == n) { g_liveNames[i] = g_liveNames.back(); g_liveNames.pop_back(); break; }
}
static void reapStaleSegments() {
  static std::once_flag once;
  std::call_once(once, [] {
    DIR* d = opendir("/dev/shm");
    if (!d) return;
    int reaped = 0;
    while (dirent* e = readdir(d)) {
      int pid = 0, id = 0;
      if (sscanf(e->d_name, "dfccl-%d-%d", &pid, &id) != 2 || pid <= 0) continue;
      if (kill((pid_t)pid, 0) == 0 || errno != ESRCH) continue;      // owner alive (or not ours to judge)
      std::string name = std::string("/") + e->d_name;
      if (shm_unlink(name.c_str()) == 0) ++reaped;
    }
    closedir(d);
    if (reaped) DF_INFO(SUB_ALLOC, "removed %d shared-memory segments of processes that no longer exist", reaped);
  });
}

ncclResult_t Heap::create(dfcclBackend_t backend, int device, size_t bytes, Heap** out, bool hostShm) {
  Heap* h = new Heap();
  h->backend_ = backend; h->device_ = device; h->heapId_ = g_heapSeq++;
  h->hostShm_ = hostShm && backend == dfcclBackendCuda;
  bytes = (bytes + (2u << 20) - 1) & ~(size_t)((2u << 20) - 1);
  h->bytes_ = bytes;
  if (backend == dfcclBackendCuda && !h->hostShm_) {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaMalloc((void**)&h->base_, bytes);
    if (e != cudaSuccess) {
      DF_WARN("symmetric heap: cudaMalloc(%zu MiB) on device %d failed: %s", bytes >> 20, device, cudaGetErrorString(e));
      (void)cudaGetLastError();
      cudaSetDevice(prev);
      delete h;
      return ncclUnhandledCudaError;
    }
    cudaSetDevice(prev);
  } else {
    char name[64];
    snprintf(name, sizeof(name), "/dfccl-%d-%d", (int)getpid(), h->heapId_);
    reapStaleSegments();
    int fd = shm_open(name, O_CREAT | O_RDWR | O_EXCL, 0600);
    if (fd < 0 && errno == EEXIST) {          // a segment carrying my own pid can only be the leftover of a dead process
      shm_unlink(name);
      fd = shm_open(name, O_CREAT | O_RDWR | O_EXCL, 0600);
    }
    if (fd < 0 || ftruncate(fd, (off_t)bytes) != 0) {
      DF_WARN("symmetric heap: shm_open/ftruncate(%s, %zu) failed: %s", name, bytes, strerror(errno));
      if (fd >= 0) { close(fd); shm_unlink(name); }
      delete h;
      return ncclSystemError;
    }
    void* p = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) { shm_unlink(name); delete h; return ncclSystemError; }
    h->base_ = (char*)p;
    h->shmName_ = name;
    rememberName(h->shmName_);
    if (h->hostShm_) {
      // the GPUs read and write the segment in place: pin it and map it into the CUDA address space (same address)
      cudaError_t e = cudaHostRegister(p, bytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
      if (e != cudaSuccess) {
        DF_WARN("symmetric heap in shared memory: cudaHostRegister(%zu MiB) failed: %s", bytes >> 20, cudaGetErrorString(e));
        (void)cudaGetLastError();
        delete h;
        return ncclUnhandledCudaError;
      }
    }
  }
  h->free_[0] = bytes;
  DF_INFO(SUB_ALLOC, "symmetric heap %d: %zu MiB at %p (%s)", h->heapId_, bytes >> 20, (void*)h->base_,
          backend != dfcclBackendCuda ? "host" : h->hostShm_ ? "cuda, in registered shared memory" : "cuda");
  *out = h;
  return ncclSuccess;
}

Heap::~Heap() {
  for (auto& kv : imports_) {
    if (!kv.second.ipc) continue;
    if (kv.second.registered) { cudaHostUnregister(kv.second.base); (void)cudaGetLastError(); }
    if (backend_ == dfcclBackendCuda && !kv.second.registered) cudaIpcCloseMemHandle(kv.second.base);
    else munmap(kv.second.base, kv.second.bytes);
  }
  if (!base_) return;
  if (backend_ == dfcclBackendCuda && !hostShm_) { cudaFree(base_); (void)cudaGetLastError(); }
  else {
    if (hostShm_) { cudaHostUnregister(base_); (void)cudaGetLastError(); }
    munmap(base_, bytes_); shm_unlink(shmName_.c_str()); forgetName(shmName_);
  }
}

ncclResult_t Heap::alloc(size_t bytes, uint64_t* off, bool zero) {
  if (bytes == 0) bytes = 1;
  bytes = (bytes + 511) & ~(size_t)511;
  std::lock_guard<std::mutex> l(mu_);
  for (auto it = free_.begin(); it != free_.end(); ++it) {
    if (it->second < bytes) continue;
    uint64_t o = it->first, len = it->second;
    free_.erase(it);
    if (len > bytes) free_[o + bytes] = len - bytes;
    live_[o] = bytes;
    used_ += bytes;
    *off = o;
    if (zero) {
      if (backend_ == dfcclBackendCuda && !hostShm_) {
        int prev = 0;
        cudaGetDevice(&prev);
        cudaSetDevice(device_);
        cudaError_t e = cudaMemset(base_ + o, 0, bytes);
        cudaSetDevice(prev);
        if (e != cudaSuccess) { DF_WARN("heap memset: %s", cudaGetErrorString(e)); return ncclUnhandledCudaError; }
      } else {
        memset(base_ + o, 0, bytes);
      }
    }
    return ncclSuccess;
  }
  DF_WARN("symmetric heap exhausted: %zu bytes requested, %zu of %zu in use (raise DFCCL_HEAP_BYTES)", bytes, used_, bytes_);
  return ncclInvalidUsage;
}

ncclResult_t Heap::free(uint64_t off) {
  std::lock_guard<std::mutex> l(mu_);
  auto it = live_.find(off);
  if (it == live_.end()) { DF_WARN("heap free: %llu is not the start of a live allocation", (unsigned long long)off); return ncclInvalidArgument; }
  uint64_t len = it->second;
  live_.erase(it);
  used_ -= len;
  auto ins = free_.emplace(off, len).first;
  auto nxt = std::next(ins);                       // merge with the following hole
  if (nxt != free_.end() && ins->first + ins->second == nxt->first) { ins->second += nxt->second; free_.erase(nxt); }
  if (ins != free_.begin()) {                      // and with the preceding one
    auto prv = std::prev(ins);
    if (prv->first + prv->second == ins->first) { prv->second += ins->second; free_.erase(ins); }
  }
  return ncclSuccess;
}

void Heap::exportHandle(HeapHandle* h) const {
  memset(h, 0, sizeof(*h));
  h->hostHash = hostHash(); h->pid = (int32_t)getpid(); h->device = device_; h->backend = backend_;
  h->heapId = heapId_; h->bytes = bytes_; h->base = (uint64_t)(uintptr_t)base_;
  h->hostShm = hostShm_ ? 1 : 0;
  if (backend_ == dfcclBackendCuda && !hostShm_) {
    cudaIpcMemHandle_t ipc;
    if (cudaIpcGetMemHandle(&ipc, base_) == cudaSuccess) memcpy(h->blob, &ipc, sizeof(ipc));
    else (void)cudaGetLastError();                 // single-process use still works through `base`
  } else {
    strncpy(h->blob, shmName_.c_str(), sizeof(h->blob) - 1);
  }
}

ncclResult_t Heap::importPeer(const HeapHandle& h, char** base) {
  if (h.backend != (int32_t)backend_) { DF_WARN("peer uses another backend"); return ncclInvalidUsage; }
  if ((h.hostShm != 0) != hostShm_) { DF_WARN("peer's heap is of another kind (device memory against shared memory)"); return ncclInvalidUsage; }
  if (h.hostHash != hostHash()) {
    DF_WARN("peer is on another host: the direct-access engine needs every rank of a communicator on one NVLink domain");
    return ncclInvalidUsage;
  }
  char key[96];
  snprintf(key, sizeof(key), "%d/%d", h.pid, h.heapId);
  std::lock_guard<std::mutex> l(mu_);
  auto it = imports_.find(key);
  if (it != imports_.end()) { *base = it->second.base; return ncclSuccess; }
  Import imp{nullptr, false, (size_t)h.bytes, false};
  if (h.pid == (int32_t)getpid()) {
    imp.base = (char*)(uintptr_t)h.base;            // (a registered segment is portable: every device of the process sees it)
    if (backend_ == dfcclBackendCuda && !hostShm_ && h.device != device_) {
      int prev = 0, can = 0;
      cudaGetDevice(&prev);
      CUDACHECK(cudaDeviceCanAccessPeer(&can, device_, h.device));
      if (!can) { DF_WARN("device %d cannot access device %d", device_, h.device); return ncclInvalidUsage; }
      cudaSetDevice(device_);
      cudaError_t e = cudaDeviceEnablePeerAccess(h.device, 0);
      cudaSetDevice(prev);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { DF_WARN("enable peer access: %s", cudaGetErrorString(e)); return ncclUnhandledCudaError; }
      (void)cudaGetLastError();
    }
  } else if (backend_ == dfcclBackendCuda && !hostShm_) {
    cudaIpcMemHandle_t ipc;
    memcpy(&ipc, h.blob, sizeof(ipc));
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(device_);
    void* p = nullptr;
    cudaError_t e = cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess);
    cudaSetDevice(prev);
    if (e != cudaSuccess) { DF_WARN("cudaIpcOpenMemHandle (peer pid %d dev %d): %s", h.pid, h.device, cudaGetErrorString(e)); (void)cudaGetLastError(); return ncclUnhandledCudaError; }
    imp.base = (char*)p; imp.ipc = true;
  } else {
    int fd = shm_open(h.blob, O_RDWR, 0600);
    if (fd < 0) { DF_WARN("shm_open(%s): %s", h.blob, strerror(errno)); return ncclSystemError; }
    void* p = mmap(nullptr, h.bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) { DF_WARN("mmap(%s): %s", h.blob, strerror(errno)); return ncclSystemError; }
    imp.base = (char*)p; imp.ipc = true;
    if (hostShm_) {
      int prev = 0;
      cudaGetDevice(&prev);
      cudaSetDevice(device_);
      cudaError_t e = cudaHostRegister(p, h.bytes, cudaHostRegisterPortable | cudaHostRegisterMapped);
      cudaSetDevice(prev);
      if (e != cudaSuccess) { DF_WARN("cudaHostRegister of the segment of pid %d: %s", h.pid, cudaGetErrorString(e)); (void)cudaGetLastError(); munmap(p, h.bytes); return ncclUnhandledCudaError; }
      imp.registered = true;
    }
  }
  imports_[key] = imp;
  *base = imp.base;
  DF_INFO(SUB_P2P, "mapped heap of pid %d dev %d at %p (%s)", h.pid, h.device, (void*)imp.base, imp.ipc ? "ipc" : "direct");
  return ncclSuccess;
}

ncclResult_t devAlloc(dfcclBackend_t be, void** p, size_t bytes) {
  if (be == dfcclBackendCuda) { CUDACHECK(cudaMalloc(p, bytes)); CUDACHECK(cudaMemset(*p, 0, bytes)); }
  else { *p = calloc(1, bytes); if (!*p) return ncclSystemError; }
  return ncclSuccess;
}
ncclResult_t devFree(dfcclBackend_t be, void* p) {
  if (!p) return ncclSuccess;
  if (be == dfcclBackendCuda) { CUDACHECK(cudaFree(p)); } else ::free(p);
  return ncclSuccess;
}
ncclResult_t pinnedAlloc(dfcclBackend_t be, void** p, size_t bytes) {
  if (be == dfcclBackendCuda) { CUDACHECK(cudaHostAlloc(p, bytes, cudaHostAllocMapped | cudaHostAllocPortable)); memset(*p, 0, bytes); }
  else { *p = calloc(1, bytes); if (!*p) return ncclSystemError; }
  return ncclSuccess;
}
ncclResult_t pinnedFree(dfcclBackend_t be, void* p) {
  if (!p) return ncclSuccess;
  if (be == dfcclBackendCuda) { CUDACHECK(cudaFreeHost(p)); } else ::free(p);
  return ncclSuccess;
}
ncclResult_t devUpload(dfcclBackend_t be, void* dst, const void* src, size_t bytes) {
  if (be == dfcclBackendCuda) { CUDACHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyHostToDevice)); } else memcpy(dst, src, bytes);
  return ncclSuccess;
}
ncclResult_t devDownload(dfcclBackend_t be, void* dst, const void* src, size_t bytes) {
  if (be == dfcclBackendCuda) { CUDACHECK(cudaMemcpy(dst, src, bytes, cudaMemcpyDeviceToHost)); } else memcpy(dst, src, bytes);
  return ncclSuccess;
}
ncclResult_t devZero(dfcclBackend_t be, void* dst, size_t bytes) {
  if (be == dfcclBackendCuda) { CUDACHECK(cudaMemset(dst, 0, bytes)); } else memset(dst, 0, bytes);
  return ncclSuccess;
}

}  // namespace dfccl
