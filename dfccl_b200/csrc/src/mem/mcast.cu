#include "mcast.h"
#include "../comm/comm.h"
#include "../common/log.h"
#include "../common/param.h"
#include <cuda.h>
#include <cstring>
#include <sys/syscall.h>
#include <unistd.h>

namespace dfccl {

ncclResult_t NvlsArena::alloc(size_t n, uint64_t* off) {
  n = (n + 511) & ~(size_t)511;
  std::lock_guard<std::mutex> l(mu);
  if (bump + n > bytes) return ncclInvalidUsage;
  *off = bump;
  marks.push_back(bump);
  bump += n;
  return ncclSuccess;
}

void NvlsArena::release(uint64_t off) {
  std::lock_guard<std::mutex> l(mu);
  if (!marks.empty() && marks.back() == off) { bump = off; marks.pop_back(); }
}

namespace {

struct Drv {
  CUresult (*mcCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*mcAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*mcBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*mcUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*mcGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
  CUresult (*memCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*memRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*memExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*memImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*memReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*memAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*memUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*memSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*memGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*devGet)(CUdevice*, int) = nullptr;
  CUresult (*devAttr)(int*, CUdevice_attribute, CUdevice) = nullptr;
  bool ok = false;
};

template <typename F>
bool entry(const char* name, F* fn) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    (void)cudaGetLastError();
    return false;
  }
  *fn = (F)p;
  return true;
}

const Drv& drv() {
  static Drv d;
  static std::once_flag once;
  std::call_once(once, [] {
    d.ok = entry("cuMulticastCreate", &d.mcCreate) && entry("cuMulticastAddDevice", &d.mcAddDevice) &&
           entry("cuMulticastBindMem", &d.mcBindMem) && entry("cuMulticastUnbind", &d.mcUnbind) &&
           entry("cuMulticastGetGranularity", &d.mcGranularity) && entry("cuMemCreate", &d.memCreate) &&
           entry("cuMemRelease", &d.memRelease) && entry("cuMemExportToShareableHandle", &d.memExport) &&
           entry("cuMemImportFromShareableHandle", &d.memImport) && entry("cuMemAddressReserve", &d.memReserve) &&
           entry("cuMemAddressFree", &d.memAddressFree) && entry("cuMemMap", &d.memMap) && entry("cuMemUnmap", &d.memUnmap) &&
           entry("cuMemSetAccess", &d.memSetAccess) && entry("cuMemGetAllocationGranularity", &d.memGranularity) &&
           entry("cuDeviceGet", &d.devGet) && entry("cuDeviceGetAttribute", &d.devAttr);
  });
  return d;
}

struct Msg { int32_t pid, fd, ok, device; uint64_t hostHash, off; };

// Every member reports whether its last step worked; the arena exists only if all did.
bool allOk(ncclComm* c, bool mine) {
  std::vector<int32_t> v(c->nranks, 0);
  v[c->rank] = mine ? 1 : 0;
  if (c->boot->allGather(v.data(), sizeof(int32_t)) != ncclSuccess) return false;
  for (int x : v) if (!x) return false;
  return true;
}

void releaseCuda(NvlsArena* a) {
  const Drv& d = drv();
  if (a->mc) { d.memUnmap((CUdeviceptr)a->mc, a->bytes); d.memAddressFree((CUdeviceptr)a->mc, a->bytes); a->mc = nullptr; }
  if (a->uc) { d.memUnmap((CUdeviceptr)a->uc, a->bytes); d.memAddressFree((CUdeviceptr)a->uc, a->bytes); a->uc = nullptr; }
  if (a->bound) { CUdevice dev; if (d.devGet(&dev, a->device) == CUDA_SUCCESS) d.mcUnbind(a->mcHandle, dev, 0, a->bytes); a->bound = false; }
  if (a->memHandle) { d.memRelease(a->memHandle); a->memHandle = 0; }
  if (a->mcHandle) { d.memRelease(a->mcHandle); a->mcHandle = 0; }
}

ncclResult_t createHost(ncclComm* c, size_t bytes, NvlsArena* a) {
  DFCHECK(c->heap->alloc(bytes, &a->heapOff, true));
  a->uc = c->heap->base() + a->heapOff;
  std::vector<Msg> all(c->nranks);
  memset(all.data(), 0, sizeof(Msg) * all.size());
  all[c->rank].off = a->heapOff;
  DFCHECK(c->boot->allGather(all.data(), sizeof(Msg)));
  a->peers.resize(c->nranks);
  for (int j = 0; j < c->nranks; ++j) a->peers[j] = c->peerHeap[j] + all[j].off;
  DFCHECK(devAlloc(c->backend, (void**)&a->peersDev, sizeof(char*) * c->nranks));
  DFCHECK(devUpload(c->backend, a->peersDev, a->peers.data(), sizeof(char*) * c->nranks));
  return ncclSuccess;
}

}  // namespace

ncclResult_t nvlsArenaCreate(ncclComm* c, size_t bytes, NvlsArena** out) {
  *out = nullptr;
  if (c->nranks < 2) return ncclSuccess;
  auto a = new NvlsArena();
  a->backend = c->backend; a->device = c->device;
  if (c->backend != dfcclBackendCuda) {
    a->bytes = (bytes + 511) & ~(size_t)511;
    ncclResult_t r = createHost(c, a->bytes, a);
    if (r != ncclSuccess) { delete a; return r; }
  } else {
    const Drv& d = drv();
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    cudaFree(0);
    CUdevice dev = 0;
    // ---- 1. can every member do it, and does each sit on a device of its own?
    std::vector<Msg> all(c->nranks);
    memset(all.data(), 0, sizeof(Msg) * all.size());
    Msg& me = all[c->rank];
    me.pid = (int32_t)getpid(); me.device = c->device; me.hostHash = hostHash(); me.fd = -1;
    int sup = 0;
    me.ok = d.ok && d.devGet(&dev, c->device) == CUDA_SUCCESS &&
            d.devAttr(&sup, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS && sup;
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)c->nranks;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 2u << 20;
    mp.size = (bytes + gran - 1) / gran * gran;
    if (me.ok) {
      size_t g = 0;
      if (d.mcGranularity(&g, &mp, CU_MULTICAST_GRANULARITY_MINIMUM) == CUDA_SUCCESS && g) gran = g; else me.ok = 0;
      mp.size = (bytes + gran - 1) / gran * gran;
    }
    a->bytes = mp.size;
    // ---- 2. the first member creates the multicast object and exports it
    int fd = -1;
    if (me.ok && c->rank == 0) {
      CUmemGenericAllocationHandle h = 0;
      CUresult r = d.mcCreate(&h, &mp);
      if (r == CUDA_SUCCESS) r = d.memExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
      if (r != CUDA_SUCCESS) { DF_INFO(SUB_INIT, "NVLS: multicast object could not be created (%d)", (int)r); me.ok = 0; }
      a->mcHandle = h;
      me.fd = fd;
    }
    bool fail = c->boot->allGather(all.data(), sizeof(Msg)) != ncclSuccess;
    for (int j = 0; j < c->nranks && !fail; ++j) {
      if (!all[j].ok || all[j].hostHash != all[c->rank].hostHash) fail = true;
      for (int k = 0; k < j; ++k) if (all[k].device == all[j].device) fail = true;     // one device per member
    }
    // ---- 3. the others take a duplicate of the descriptor and import it
    bool mine = !fail;
    if (mine && c->rank != 0) {
      int local = -1;
      if (all[0].pid == (int32_t)getpid()) local = dup(all[0].fd);
      else {
        long pfd = syscall(SYS_pidfd_open, (pid_t)all[0].pid, 0);
        if (pfd >= 0) { local = (int)syscall(SYS_pidfd_getfd, (int)pfd, all[0].fd, 0); close((int)pfd); }
      }
      CUmemGenericAllocationHandle h = 0;
      if (local < 0 || d.memImport(&h, (void*)(uintptr_t)local, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS) {
        DF_INFO(SUB_INIT, "NVLS: could not import the multicast handle (descriptor %d)", local);
        mine = false;
      }
      if (local >= 0) close(local);
      a->mcHandle = h;
    }
    bool ok = allOk(c, mine);
    if (fd >= 0) close(fd);
    // ---- 4. add the devices (all of them before anything is bound), then bind the local memory
    if (ok) ok = allOk(c, d.mcAddDevice(a->mcHandle, dev) == CUDA_SUCCESS);
    if (ok) {
      CUmemAllocationProp ap;
      memset(&ap, 0, sizeof(ap));
      ap.type = CU_MEM_ALLOCATION_TYPE_PINNED;
      ap.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
      ap.location.id = c->device;
      ap.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
      CUmemGenericAllocationHandle mh = 0;
      CUresult r = d.memCreate(&mh, a->bytes, &ap, 0);
      if (r == CUDA_SUCCESS) { a->memHandle = mh; r = d.mcBindMem(a->mcHandle, 0, mh, 0, a->bytes, 0); if (r == CUDA_SUCCESS) a->bound = true; }
      CUmemAccessDesc acc;
      memset(&acc, 0, sizeof(acc));
      acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = c->device; acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      CUdeviceptr va = 0;
      if (r == CUDA_SUCCESS) r = d.memReserve(&va, a->bytes, gran, 0, 0);
      if (r == CUDA_SUCCESS) { r = d.memMap(va, a->bytes, 0, a->memHandle, 0); if (r == CUDA_SUCCESS) a->uc = (char*)va; else d.memAddressFree(va, a->bytes); }
      if (r == CUDA_SUCCESS) r = d.memSetAccess(va, a->bytes, &acc, 1);
      if (r == CUDA_SUCCESS && cudaMemset(a->uc, 0, a->bytes) != cudaSuccess) r = CUDA_ERROR_UNKNOWN;
      if (r != CUDA_SUCCESS) DF_INFO(SUB_INIT, "NVLS: local memory could not be created, bound or mapped (%d)", (int)r);
      ok = allOk(c, r == CUDA_SUCCESS);              // also the barrier: every member is bound before anyone maps the multicast view
    }
    if (ok) {
      CUmemAccessDesc acc;
      memset(&acc, 0, sizeof(acc));
      acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE; acc.location.id = c->device; acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
      CUdeviceptr va = 0;
      CUresult r = d.memReserve(&va, a->bytes, gran, 0, 0);
      if (r == CUDA_SUCCESS) { r = d.memMap(va, a->bytes, 0, a->mcHandle, 0); if (r == CUDA_SUCCESS) a->mc = (char*)va; else d.memAddressFree(va, a->bytes); }
      if (r == CUDA_SUCCESS) r = d.memSetAccess(va, a->bytes, &acc, 1);
      if (r == CUDA_SUCCESS) cudaDeviceSynchronize();
      ok = allOk(c, r == CUDA_SUCCESS);
    }
    cudaSetDevice(prev);
    if (!ok) {
      if (d.ok) releaseCuda(a);
      delete a;
      DF_INFO(SUB_INIT, "NVLS arena not available on this communicator; collectives use peer loads and stores");
      return ncclSuccess;
    }
  }
  // the front of the arena stages stream-ordered collectives whose buffers live elsewhere
  a->streamBytes = std::min<size_t>(a->bytes / 2, (size_t)paramI64("NVLS_STREAM_BYTES", 64ll << 20)) & ~(size_t)1023;
  a->bump = a->streamBytes;
  DF_INFO(SUB_INIT, "NVLS arena: %zu MiB (%zu MiB stream staging), unicast %p multicast %p", a->bytes >> 20, a->streamBytes >> 20,
          (void*)a->uc, (void*)a->mc);
  *out = a;
  return ncclSuccess;
}

void nvlsArenaDestroy(ncclComm* c, NvlsArena* a) {
  if (!a) return;
  if (a->backend == dfcclBackendCuda) {
    int prev = 0;
    cudaGetDevice(&prev);
    cudaSetDevice(a->device);
    cudaDeviceSynchronize();
    releaseCuda(a);
    cudaSetDevice(prev);
  } else {
    c->heap->free(a->heapOff);
    devFree(a->backend, a->peersDev);
  }
  delete a;
}

}  // namespace dfccl
