// Introspection entry points used by tests and tools: topology, tuner, logging.
#include "../common/log.h"
#include "../common/param.h"
#include "../topo/topo.h"
#include "../comm/comm.h"
#include <cstring>

using namespace dfccl;
#define DF_API extern "C" __attribute__((visibility("default")))

// Writes the cached system topology as XML into buf; returns the full length.
DF_API int dfcclTopoXml(char* buf, int cap) {
  const Topology* t = nullptr;
  if (topoGet(&t) != ncclSuccess) return -1;
  std::string s = topoToXml(*t);
  if (buf && cap > 0) { strncpy(buf, s.c_str(), cap - 1); buf[cap - 1] = 0; }
  return (int)s.size();
}
DF_API void dfcclTopoReset(void) { topoResetCache(); }
DF_API int dfcclTopoGpuCount(void) {
  const Topology* t = nullptr;
  if (topoGet(&t) != ncclSuccess) return -1;
  return (int)t->gpus.size();
}
// Path policy of the (detected or injected) topology: may devices a and b use one another's memory directly?
DF_API int dfcclTopoP2pAllowed(int a, int b) {
  const Topology* t = nullptr;
  if (topoGet(&t) != ncclSuccess) return -1;
  return topoP2pAllowed(*t, a, b) ? 1 : 0;
}
DF_API ncclResult_t dfcclTunerChoose(int kind, size_t bytes, int nranks, int maxBlocks, int nvls, int pinnedAlgo, int* algo,
                                     int* nBlocks, double* predictedUs) {
  const Topology* t = nullptr;
  DFCHECK(topoGet(&t));
  TunerChoice c = tunerChoose(*t, kind, bytes, nranks, maxBlocks, nvls != 0, pinnedAlgo, 0);
  if (algo) *algo = c.algo;
  if (nBlocks) *nBlocks = c.nBlocks;
  if (predictedUs) *predictedUs = c.predictedUs;
  return ncclSuccess;
}
DF_API double dfcclTunerPredictUs(int kind, int algo, size_t bytes, int nranks, int nBlocks) {
  const Topology* t = nullptr;
  if (topoGet(&t) != ncclSuccess) return -1.0;
  return tunerPredictUs(*t, kind, algo, bytes, nranks, nBlocks);
}
DF_API void dfcclLogReset(void) { logReset(); }
DF_API const char* dfcclLastError(void) { return lastError(); }
DF_API long long dfcclParam(const char* name, long long dflt) { return paramI64(name, dflt); }

// Which transport the communicator's members selected together: 0 = peer memory (NVLink / same process), 1 = heap in
// registered host shared memory (GPUs of one host without peer access), 2 = host-staged over the network transport.
DF_API ncclResult_t dfcclCommTransport(ncclComm_t comm, int* kind) {
  if (!comm || !kind) return ncclInvalidArgument;
  *kind = comm->netMode ? 2 : comm->shmMode ? 1 : 0;
  return ncclSuccess;
}

// Base address of `peer`'s symmetric heap as mapped in this process (own base for peer == rank):
// a buffer at offset o of the peer's heap is at base + o here.
DF_API ncclResult_t dfcclHeapPeerBase(ncclComm_t comm, int peer, void** base) {
  if (!comm || !base || peer < 0 || peer >= comm->nranks) return ncclInvalidArgument;
  *base = comm->peerHeap[peer];
  return ncclSuccess;
}
