// System topology and the size -> schedule tuner.
//
// The reference detects PCI/NVLink topology from sysfs + NVML into an XML tree,
// searches rings and trees over it and feeds an analytic latency / bandwidth
// model (src/graph/{xml,topo,paths,search,connect,tuning}.cc; fake systems are
// injected with NCCL_TOPO_FILE, dumped with NCCL_TOPO_DUMP_FILE,
// src/graph/topo.cc:598-605,667-671).  On an NVSwitch machine every GPU reaches
// every peer at full link bandwidth, so the graph search collapses to a flat
// model: what remains is (a) detection - peer access matrix, NVLink presence,
// multicast (NVLS) capability - with the same file injection / dump hooks for
// tests, and (b) the cost model that picks one-shot / two-shot / NVLS and the
// number of daemon blocks per collective.
#pragma once
#include <string>
#include <vector>
#include "dfccl.h"

namespace dfccl {

enum P2pType : int { P2P_NONE = 0, P2P_PCI = 1, P2P_NVLINK = 2, P2P_SELF = 3 };

struct GpuInfo {
  int dev = 0;
  std::string name, busId;
  int cc = 0;                 // 100 for sm_100
  int sms = 0;
  size_t memBytes = 0;
  int l2Bytes = 0;
  bool multicast = false;     // CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED
  int nvlinks = -1;           // active links reported by NVML, -1 = unknown
};

struct Topology {
  std::vector<GpuInfo> gpus;
  std::vector<int> p2p;       // gpus.size()^2 entries of P2pType
  bool nvswitch = false;
  double linkGBs = 770.0;     // per direction per GPU, achievable
  double hbmGBs = 6500.0;
  double perBlockGBs = 28.0;  // what one daemon block moves over the fabric
  double hopUs = 1.8;         // one-way flag latency GPU -> GPU
  int p2pType(int a, int b) const { return p2p.empty() ? P2P_NONE : p2p[a * gpus.size() + b]; }
  bool allNvlink() const;
};

ncclResult_t topoDetect(Topology* t);                         // CUDA runtime (+ NVML when loadable)
ncclResult_t topoLoadFile(const char* path, Topology* t);
ncclResult_t topoParse(const std::string& xml, Topology* t);
std::string topoToXml(const Topology& t);
// Cached system topology; honours TOPO_FILE (inject) and TOPO_DUMP_FILE (write once).
ncclResult_t topoGet(const Topology** t);
void topoResetCache();                                        // tests

// Path policy (role of the reference's ncclTopoCheckP2p and its NCCL_P2P_LEVEL knob, src/graph/paths.cc:251-341): may
// members on devices a and b use one another's memory directly?  No when the pair has no peer access, when
// P2P_DISABLE is set, or when the pair's path is farther than P2P_LEVEL allows: LOC = the same device only,
// NVL = NVLink only, PIX / PXB / PHB / SYS = PCIe paths too (the driver reports one kind of PCIe peer path; the four
// names are accepted for compatibility).  Devices the topology does not know are left to the mapping attempt.
bool topoP2pAllowed(const Topology& t, int a, int b);

struct TunerChoice { int algo; int nBlocks; double predictedUs; };
// bytes: payload per rank as NCCL counts it (AllGather: sendcount bytes, ReduceScatter: recvcount bytes)
double tunerPredictUs(const Topology& t, int kind, int algo, size_t bytes, int nranks, int nBlocks);
TunerChoice tunerChoose(const Topology& t, int kind, size_t bytes, int nranks, int maxBlocks, bool nvlsAvailable,
                        int pinnedAlgo = dfcclAlgoAuto, int pinnedBlocks = 0);
size_t tunerWireBytes(int kind, int algo, size_t bytes, int nranks);

}  // namespace dfccl
