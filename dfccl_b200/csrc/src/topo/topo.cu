#include "topo.h"
#include "../common/log.h"
#include "../common/param.h"
#include <cctype>
#include <algorithm>
#include <cmath>
#include <cstring>
#include <dlfcn.h>
#include <fstream>
#include <mutex>
#include <sstream>
#include <cuda.h>
#include <cuda_runtime.h>

namespace dfccl {

bool Topology::allNvlink() const {
  size_t n = gpus.size();
  for (size_t a = 0; a < n; ++a)
    for (size_t b = 0; b < n; ++b)
      if (a != b && p2p[a * n + b] != P2P_NVLINK) return false;
  return n > 0;
}

// ---- NVML, loaded lazily so that the library has no link-time dependency on it
// (the reference wraps NVML the same way, src/misc/nvmlwrap.cc)
namespace {
struct Nvml {
  void* lib = nullptr;
  int (*init)() = nullptr;
  int (*byBusId)(const char*, void**) = nullptr;
  int (*linkState)(void*, unsigned, int*) = nullptr;
  bool ok = false;
  Nvml() {
    lib = dlopen("libnvidia-ml.so.1", RTLD_NOW | RTLD_LOCAL);
    if (!lib) return;
    init = (int (*)())dlsym(lib, "nvmlInit_v2");
    byBusId = (int (*)(const char*, void**))dlsym(lib, "nvmlDeviceGetHandleByPciBusId_v2");
    linkState = (int (*)(void*, unsigned, int*))dlsym(lib, "nvmlDeviceGetNvLinkState");
    ok = init && byBusId && linkState && init() == 0;
  }
};
Nvml& nvml() { static Nvml n; return n; }
}  // namespace

ncclResult_t topoDetect(Topology* t) {
  *t = Topology();
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
  typedef CUresult (*GetAttr)(int*, CUdevice_attribute, CUdevice);
  GetAttr cuAttr = nullptr;
  if (n > 0) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuDeviceGetAttribute", &fn, cudaEnableDefault, &q) == cudaSuccess) cuAttr = (GetAttr)fn;
    (void)cudaGetLastError();
  }
  for (int d = 0; d < n; ++d) {
    cudaDeviceProp p;
    CUDACHECK(cudaGetDeviceProperties(&p, d));
    GpuInfo g;
    g.dev = d; g.name = p.name; g.cc = p.major * 10 + p.minor; g.sms = p.multiProcessorCount;
    g.memBytes = p.totalGlobalMem; g.l2Bytes = p.l2CacheSize;
    char bus[32];
    snprintf(bus, sizeof(bus), "%04x:%02x:%02x.0", p.pciDomainID, p.pciBusID, p.pciDeviceID);
    g.busId = bus;
    int mc = 0;
    if (cuAttr && cuAttr(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, d) == CUDA_SUCCESS) g.multicast = mc != 0;
    if (nvml().ok) {
      void* h = nullptr;
      if (nvml().byBusId(bus, &h) == 0) {
        int active = 0;
        for (unsigned l = 0; l < 18; ++l) { int on = 0; if (nvml().linkState(h, l, &on) == 0 && on) ++active; }
        g.nvlinks = active;
      }
    }
    t->gpus.push_back(g);
  }
  t->p2p.assign((size_t)n * n, P2P_NONE);
  for (int a = 0; a < n; ++a)
    for (int b = 0; b < n; ++b) {
      if (a == b) { t->p2p[a * n + b] = P2P_SELF; continue; }
      int can = 0, perf = 0, native = 0;
      cudaDeviceCanAccessPeer(&can, a, b);
      if (!can) continue;
      cudaDeviceGetP2PAttribute(&perf, cudaDevP2PAttrPerformanceRank, a, b);
      cudaDeviceGetP2PAttribute(&native, cudaDevP2PAttrNativeAtomicSupported, a, b);
      t->p2p[a * n + b] = native ? P2P_NVLINK : P2P_PCI;      // native atomics exist only over NVLink
    }
  (void)cudaGetLastError();
  // all-to-all NVLink among more than two GPUs means a switch (direct meshes stop at pairs here)
  t->nvswitch = n > 2 && t->allNvlink();
  if (!t->gpus.empty() && t->gpus[0].cc < 100) { t->linkGBs = 370.0; t->hbmGBs = 3000.0; }
  return ncclSuccess;
}

// ---- tiny XML subset: <system ...> <gpu .../> <p2p a= b= type=/> </system>
static std::string attr(const std::string& tag, const char* key) {
  std::string k = std::string(key) + "=\"";
  size_t p = tag.find(k);
  if (p == std::string::npos) return "";
  p += k.size();
  size_t e = tag.find('"', p);
  return e == std::string::npos ? "" : tag.substr(p, e - p);
}

ncclResult_t topoParse(const std::string& xml, Topology* t) {
  *t = Topology();
  std::vector<std::pair<std::pair<int, int>, int>> links;
  size_t pos = 0;
  bool sawSystem = false;
  while ((pos = xml.find('<', pos)) != std::string::npos) {
    size_t end = xml.find('>', pos);
    if (end == std::string::npos) break;
    std::string tag = xml.substr(pos + 1, end - pos - 1);
    pos = end + 1;
    if (tag.compare(0, 6, "system") == 0) {
      sawSystem = true;
      t->nvswitch = attr(tag, "nvswitch") == "1";
      if (!attr(tag, "link_gbs").empty()) t->linkGBs = atof(attr(tag, "link_gbs").c_str());
      if (!attr(tag, "hbm_gbs").empty()) t->hbmGBs = atof(attr(tag, "hbm_gbs").c_str());
      if (!attr(tag, "block_gbs").empty()) t->perBlockGBs = atof(attr(tag, "block_gbs").c_str());
      if (!attr(tag, "hop_us").empty()) t->hopUs = atof(attr(tag, "hop_us").c_str());
    } else if (tag.compare(0, 3, "gpu") == 0) {
      GpuInfo g;
      g.dev = atoi(attr(tag, "dev").c_str()); g.name = attr(tag, "name"); g.busId = attr(tag, "busid");
      g.cc = atoi(attr(tag, "sm").c_str()); g.sms = atoi(attr(tag, "sms").c_str());
      g.memBytes = (size_t)atoll(attr(tag, "mem").c_str()); g.l2Bytes = atoi(attr(tag, "l2").c_str());
      g.multicast = attr(tag, "multicast") == "1";
      g.nvlinks = attr(tag, "nvlinks").empty() ? -1 : atoi(attr(tag, "nvlinks").c_str());
      t->gpus.push_back(g);
    } else if (tag.compare(0, 3, "p2p") == 0) {
      std::string ty = attr(tag, "type");
      int v = ty == "NVL" ? P2P_NVLINK : ty == "PCI" ? P2P_PCI : P2P_NONE;
      links.push_back({{atoi(attr(tag, "a").c_str()), atoi(attr(tag, "b").c_str())}, v});
    }
  }
  if (!sawSystem) { DF_WARN("topology file has no <system> element"); return ncclInvalidArgument; }
  size_t n = t->gpus.size();
  t->p2p.assign(n * n, P2P_NONE);
  for (size_t i = 0; i < n; ++i) t->p2p[i * n + i] = P2P_SELF;
  for (auto& l : links) {
    int a = l.first.first, b = l.first.second;
    if (a < 0 || b < 0 || (size_t)a >= n || (size_t)b >= n) { DF_WARN("topology file: p2p %d-%d out of range", a, b); return ncclInvalidArgument; }
    t->p2p[a * n + b] = l.second;
    t->p2p[b * n + a] = l.second;
  }
  return ncclSuccess;
}

ncclResult_t topoLoadFile(const char* path, Topology* t) {
  std::ifstream in(path);
  if (!in) { DF_WARN("cannot open topology file %s", path); return ncclSystemError; }
  std::stringstream ss;
  ss << in.rdbuf();
  return topoParse(ss.str(), t);
}

std::string topoToXml(const Topology& t) {
  std::ostringstream o;
  o << "<system nvswitch=\"" << (t.nvswitch ? 1 : 0) << "\" link_gbs=\"" << t.linkGBs << "\" hbm_gbs=\"" << t.hbmGBs
    << "\" block_gbs=\"" << t.perBlockGBs << "\" hop_us=\"" << t.hopUs << "\">\n";
  for (auto& g : t.gpus)
    o << "  <gpu dev=\"" << g.dev << "\" name=\"" << g.name << "\" busid=\"" << g.busId << "\" sm=\"" << g.cc << "\" sms=\""
      << g.sms << "\" mem=\"" << g.memBytes << "\" l2=\"" << g.l2Bytes << "\" multicast=\"" << (g.multicast ? 1 : 0)
      << "\" nvlinks=\"" << g.nvlinks << "\"/>\n";
  size_t n = t.gpus.size();
  for (size_t a = 0; a < n; ++a)
    for (size_t b = a + 1; b < n; ++b) {
      int v = t.p2p[a * n + b];
      if (v == P2P_NONE) continue;
      o << "  <p2p a=\"" << a << "\" b=\"" << b << "\" type=\"" << (v == P2P_NVLINK ? "NVL" : "PCI") << "\"/>\n";
    }
  o << "</system>\n";
  return o.str();
}

bool topoP2pAllowed(const Topology& t, int a, int b) {
  if (paramI64("P2P_DISABLE", 0) != 0) return false;
  const int n = (int)t.gpus.size();
  if (a < 0 || b < 0 || a >= n || b >= n) return true;
  const int type = t.p2pType(a, b);
  if (type == P2P_NONE) return false;
  std::string level = paramStr("P2P_LEVEL", "SYS");
  for (auto& ch : level) ch = (char)toupper((unsigned char)ch);
  if (level == "LOC" || level == "0") return type == P2P_SELF;
  if (level == "NVL" || level == "1") return type == P2P_SELF || type == P2P_NVLINK;
  return true;                                        // PIX, PXB, PHB, SYS (2..5): any peer path the driver offers
}

namespace {
std::mutex g_mu;
Topology g_topo;
bool g_have = false;
}  // namespace

void topoResetCache() { std::lock_guard<std::mutex> l(g_mu); g_have = false; }

ncclResult_t topoGet(const Topology** t) {
  std::lock_guard<std::mutex> l(g_mu);
  if (!g_have) {
    std::string inject = paramStr("TOPO_FILE", "");
    if (!inject.empty()) { DFCHECK(topoLoadFile(inject.c_str(), &g_topo)); DF_INFO(SUB_GRAPH, "topology loaded from %s", inject.c_str()); }
    else DFCHECK(topoDetect(&g_topo));
    if (double v = paramF64("LINK_GBS", 0)) g_topo.linkGBs = v;
    if (double v = paramF64("BLOCK_GBS", 0)) g_topo.perBlockGBs = v;
    std::string dump = paramStr("TOPO_DUMP_FILE", "");
    if (!dump.empty()) { std::ofstream o(dump); o << topoToXml(g_topo); }
    g_have = true;
  }
  *t = &g_topo;
  return ncclSuccess;
}

// ---- cost model
size_t tunerWireBytes(int kind, int algo, size_t bytes, int n) {
  if (n <= 1) return 0;
  switch (kind) {
    case dfcclCollAllReduce:
      if (algo == dfcclAlgoOneShot) return bytes * (n - 1);
      if (algo == dfcclAlgoNvls) return 2 * bytes / n;            // the switch reduces and replicates
      return 2 * bytes * (n - 1) / n;
    case dfcclCollAllGather: return bytes * (n - 1);               // my slice to every peer
    case dfcclCollReduceScatter: return bytes * (n - 1);           // every peer's slice of my chunk
    case dfcclCollBroadcast: return bytes;                         // per non-root; the root's egress is (n-1) x
    case dfcclCollReduce: return 2 * bytes * (n - 1) / n;
    default: return bytes;
  }
}

double tunerPredictUs(const Topology& t, int kind, int algo, size_t bytes, int n, int nBlocks) {
  if (n <= 1) return 1.0 + (double)bytes * 2 / (t.hbmGBs * 1e3);
  // three dependent hops: arrival flag, remote load round trip (or store), done flag
  double lat = t.hopUs * (algo == dfcclAlgoOneShot ? 3.0 : 4.0);
  double bw = std::min(t.linkGBs, t.perBlockGBs * nBlocks * (algo == dfcclAlgoNvls ? 3.0 : 1.0));
  double wire = (double)tunerWireBytes(kind, algo, bytes, n);
  if (kind == dfcclCollBroadcast) bw = std::min(bw, t.linkGBs / (n - 1));   // root egress shared by the pullers
  return lat + wire / (bw * 1e3);
}

TunerChoice tunerChoose(const Topology& t, int kind, size_t bytes, int n, int maxBlocks, bool nvls, int pinnedAlgo, int pinnedBlocks) {
  std::string envAlgo = paramStr("ALGO", "");
  if (pinnedAlgo == dfcclAlgoAuto && !envAlgo.empty()) {
    if (!strcasecmp(envAlgo.c_str(), "oneshot")) pinnedAlgo = dfcclAlgoOneShot;
    else if (!strcasecmp(envAlgo.c_str(), "twoshot")) pinnedAlgo = dfcclAlgoTwoShot;
    else if (!strcasecmp(envAlgo.c_str(), "nvls")) pinnedAlgo = dfcclAlgoNvls;
    else if (!strcasecmp(envAlgo.c_str(), "push")) pinnedAlgo = dfcclAlgoAuto;      // chosen by the callers, by size
    else DF_INFO(SUB_TUNING, "ALGO=%s names no schedule of this engine (oneshot|twoshot|nvls|push); ignored", envAlgo.c_str());
  }
  if (pinnedAlgo == dfcclAlgoPush) pinnedAlgo = dfcclAlgoAuto;                      // block count as for the size; the callers switch the schedule
  if (pinnedBlocks == 0) pinnedBlocks = (int)paramI64("NBLOCKS", 0);
  const size_t minPerBlock = (size_t)paramI64("MIN_BYTES_PER_BLOCK", 32 << 10);
  TunerChoice best{dfcclAlgoTwoShot, 1, 1e30};
  int algos[3] = {dfcclAlgoOneShot, dfcclAlgoTwoShot, dfcclAlgoNvls};
  for (int a : algos) {
    if (pinnedAlgo != dfcclAlgoAuto && a != pinnedAlgo) continue;
    if (a == dfcclAlgoNvls && !(nvls && kind == dfcclCollAllReduce)) continue;
    if (a == dfcclAlgoNvls && pinnedAlgo != dfcclAlgoNvls && bytes < (size_t)paramI64("NVLS_MIN_BYTES", 256 << 10)) continue;
    if (a == dfcclAlgoOneShot && kind != dfcclCollAllReduce) continue;
    size_t work = bytes * (kind == dfcclCollAllGather || kind == dfcclCollReduceScatter ? 1 : 1);
    int nb = pinnedBlocks ? pinnedBlocks : (int)std::min<size_t>(maxBlocks, std::max<size_t>(1, work / minPerBlock));
    nb = std::max(1, std::min(nb, maxBlocks));
    double us = tunerPredictUs(t, kind, a, bytes, n, nb);
    if (us < best.predictedUs) best = {a, nb, us};
  }
  if (best.predictedUs >= 1e30) {      // the pinned schedule does not exist for this kind: fall back
    int nb = pinnedBlocks ? pinnedBlocks : (int)std::min<size_t>(maxBlocks, std::max<size_t>(1, bytes / minPerBlock));
    nb = std::max(1, std::min(nb, maxBlocks));
    best = {dfcclAlgoTwoShot, nb, tunerPredictUs(t, kind, dfcclAlgoTwoShot, bytes, n, nb)};
  }
  return best;
}

}  // namespace dfccl
