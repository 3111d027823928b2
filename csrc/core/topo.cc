// Topology of the NVLink / NVSwitch domain.
//
// The reference walks sysfs into an XML tree of GPUs, PCI switches, CPUs and
// NICs and computes GPU-NIC distances for its inter-node transports
// (flagcx/core/topo.cc, paths.cc, xml.cc); it has no NVLink detection at all.
// Inside one NVSwitch domain the graph is flat - every GPU reaches every peer
// at full NVLink bandwidth - so the probe here records what the kernels need
// to know: which peers are directly addressable, whether native atomics and a
// multicast object are available, and the link class of each pair.  Rank 0
// writes the result as XML when FLAGCX_TOPO_DUMP_FILE is set.
#include "comm.h"
#include "log.h"

#include <cstring>
#include <cuda_runtime.h>
#include <dlfcn.h>

namespace fcx {

// NVLink state through the management library, loaded at run time (libnvidia-ml.so.1, or the library named by
// FLAGCX_NVML_LIBRARY: the tests point it at a stand-in).  Read-only queries; nothing is ever set.
namespace {
struct Nvml {
  void *h = nullptr;
  int (*init)() = nullptr;
  int (*shutdown)() = nullptr;
  int (*byBusId)(const char *, void **) = nullptr;
  int (*linkState)(void *, unsigned, unsigned *) = nullptr;
  int (*linkVersion)(void *, unsigned, unsigned *) = nullptr;
  bool ok = false;
  Nvml() {
    std::string lib = envStr("NVML_LIBRARY", "libnvidia-ml.so.1");
    h = dlopen(lib.c_str(), RTLD_NOW | RTLD_LOCAL);
    if (!h) return;
    init = (int (*)())dlsym(h, "nvmlInit_v2");
    shutdown = (int (*)())dlsym(h, "nvmlShutdown");
    byBusId = (int (*)(const char *, void **))dlsym(h, "nvmlDeviceGetHandleByPciBusId_v2");
    linkState = (int (*)(void *, unsigned, unsigned *))dlsym(h, "nvmlDeviceGetNvLinkState");
    linkVersion = (int (*)(void *, unsigned, unsigned *))dlsym(h, "nvmlDeviceGetNvLinkVersion");
    ok = init && shutdown && byBusId && linkState;
  }
  ~Nvml() { if (h) dlclose(h); }
};
}  // namespace

// Number of NVLink links that are up on the GPU with this PCI bus id, and their version (0 when unknown).
// Returns false when the management library cannot be used.
bool topoNvlinkCount(const char *busId, int *active, int *version) {
  *active = 0;
  *version = 0;
  Nvml nv;
  if (!nv.ok || nv.init() != 0) return false;
  void *dev = nullptr;
  bool found = nv.byBusId(busId, &dev) == 0;
  if (found) {
    for (unsigned link = 0; link < 32; link++) {
      unsigned up = 0;
      if (nv.linkState(dev, link, &up) != 0) break;  // past the last link of this GPU
      if (up) {
        (*active)++;
        unsigned v = 0;
        if (nv.linkVersion && nv.linkVersion(dev, link, &v) == 0) *version = (int)v;
      }
    }
  }
  nv.shutdown();
  return found;
}

// FLAGCX_TOPO_FILE (reference: flagcx/core/topo.cc:337-389, sample test/unittest/topo_demo.xml): lines
// <gpu dev="N" net="name"> attach a network port to a GPU.  Returns the port of every device index found.
static bool readTopoFile(const std::string &path, std::vector<std::string> *netOfDev, int *ranks) {
  FILE *f = fopen(path.c_str(), "r");
  if (!f) return false;
  char line[512];
  *ranks = -1;
  while (fgets(line, sizeof line, f)) {
    const char *at = strstr(line, "ranks=\"");
    if (strstr(line, "<system") && at) *ranks = atoi(at + 7);  // a dump of this library states the world it describes
    const char *g = strstr(line, "<gpu");
    if (!g) continue;
    const char *d = strstr(g, "dev=\""), *n = strstr(g, "net=\"");
    if (!d) continue;
    int dev = atoi(d + 5);
    if (dev < 0 || dev >= 1024) continue;
    std::string net;
    if (n) {
      const char *e = strchr(n + 5, '"');
      if (e) net.assign(n + 5, e);
    }
    if ((int)netOfDev->size() <= dev) netOfDev->resize(dev + 1);
    (*netOfDev)[dev] = net;
  }
  fclose(f);
  return true;
}

struct TopoRank {
  int cudaDev, smCount, multicast, ccMajor, ccMinor;
  int nvlinks, nvlinkVersion, fabric;  // links that are up, their generation, fabric (multi-node NVLink) handles supported
  unsigned long long memBytes;
  char name[64];
  char busId[32];
  int access[FCX_MAX_RANKS];   // 1 if this rank's GPU can address that rank's GPU
  int atomics[FCX_MAX_RANKS];  // native atomics over the link
  int perfRank[FCX_MAX_RANKS]; // CUDA's relative link performance (0 best)
};

static const char *pathType(const TopoRank &a, int self, int other) {
  if (self == other) return "LOC";
  return a.access[other] ? "NVL" : "SYS";  // NVLink through the switch, or across the host
}

flagcxResult_t topoProbeAndDump(flagcxComm *c) {
  std::string dump = envStr("TOPO_DUMP_FILE", "");
  std::string given = envStr("TOPO_FILE", "");
  if (!given.empty()) {
    // A topology supplied by the user (reference: FLAGCX_TOPO_FILE): it says which network port each GPU is
    // attached to.  Inside one NVSwitch domain the ports only matter to the hierarchical planner, which takes
    // the GPUs with distinct ports as the ranks of a cluster that talk to the other clusters.
    std::vector<std::string> netOfDev;
    int ranks = -1;
    if (!readTopoFile(given, &netOfDev, &ranks)) { FCX_WARN("cannot read topology file %s", given.c_str()); return flagcxSystemError; }
    if (ranks >= 0 && ranks != c->nranks && c->rank == 0)
      FCX_WARN("topology file %s describes %d ranks, the communicator has %d", given.c_str(), ranks, c->nranks);
    c->netOfRank.assign(c->nranks, "");
    int known = 0;
    for (int r = 0; r < c->nranks; r++) {
      // host-only ranks have no device index: they are numbered by rank
      int dev = c->peers[r].hostOnly ? r : c->peers[r].cudaDev;
      if (dev >= 0 && dev < (int)netOfDev.size()) { c->netOfRank[r] = netOfDev[dev]; known += !netOfDev[dev].empty(); }
    }
    if (c->rank == 0) FCX_INFO(SUB_GRAPH, "topology file %s: network port known for %d of %d ranks", given.c_str(), known, c->nranks);
  }
  bool detect = envStr("ENABLE_TOPO_DETECT", "") == "TRUE" || !dump.empty();
  if (!detect || c->hostOnly) return flagcxSuccess;
  const int n = c->nranks;
  std::vector<TopoRank> all(n);
  TopoRank &me = all[c->rank];
  memset(&me, 0, sizeof me);
  cudaDeviceProp p;
  FCX_CHECK(cudaToResult(cudaGetDeviceProperties(&p, c->cudaDev), "device properties"));
  me.cudaDev = c->cudaDev;
  me.smCount = p.multiProcessorCount;
  me.ccMajor = p.major;
  me.ccMinor = p.minor;
  me.memBytes = p.totalGlobalMem;
  me.multicast = c->heap.mcBase != nullptr;
  topoNvlinkCount(c->peers[c->rank].busId, &me.nvlinks, &me.nvlinkVersion);
  {
    int v = 0;  // CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_FABRIC_SUPPORTED
    if (cudaDeviceGetAttribute(&v, (cudaDeviceAttr)128, c->cudaDev) == cudaSuccess) me.fabric = v;
    cudaGetLastError();
  }
  snprintf(me.name, sizeof me.name, "%s", p.name);
  snprintf(me.busId, sizeof me.busId, "%s", c->peers[c->rank].busId);
  for (int r = 0; r < n && r < FCX_MAX_RANKS; r++) {
    int peerDev = c->peers[r].cudaDev;
    if (r == c->rank) { me.access[r] = 1; me.atomics[r] = 1; continue; }
    int v = 0;
    // ranks are separate processes: the peer's device index is valid here only if both see the same device list
    if (cudaDeviceCanAccessPeer(&v, c->cudaDev, peerDev) == cudaSuccess) me.access[r] = v;
    if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrNativeAtomicSupported, c->cudaDev, peerDev) == cudaSuccess) me.atomics[r] = v;
    if (cudaDeviceGetP2PAttribute(&v, cudaDevP2PAttrPerformanceRank, c->cudaDev, peerDev) == cudaSuccess) me.perfRank[r] = v;
    cudaGetLastError();
  }
  FCX_CHECK(c->bs.allGather(all.data(), sizeof(TopoRank)));
  if (c->rank != 0 || dump.empty()) return flagcxSuccess;
  FILE *f = fopen(dump.c_str(), "w");
  if (!f) { FCX_WARN("cannot write topology file %s", dump.c_str()); return flagcxSystemError; }
  fprintf(f, "<system version=\"1\" domain=\"nvswitch\" ranks=\"%d\" multicast=\"%d\">\n", n, me.multicast);
  for (int r = 0; r < n; r++) {
    const TopoRank &t = all[r];
    fprintf(f, "  <gpu rank=\"%d\" dev=\"%d\" busid=\"%s\" name=\"%s\" sm=\"%d.%d\" sms=\"%d\" mem_gib=\"%.1f\" cluster=\"%d\" nvlinks=\"%d\" "
               "nvlink_version=\"%d\" fabric=\"%d\" net=\"%s\">\n", r, t.cudaDev, t.busId, t.name, t.ccMajor, t.ccMinor, t.smCount,
            t.memBytes / 1073741824.0, c->clusterOf[r], t.nvlinks, t.nvlinkVersion, t.fabric,
            r < (int)c->netOfRank.size() ? c->netOfRank[r].c_str() : "");
    for (int q = 0; q < n; q++)
      fprintf(f, "    <path to=\"%d\" type=\"%s\" access=\"%d\" atomics=\"%d\" perf_rank=\"%d\"/>\n", q, pathType(t, r, q), t.access[q],
              t.atomics[q], t.perfRank[q]);
    fprintf(f, "  </gpu>\n");
  }
  fprintf(f, "</system>\n");
  fclose(f);
  FCX_INFO(SUB_GRAPH, "topology written to %s", dump.c_str());
  return flagcxSuccess;
}

}  // namespace fcx
