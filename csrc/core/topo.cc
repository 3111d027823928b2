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

namespace fcx {

struct TopoRank {
  int cudaDev, smCount, multicast, ccMajor, ccMinor;
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
    // A topology supplied by the user replaces the probe (reference: FLAGCX_TOPO_FILE).  Inside one NVSwitch
    // domain nothing is derived from it; it is checked against the communicator and reported.
    if (c->rank == 0) {
      FILE *f = fopen(given.c_str(), "r");
      if (!f) { FCX_WARN("cannot read topology file %s", given.c_str()); return flagcxSystemError; }
      char line[512];
      int ranks = -1;
      while (fgets(line, sizeof line, f)) {
        const char *at = strstr(line, "ranks=\"");
        if (strstr(line, "<system") && at) { ranks = atoi(at + 7); break; }
      }
      fclose(f);
      if (ranks != c->nranks) FCX_WARN("topology file %s describes %d ranks, the communicator has %d", given.c_str(), ranks, c->nranks);
      else FCX_INFO(SUB_GRAPH, "topology taken from %s (%d ranks)", given.c_str(), ranks);
    }
    return flagcxSuccess;
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
    fprintf(f, "  <gpu rank=\"%d\" dev=\"%d\" busid=\"%s\" name=\"%s\" sm=\"%d.%d\" sms=\"%d\" mem_gib=\"%.1f\" cluster=\"%d\">\n", r, t.cudaDev,
            t.busId, t.name, t.ccMajor, t.ccMinor, t.smCount, t.memBytes / 1073741824.0, c->clusterOf[r]);
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
