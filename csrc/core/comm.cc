// Communicator life cycle, memory API and queries.
// Reference behaviour being matched: flagcx/flagcx.cc:129-697.
#include "comm.h"
#include "hosttypes.h"
#include "log.h"

#include <algorithm>
#include <cstring>
#include <set>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <unistd.h>

namespace fcx {

// Live communicators, and destroyed ones that still lend heap memory out.  validComm never dereferences a
// pointer that is in neither set, so a stale handle is refused instead of read.
static std::mutex gCommMu;
static std::set<flagcxComm *> gLive, gLent;

bool validComm(flagcxComm_t c) {
  if (!c) return false;
  std::lock_guard<std::mutex> lk(gCommMu);
  return gLive.count(c) != 0 && c->magic == 0xF1A6C0DE && !c->destroyed;
}

flagcxResult_t cudaToResult(cudaError_t e, const char *what) {
  if (e == cudaSuccess) return flagcxSuccess;
  FCX_WARN("%s: %s", what, cudaGetErrorString(e));
  cudaGetLastError();
  return flagcxUnhandledDeviceError;
}

void fifoStop(flagcxComm *c);     // fifo.cc
void c2cDestroy(flagcxComm *c);   // c2c/planner.cc
flagcxResult_t topoProbeAndDump(flagcxComm *c);  // topo.cc
bool topoNvlinkCount(const char *busId, int *active, int *version);

// Clusters: ranks with the same vendor string form a cluster; each cluster
// can further be cut into k equal parts with FLAGCX_CLUSTER_SPLIT_LIST
// (reference: flagcx/core/cluster.cc:23-124).  On a box of identical GPUs the
// split list is the only way to get more than one cluster.
static void detectClusters(flagcxComm *c) {
  const int n = c->nranks;
  c->clusterOf.assign(n, 0);
  int nc = 0;
  for (int r = 0; r < n; r++) {
    if (r > 0 && strncmp(c->peers[r].vendor, c->peers[r - 1].vendor, sizeof c->peers[r].vendor) != 0) nc++;
    c->clusterOf[r] = nc;
  }
  nc++;
  std::string split = envStr("CLUSTER_SPLIT_LIST", "");
  if (!split.empty()) {
    std::vector<int> ks;
    for (size_t pos = 0; pos <= split.size();) {
      size_t comma = split.find(',', pos);
      ks.push_back(atoi(split.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos).c_str()));
      if (comma == std::string::npos) break;
      pos = comma + 1;
    }
    std::vector<int> out(n);
    int next = 0;
    for (int cl = 0; cl < nc; cl++) {
      std::vector<int> members;
      for (int r = 0; r < n; r++)
        if (c->clusterOf[r] == cl) members.push_back(r);
      int k = cl < (int)ks.size() ? ks[cl] : 1;
      if (k < 1 || (int)members.size() % k != 0) {
        FCX_WARN("FLAGCX_CLUSTER_SPLIT_LIST: cluster %d has %zu ranks, not divisible by %d; left whole", cl, members.size(), k);
        k = 1;
      }
      int per = (int)members.size() / k;
      for (int i = 0; i < (int)members.size(); i++) out[members[i]] = next + i / per;
      next += k;
    }
    c->clusterOf = out;
    nc = next;
  }
  c->nclusters = nc;
  c->myCluster = c->clusterOf[c->rank];
}

flagcxResult_t commCreate(flagcxComm **out, int nranks, const BootstrapHandle &h, int rank, double heapScale, unsigned flags,
                          size_t stageOverride, size_t userOverride) {
  if (nranks < 1 || rank < 0 || rank >= nranks) return flagcxInvalidArgument;
  std::unique_ptr<flagcxComm> c(new flagcxComm);
  c->rank = rank;
  c->nranks = nranks;
  c->bs.setAbortFlag(&c->abortFlag);
  FCX_CHECK(c->bs.init(h, rank, nranks));

  int ndev = 0;
  bool haveGpu = cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0;
  cudaGetLastError();
  bool forceHost = envInt("USE_HOST_COMM", 0) != 0;
  // Variables of the reference that select between its own transports and the vendor library have nothing to
  // select here (every path is this library's own): they are accepted and reported, never an error.
  for (const char *name : {"USE_HETERO_COMM", "RUNTIME_PROXY", "FORCE_NET_SOCKET", "USENET", "DMABUF_ENABLE", "C2C_SEARCH_GRANULARITY"})
    if (!envStr(name, "").empty()) FCX_INFO(SUB_ENV, "FLAGCX_%s=%s accepted; it changes nothing inside one NVSwitch domain", name, envStr(name, "").c_str());
  if (flags & FLAGCX_INIT_HOST_ONLY) haveGpu = false;  // buffers of this communicator are host memory
  c->hostOnly = !haveGpu;
  c->hostFallback = haveGpu && forceHost;
  if (haveGpu) cudaGetDevice(&c->cudaDev);
  setLogRank(rank, c->cudaDev);

  c->peers.resize(nranks);
  PeerInfo &me = c->peers[rank];
  memset(&me, 0, sizeof me);
  me.hostHash = hostHash();
  me.pid = getpid();
  me.cudaDev = c->cudaDev;
  me.hostOnly = c->hostOnly || c->hostFallback;
  snprintf(me.vendor, sizeof me.vendor, "%s", haveGpu ? "NVIDIA" : "HOST");
  if (haveGpu) cudaDeviceGetPCIBusId(me.busId, sizeof me.busId, c->cudaDev);
  FCX_CHECK(c->bs.allGather(c->peers.data(), sizeof(PeerInfo)));

  bool anyHost = false;
  for (auto &p : c->peers) anyHost = anyHost || p.hostOnly;
  if (anyHost && !c->hostOnly) c->hostFallback = true;  // one rank without a GPU path drags all to the host path
  detectClusters(c.get());

  if (!c->hostOnly && !c->hostFallback) {
    if (nranks > FCX_MAX_RANKS) {
      FCX_WARN("this build drives one NVSwitch domain: at most %d ranks per communicator, got %d", FCX_MAX_RANKS, nranks);
      return flagcxNotSupported;
    }
    for (int r = 0; r < nranks; r++) {
      if (c->peers[r].hostHash != me.hostHash) {
        FCX_WARN("rank %d is on another host; the inter-node transport is not part of this build", r);
        return flagcxNotSupported;
      }
      if (r != rank && c->peers[r].cudaDev == c->cudaDev && strcmp(c->peers[r].busId, me.busId) == 0) {
        FCX_WARN("ranks %d and %d use the same GPU %s", rank, r, me.busId);
        return flagcxInvalidUsage;
      }
    }
    size_t stage = (size_t)((double)envInt("STAGE_BYTES", 512ll << 20) * heapScale);
    if (stageOverride) stage = stageOverride;
    stage = std::max<size_t>(stage, 1u << 20) & ~(size_t)4095;
    size_t chunk = (size_t)envInt("P2P_CHUNK_BYTES", 16ll << 20) & ~(size_t)4095;
    size_t user = (size_t)((double)envInt("HEAP_USER_BYTES", 512ll << 20) * heapScale);
    if (userOverride) user = (userOverride + 4095) & ~(size_t)4095;
    size_t p2pOff = FCX_OFF_STAGE + 2 * stage;
    size_t userOff = p2pOff + (size_t)FCX_MAX_RANKS * 2 * chunk;
    size_t total = userOff + user;
    int mode = (int)envInt("HEAP_MODE", 0);  // 0 auto, 1 vmm, 2 ipc
    bool wantMc = envInt("NVLS_ENABLE", 1) != 0;
    FCX_CHECK(c->heap.create(c->bs, c->cudaDev, total, mode, wantMc));
    FCX_CHECK(cudaToResult(cudaMemset(c->heap.base[rank], 0, FCX_OFF_STAGE), "clearing the control block"));
    FCX_CHECK(cudaToResult(cudaHostAlloc((void **)&c->errHost, 4096, cudaHostAllocMapped), "cudaHostAlloc"));
    memset(c->errHost, 0, 4096);
    c->abortHost = (uint32_t *)((char *)c->errHost + 2048);
    FCX_CHECK(cudaToResult(cudaMalloc((void **)&c->segsDev, sizeof(char *) * FCX_MAX_SEGS * FCX_MAX_RANKS), "cudaMalloc"));
    cudaMemset(c->segsDev, 0, sizeof(char *) * FCX_MAX_SEGS * FCX_MAX_RANKS);
    c->segs.resize(FCX_MAX_SEGS);

    FcxDevComm &d = c->dev;
    d.rank = rank;
    d.nranks = nranks;
    for (int r = 0; r < nranks; r++) d.heap[r] = c->heap.base[r];
    d.mcHeap = c->heap.mcBase;
    d.heapBytes = c->heap.bytes;
    d.stageBytes = stage;
    d.pipeBytes = (unsigned int)std::min<int64_t>(envInt("PIPE_BYTES", 16ll << 20), 1ll << 30);
    d.p2pOff = p2pOff;
    d.p2pChunkBytes = chunk;
    d.userOff = userOff;
    void *devErr = nullptr, *devAbort = nullptr;
    cudaHostGetDevicePointer(&devErr, c->errHost, 0);
    cudaHostGetDevicePointer(&devAbort, c->abortHost, 0);
    d.err = (FcxDevError *)devErr;
    d.abortWord = (volatile uint32_t *)devAbort;
    d.timeoutNs = (uint64_t)envInt("KERNEL_TIMEOUT_MS", 30000) * 1000000ull;
    d.segs = c->segsDev;
    c->arena.reset(userOff, c->heap.bytes - userOff);
    FCX_CHECK(cudaToResult(cudaDeviceSynchronize(), "device sync after heap set-up"));
    FCX_CHECK(c->bs.barrier());  // nobody launches before every control block is clear
    FCX_INFO(SUB_INIT, "comm %p rank %d/%d: heap %zu MiB (%s%s), stage 2x%zu MiB", (void *)c.get(), rank, nranks,
             c->heap.bytes >> 20, c->heap.vmm ? "vmm" : "ipc", c->heap.mcBase ? "+multicast" : "", stage >> 20);
  }

  FCX_CHECK(topoProbeAndDump(c.get()));

  TunerCaps caps;
  caps.nranks = nranks;
  caps.multicast = c->heap.mcBase != nullptr;
  caps.stageBytes = c->dev.stageBytes;
  caps.pipeBytes = c->dev.pipeBytes;
  caps.maxCtas = (int)std::min<int64_t>(envInt("MAX_CTAS", 128), FCX_MAX_CTAS);
  c->zcMcMode = (int)envInt("ZC_MC", 1);
  c->zcAgMcMode = (int)envInt("ZC_AG_MC", 1);
  c->tuner.reset(new Tuner(&c->bs, caps));
  // Measured table shipped with the library for this GPU model and world size (written by the tuning tool on
  // such a machine); FLAGCX_TUNER_CACHE replaces it, FLAGCX_TUNER_DEFAULTS=0 leaves the cost-model prior alone.
  if (!c->hostOnly && !c->hostFallback && envStr("TUNER_CACHE", "").empty() && envInt("TUNER_DEFAULTS", 1) != 0) {
    cudaDeviceProp prop;
    Dl_info info;
    if (cudaGetDeviceProperties(&prop, c->cudaDev) == cudaSuccess && dladdr((void *)&commCreate, &info) && info.dli_fname) {
      std::string dir = info.dli_fname;
      size_t slash = dir.rfind('/');
      dir = slash == std::string::npos ? "." : dir.substr(0, slash);
      std::string model;
      for (const char *q = prop.name; *q; q++)
        if (isalnum((unsigned char)*q)) model += (char)tolower((unsigned char)*q);
      std::string path = dir + "/tuned/" + model + "_" + std::to_string(nranks) + "gpu.json";
      if (access(path.c_str(), R_OK) == 0 && c->tuner->load(path) == flagcxSuccess)
        FCX_INFO(SUB_TUNING, "tuner: measured table %s", path.c_str());
    }
    cudaGetLastError();
  }
  flagcxComm *raw = c.release();
  *out = raw;
  { std::lock_guard<std::mutex> lk(gCommMu); gLive.insert(raw); }
  // FLAGCX_KERNEL_PROXY=1 (reference: flagcx/core/proxy.cc:1074-1182): start the thread that serves the
  // device->host request queue with the communicator instead of at the first flagcxCommFifoBuffer call.
  if (envInt("KERNEL_PROXY", 0) != 0 && !raw->hostOnly && raw->heap.bytes) {
    void *queue = nullptr;
    flagcxCommFifoBuffer(raw, &queue);
  }
  return flagcxSuccess;
}

// Unmap the heap and free what hangs off the communicator.
static void commRelease(flagcxComm *c) {
  if (!c->hostOnly && c->heap.bytes) {
    for (auto &s : c->segs)
      if (s.used)
        for (int r = 0; r < c->nranks; r++)
          if (r != c->rank && s.peer[r]) cudaIpcCloseMemHandle(s.peer[r]);
    c->heap.destroy();
    if (c->errHost) cudaFreeHost(c->errHost);
    if (c->segsDev) cudaFree(c->segsDev);
    cudaGetLastError();
  }
  delete c;
}

flagcxResult_t commFree(flagcxComm *c) {
  if (!c) return flagcxSuccess;
  {
    std::lock_guard<std::mutex> lk(gCommMu);
    if (!gLive.count(c)) return flagcxSuccess;  // already destroyed (a child freed with its parent, or twice)
  }
  while (!c->children.empty()) commFree(c->children.back());  // each child takes itself off the list
  if (c->parent) {
    auto &sib = c->parent->children;
    sib.erase(std::remove(sib.begin(), sib.end(), c), sib.end());
    c->parent = nullptr;
  }
  fifoStop(c);
  c2cDestroy(c);
  if (!c->hostOnly && c->heap.bytes) {
    cudaDeviceSynchronize();
    cudaGetLastError();
    std::string cache = envStr("TUNER_CACHE", "");
    if (!cache.empty() && c->rank == 0 && c->tuner) c->tuner->save(cache);
    if (logEnabled(LOG_INFO, SUB_COLL)) {
      for (int op = 0; op < flagcxNumCommOps; op++)
        if (c->counters.calls[op])
          FCX_INFO(SUB_COLL, "comm %p: op %d: %llu calls, %llu bytes", (void *)c, op, (unsigned long long)c->counters.calls[op],
                   (unsigned long long)c->counters.bytes[op]);
    }
    // Peers must stop touching this heap before it is unmapped.
    if (!c->abortFlag.load()) c->bs.barrier();
  }
  FCX_INFO(SUB_INIT, "communicator %p (rank %d of %d) destroyed", (void *)c, c->rank, c->nranks);
  c->bs.close();
  bool lent;
  {
    std::lock_guard<std::mutex> lk(gCommMu);
    gLive.erase(c);
    c->destroyed = true;
    lent = c->heapRefs.load() > 0;
    if (lent) gLent.insert(c);
  }
  if (lent) {
    FCX_INFO(SUB_ALLOC, "communicator %p: %d heap buffers are still held; the heap stays mapped until they are released", (void *)c,
             c->heapRefs.load());
    return flagcxSuccess;
  }
  commRelease(c);
  return flagcxSuccess;
}

// A holder of heap memory that may outlive the communicator (a tensor) takes a reference when it gets the
// memory and gives it back with the pointer.
flagcxResult_t commHeapRetain(flagcxComm *c) {
  std::lock_guard<std::mutex> lk(gCommMu);
  if (!gLive.count(c)) return flagcxInvalidArgument;
  c->heapRefs.fetch_add(1);
  return flagcxSuccess;
}

flagcxResult_t commHeapRelease(flagcxComm *c, void *ptr) {
  bool last = false, live = false;
  {
    std::lock_guard<std::mutex> lk(gCommMu);
    live = gLive.count(c) != 0;
    if (!live && !gLent.count(c)) return flagcxInvalidArgument;
    if (c->heapRefs.fetch_sub(1) == 1 && !live) { gLent.erase(c); last = true; }
  }
  if (live && ptr) {
    char *base = c->heap.base[c->rank];
    if ((char *)ptr >= base && (char *)ptr < base + c->heap.bytes) c->arena.free((char *)ptr - base);
  }
  if (last) commRelease(c);
  return flagcxSuccess;
}

}  // namespace fcx

using namespace fcx;

// ------------------------------------------------------------------ device handle table

namespace {

flagcxResult_t dhSync() { return cudaToResult(cudaDeviceSynchronize(), "deviceSynchronize"); }
flagcxResult_t dhMemcpy(void *dst, void *src, size_t size, flagcxMemcpyType_t type, flagcxStream_t stream) {
  cudaMemcpyKind k = type == flagcxMemcpyHostToDevice ? cudaMemcpyHostToDevice
                     : type == flagcxMemcpyDeviceToHost ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
  if (stream) return cudaToResult(cudaMemcpyAsync(dst, src, size, k, stream->base), "deviceMemcpy");
  return cudaToResult(cudaMemcpy(dst, src, size, k), "deviceMemcpy");
}
flagcxResult_t dhMemset(void *ptr, int value, size_t size, flagcxMemType_t type, flagcxStream_t stream) {
  if (type == flagcxMemHost) { memset(ptr, value, size); return flagcxSuccess; }
  if (stream) return cudaToResult(cudaMemsetAsync(ptr, value, size, stream->base), "deviceMemset");
  return cudaToResult(cudaMemset(ptr, value, size), "deviceMemset");
}
flagcxResult_t dhMalloc(void **ptr, size_t size, flagcxMemType_t type, flagcxStream_t stream) {
  if (type == flagcxMemHost) return cudaToResult(cudaHostAlloc(ptr, size, cudaHostAllocMapped), "deviceMalloc(host)");
  if (type == flagcxMemManaged) return cudaToResult(cudaMallocManaged(ptr, size), "deviceMalloc(managed)");
  if (stream) return cudaToResult(cudaMallocAsync(ptr, size, stream->base), "deviceMalloc(async)");
  return cudaToResult(cudaMalloc(ptr, size), "deviceMalloc");
}
flagcxResult_t dhFree(void *ptr, flagcxMemType_t type, flagcxStream_t stream) {
  if (type == flagcxMemHost) return cudaToResult(cudaFreeHost(ptr), "deviceFree(host)");
  if (stream && type == flagcxMemDevice) return cudaToResult(cudaFreeAsync(ptr, stream->base), "deviceFree(async)");
  return cudaToResult(cudaFree(ptr), "deviceFree");
}
flagcxResult_t dhSetDevice(int dev) { return cudaToResult(cudaSetDevice(dev), "setDevice"); }
flagcxResult_t dhGetDevice(int *dev) { return cudaToResult(cudaGetDevice(dev), "getDevice"); }
flagcxResult_t dhGetDeviceCount(int *n) {
  if (cudaGetDeviceCount(n) != cudaSuccess) { cudaGetLastError(); *n = 0; }
  return flagcxSuccess;
}
flagcxResult_t dhGetVendor(char *vendor) { strcpy(vendor, "NVIDIA"); return flagcxSuccess; }
flagcxResult_t dhHostGetDevicePointer(void **pDevice, void *pHost) {
  return cudaToResult(cudaHostGetDevicePointer(pDevice, pHost, 0), "hostGetDevicePointer");
}
flagcxResult_t dhStreamCreate(flagcxStream_t *s) {
  *s = new flagcxStream;
  return cudaToResult(cudaStreamCreateWithFlags(&(*s)->base, cudaStreamNonBlocking), "streamCreate");
}
flagcxResult_t dhStreamDestroy(flagcxStream_t s) {
  if (!s) return flagcxSuccess;
  cudaError_t e = cudaStreamDestroy(s->base);
  delete s;
  return cudaToResult(e, "streamDestroy");
}
flagcxResult_t dhStreamCopy(flagcxStream_t *out, void *old) {
  *out = new flagcxStream;
  (*out)->base = (cudaStream_t)old;  // the handle itself travels in the pointer, as in the reference's CUDA adaptor
  return flagcxSuccess;
}
flagcxResult_t dhStreamFree(flagcxStream_t s) { delete s; return flagcxSuccess; }
flagcxResult_t dhStreamSync(flagcxStream_t s) { return cudaToResult(cudaStreamSynchronize(s ? s->base : 0), "streamSynchronize"); }
flagcxResult_t dhStreamQuery(flagcxStream_t s) {
  cudaError_t e = cudaStreamQuery(s ? s->base : 0);
  if (e == cudaErrorNotReady) { cudaGetLastError(); return flagcxInProgress; }
  return cudaToResult(e, "streamQuery");
}
flagcxResult_t dhStreamWaitEvent(flagcxStream_t s, flagcxEvent_t e) {
  return cudaToResult(cudaStreamWaitEvent(s ? s->base : 0, e->base, 0), "streamWaitEvent");
}
flagcxResult_t dhEventCreate(flagcxEvent_t *e, flagcxEventType_t type) {
  *e = new flagcxEvent;
  return cudaToResult(cudaEventCreateWithFlags(&(*e)->base, type == flagcxEventDisableTiming ? cudaEventDisableTiming : cudaEventDefault),
                      "eventCreate");
}
flagcxResult_t dhEventDestroy(flagcxEvent_t e) {
  if (!e) return flagcxSuccess;
  cudaError_t r = cudaEventDestroy(e->base);
  delete e;
  return cudaToResult(r, "eventDestroy");
}
flagcxResult_t dhEventRecord(flagcxEvent_t e, flagcxStream_t s) { return cudaToResult(cudaEventRecord(e->base, s ? s->base : 0), "eventRecord"); }
flagcxResult_t dhEventSync(flagcxEvent_t e) { return cudaToResult(cudaEventSynchronize(e->base), "eventSynchronize"); }
flagcxResult_t dhEventQuery(flagcxEvent_t e) {
  cudaError_t r = cudaEventQuery(e->base);
  if (r == cudaErrorNotReady) { cudaGetLastError(); return flagcxInProgress; }
  return cudaToResult(r, "eventQuery");
}
flagcxResult_t dhIpcCreate(flagcxIpcMemHandle_t *h, size_t *size) {
  *h = new flagcxIpcMemHandle;
  if (size) *size = sizeof(cudaIpcMemHandle_t);
  return flagcxSuccess;
}
flagcxResult_t dhIpcGet(flagcxIpcMemHandle_t h, void *devPtr) { return cudaToResult(cudaIpcGetMemHandle(&h->base, devPtr), "ipcMemHandleGet"); }
flagcxResult_t dhIpcOpen(flagcxIpcMemHandle_t h, void **devPtr) {
  return cudaToResult(cudaIpcOpenMemHandle(devPtr, h->base, cudaIpcMemLazyEnablePeerAccess), "ipcMemHandleOpen");
}
flagcxResult_t dhIpcClose(void *devPtr) { return cudaToResult(cudaIpcCloseMemHandle(devPtr), "ipcMemHandleClose"); }
flagcxResult_t dhIpcFree(flagcxIpcMemHandle_t h) { delete h; return flagcxSuccess; }

flagcxDeviceHandle gDevHandle = {
    dhSync, dhMemcpy, dhMemset, dhMalloc, dhFree, dhSetDevice, dhGetDevice, dhGetDeviceCount, dhGetVendor,
    dhHostGetDevicePointer, dhStreamCreate, dhStreamDestroy, dhStreamCopy, dhStreamFree, dhStreamSync, dhStreamQuery,
    dhStreamWaitEvent, dhEventCreate, dhEventDestroy, dhEventRecord, dhEventSync, dhEventQuery, dhIpcCreate, dhIpcGet,
    dhIpcOpen, dhIpcClose, dhIpcFree};

}  // namespace

// ------------------------------------------------------------------ public API

extern "C" {

size_t getFlagcxDataTypeSize(flagcxDataType_t dtype) { return dtypeSize(dtype); }

flagcxResult_t flagcxHandleInit(flagcxHandlerGroup_t *handler) {
  if (!handler) return flagcxInvalidArgument;
  flagcxHandlerGroup *h = (flagcxHandlerGroup *)calloc(1, sizeof *h);
  h->uniqueId = (flagcxUniqueId_t)calloc(1, sizeof(flagcxUniqueId));
  h->comm = nullptr;
  h->devHandle = (flagcxDeviceHandle_t)malloc(sizeof(flagcxDeviceHandle));
  *h->devHandle = gDevHandle;
  *handler = h;
  return flagcxSuccess;
}

flagcxResult_t flagcxHandleFree(flagcxHandlerGroup_t handler) {
  if (!handler) return flagcxSuccess;
  free(handler->uniqueId);
  free(handler->devHandle);
  free(handler);
  return flagcxSuccess;
}

flagcxResult_t flagcxGetVersion(int *version) {
  if (!version) return flagcxInvalidArgument;
  *version = 1 * 10000 + 0 * 100 + 0;
  return flagcxSuccess;
}

flagcxResult_t flagcxGetUniqueId(flagcxUniqueId_t *uniqueId) {
  if (!uniqueId) return flagcxInvalidArgument;
  if (!*uniqueId) *uniqueId = (flagcxUniqueId_t)calloc(1, sizeof(flagcxUniqueId));
  memset((*uniqueId)->internal, 0, FLAGCX_UNIQUE_ID_BYTES);
  BootstrapHandle h;
  FCX_CHECK(Bootstrap::createId(&h));
  memcpy((*uniqueId)->internal, &h, sizeof h);
  return flagcxSuccess;
}

flagcxResult_t flagcxCommInitRank(flagcxComm_t *comm, int nranks, flagcxUniqueId_t commId, int rank) {
  if (!comm || !commId) return flagcxInvalidArgument;
  BootstrapHandle h;
  memcpy(&h, commId->internal, sizeof h);
  flagcxComm *c = nullptr;
  FCX_CHECK(commCreate(&c, nranks, h, rank, 1.0, 0));
  *comm = c;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommInitRankEx(flagcxComm_t *comm, int nranks, flagcxUniqueId_t commId, int rank, unsigned flags) {
  if (!comm || !commId) return flagcxInvalidArgument;
  BootstrapHandle h;
  memcpy(&h, commId->internal, sizeof h);
  flagcxComm *c = nullptr;
  FCX_CHECK(commCreate(&c, nranks, h, rank, 1.0, flags));
  *comm = c;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommFinalize(flagcxComm_t comm) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  if (!comm->hostOnly) FCX_CHECK(cudaToResult(cudaDeviceSynchronize(), "finalize"));
  return flagcxSuccess;
}

flagcxResult_t flagcxCommDestroy(flagcxComm_t comm) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  return commFree(comm);
}

flagcxResult_t flagcxCommAbort(flagcxComm_t comm) {
  // Ask every waiter (host sockets and device kernels) to leave, then free.
  if (!validComm(comm)) return flagcxInvalidArgument;
  comm->abortFlag.store(1);
  if (comm->abortHost) {
    *(volatile uint32_t *)comm->abortHost = 1;
    cudaDeviceSynchronize();
    cudaGetLastError();
  }
  return commFree(comm);
}

// Suspend/Resume: the reference declares them and every NVIDIA path answers
// "unsupported" (flagcx/adaptor/ccl/nccl_adaptor.cc:46-52).  Here Suspend
// drains the device and Resume clears a recorded device error.
flagcxResult_t flagcxCommSuspend(flagcxComm_t comm) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  if (!comm->hostOnly) FCX_CHECK(cudaToResult(cudaDeviceSynchronize(), "suspend"));
  return flagcxSuccess;
}
flagcxResult_t flagcxCommResume(flagcxComm_t comm) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  return flagcxCommClearError(comm);
}

const char *flagcxGetErrorString(flagcxResult_t result) {
  switch (result) {
    case flagcxSuccess: return "no error";
    case flagcxUnhandledDeviceError: return "unhandled device (CUDA) error";
    case flagcxSystemError: return "unhandled system error";
    case flagcxInternalError: return "internal error";
    case flagcxInvalidArgument: return "invalid argument";
    case flagcxInvalidUsage: return "invalid usage";
    case flagcxRemoteError: return "remote process exited, timed out or there was a network error";
    case flagcxInProgress: return "operation in progress";
    case flagcxUnhandledCCLError: return "unhandled collective library error";
    case flagcxNotSupported: return "operation not supported";
    default: return "unknown result code";
  }
}

const char *flagcxGetLastError(flagcxComm_t) { return lastErrorText(); }

flagcxResult_t flagcxCommGetAsyncError(flagcxComm_t comm, flagcxResult_t *asyncError) {
  if (!validComm(comm) || !asyncError) return flagcxInvalidArgument;
  *asyncError = flagcxSuccess;
  if (comm->errHost && *(volatile uint32_t *)&comm->errHost->code != 0) *asyncError = flagcxRemoteError;
  if (comm->abortFlag.load()) *asyncError = flagcxRemoteError;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommCount(const flagcxComm_t comm, int *count) {
  if (!validComm(comm) || !count) return flagcxInvalidArgument;
  *count = comm->nranks;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommGetDeviceNumber(const flagcxComm_t comm, int *device) {
  if (!validComm(comm) || !device) return flagcxInvalidArgument;
  *device = comm->cudaDev;
  return flagcxSuccess;
}
flagcxResult_t flagcxCommUserRank(const flagcxComm_t comm, int *rank) {
  if (!validComm(comm) || !rank) return flagcxInvalidArgument;
  *rank = comm->rank;
  return flagcxSuccess;
}
flagcxResult_t flagcxIsHomoComm(flagcxComm_t comm, int *isHomo) {
  if (!validComm(comm) || !isHomo) return flagcxInvalidArgument;
  *isHomo = comm->nclusters == 1;
  return flagcxSuccess;
}

// ---- memory

flagcxResult_t flagcxMemAlloc(void **ptr, size_t size, flagcxComm_t comm) {
  if (!ptr) return flagcxInvalidArgument;
  if (comm && validComm(comm) && !comm->hostOnly && comm->heap.bytes) {
    size_t off = comm->arena.alloc(size);
    if (off == ~(size_t)0) {
      FCX_WARN("flagcxMemAlloc: the symmetric heap has no room for %zu bytes (%zu free); raise FLAGCX_HEAP_USER_BYTES", size,
               comm->arena.bytesFree());
      return flagcxSystemError;
    }
    *ptr = comm->heap.base[comm->rank] + off;
    return flagcxSuccess;
  }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    *ptr = malloc(size);
    return *ptr ? flagcxSuccess : flagcxSystemError;
  }
  return cudaToResult(cudaMalloc(ptr, size), "flagcxMemAlloc");
}

flagcxResult_t flagcxMemFree(void *ptr, flagcxComm_t comm) {
  if (!ptr) return flagcxSuccess;
  if (comm && validComm(comm) && comm->heap.bytes) {
    char *base = comm->heap.base[comm->rank];
    if ((char *)ptr >= base && (char *)ptr < base + comm->heap.bytes)
      return comm->arena.free((char *)ptr - base) ? flagcxSuccess : flagcxInvalidArgument;
  }
  int ndev = 0;
  if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    free(ptr);
    return flagcxSuccess;
  }
  return cudaToResult(cudaFree(ptr), "flagcxMemFree");
}

// Registration is collective: every rank registers its n-th buffer with its
// n-th call.  Buffers inside the heap need nothing.  Others are exported with
// CUDA IPC; `buff` must be the start of its allocation.
flagcxResult_t flagcxCommRegister(const flagcxComm_t comm, void *buff, size_t size, void **handle) {
  if (!validComm(comm) || !buff || !handle) return flagcxInvalidArgument;
  if (comm->hostOnly || !comm->heap.bytes) { *handle = buff; return flagcxSuccess; }
  char *base = comm->heap.base[comm->rank];
  std::vector<int> inHeap(comm->nranks, 0);
  inHeap[comm->rank] = ((char *)buff >= base && (char *)buff + size <= base + comm->heap.bytes) ? 1 : 0;
  FCX_CHECK(comm->bs.allGather(inHeap.data(), sizeof(int)));
  bool all = true;
  for (int x : inHeap) all = all && x;
  if (all) { *handle = buff; return flagcxSuccess; }
  int slot = -1;
  for (int i = 1; i < FCX_MAX_SEGS; i++)
    if (!comm->segs[i].used) { slot = i; break; }
  if (slot < 0) return flagcxInternalError;
  std::vector<cudaIpcMemHandle_t> hs(comm->nranks);
  std::vector<int> ok(comm->nranks, 0);
  ok[comm->rank] = cudaIpcGetMemHandle(&hs[comm->rank], buff) == cudaSuccess;
  cudaGetLastError();
  FCX_CHECK(comm->bs.allGather(hs.data(), sizeof(cudaIpcMemHandle_t)));
  FCX_CHECK(comm->bs.allGather(ok.data(), sizeof(int)));
  for (int x : ok)
    if (!x) {
      FCX_WARN("flagcxCommRegister: a rank could not export its buffer (is it the start of a cudaMalloc allocation?)");
      return flagcxInvalidArgument;
    }
  Segment &s = comm->segs[slot];
  s = Segment();
  s.localBase = (char *)buff;
  s.bytes = size;
  for (int r = 0; r < comm->nranks; r++) {
    if (r == comm->rank) { s.peer[r] = (char *)buff; continue; }
    void *q = nullptr;
    if (cudaIpcOpenMemHandle(&q, hs[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
      cudaGetLastError();
      return flagcxUnhandledDeviceError;
    }
    s.peer[r] = (char *)q;
  }
  s.used = true;
  FCX_CHECK(cudaToResult(cudaMemcpy(&comm->segsDev[slot], s.peer, sizeof s.peer, cudaMemcpyHostToDevice), "segment table"));
  *handle = &s;
  FCX_INFO(SUB_REG, "registered %p (%zu bytes) as segment %d", buff, size, slot);
  return flagcxSuccess;
}

flagcxResult_t flagcxCommDeregister(const flagcxComm_t comm, void *handle) {
  if (!validComm(comm) || !handle) return flagcxInvalidArgument;
  for (auto &s : comm->segs)
    if (&s == handle && s.used) {
      cudaDeviceSynchronize();
      comm->bs.barrier();
      for (int r = 0; r < comm->nranks; r++)
        if (r != comm->rank && s.peer[r]) cudaIpcCloseMemHandle(s.peer[r]);
      cudaGetLastError();
      s = Segment();
      return flagcxSuccess;
    }
  return flagcxSuccess;  // heap buffers and host buffers carry no state
}

// ---- extensions

flagcxResult_t flagcxTopoNvlinkCount(const char *busId, int *activeLinks, int *version) {
  if (!busId || !activeLinks || !version) return flagcxInvalidArgument;
  return topoNvlinkCount(busId, activeLinks, version) ? flagcxSuccess : flagcxNotSupported;
}
flagcxResult_t flagcxCommGetNetOfRank(flagcxComm_t comm, int rank, char *out, size_t outBytes) {
  if (!validComm(comm) || !out || !outBytes || rank < 0 || rank >= comm->nranks) return flagcxInvalidArgument;
  snprintf(out, outBytes, "%s", rank < (int)comm->netOfRank.size() ? comm->netOfRank[rank].c_str() : "");
  return flagcxSuccess;
}

flagcxResult_t flagcxCommSetZeroCopyMulticast(flagcxComm_t comm, int mode) {
  if (!validComm(comm) || mode < 0 || mode > 2) return flagcxInvalidArgument;
  comm->zcMcMode = comm->zcAgMcMode = mode;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommHeapRetain(flagcxComm_t comm) { return commHeapRetain(comm); }
flagcxResult_t flagcxCommHeapRelease(flagcxComm_t comm, void *ptr) { return commHeapRelease(comm, ptr); }

flagcxResult_t flagcxCommGetCounters(flagcxComm_t comm, flagcxCommCounters *out) {
  if (!validComm(comm) || !out) return flagcxInvalidArgument;
  *out = comm->counters;
  if (comm->errHost && comm->errHost->code == FCX_ERR_TIMEOUT) out->timeouts = 1;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommGetClusterInfo(flagcxComm_t comm, int *nclusters, int *myCluster, int *clusterOfRank) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  if (nclusters) *nclusters = comm->nclusters;
  if (myCluster) *myCluster = comm->myCluster;
  if (clusterOfRank) memcpy(clusterOfRank, comm->clusterOf.data(), comm->nranks * sizeof(int));
  return flagcxSuccess;
}

flagcxResult_t flagcxCommHeapInfo(flagcxComm_t comm, void **peerBases, void **mcBase, size_t *heapBytes) {
  if (!validComm(comm) || !comm->heap.bytes) return flagcxInvalidArgument;
  if (peerBases) for (int r = 0; r < comm->nranks; r++) peerBases[r] = comm->heap.base[r];
  if (mcBase) *mcBase = comm->heap.mcBase;
  if (heapBytes) *heapBytes = comm->heap.bytes;
  return flagcxSuccess;
}

flagcxResult_t flagcxHeapOffset(flagcxComm_t comm, const void *ptr, size_t *offset) {
  if (!validComm(comm) || !comm->heap.bytes || !offset) return flagcxInvalidArgument;
  const char *base = comm->heap.base[comm->rank];
  if ((const char *)ptr < base || (const char *)ptr >= base + comm->heap.bytes) return flagcxInvalidArgument;
  *offset = (const char *)ptr - base;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommDeviceDescriptor(flagcxComm_t comm, void *out, size_t outBytes) {
  if (!validComm(comm) || !out || outBytes < sizeof(FcxDevComm) || !comm->heap.bytes) return flagcxInvalidArgument;
  memcpy(out, &comm->dev, sizeof(FcxDevComm));
  return flagcxSuccess;
}

flagcxResult_t flagcxCommAllocSignals(flagcxComm_t comm, int n, int *first) {
  if (!validComm(comm) || !first || n < 1) return flagcxInvalidArgument;
  std::lock_guard<std::mutex> lk(comm->mu);
  if (comm->nextSignal + n > FCX_DEVAPI_SIGNALS - 16) return flagcxInternalError;
  *first = comm->nextSignal;
  comm->nextSignal += n;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommSetTimeoutMs(flagcxComm_t comm, int ms) {
  if (!validComm(comm) || ms < 1) return flagcxInvalidArgument;
  comm->dev.timeoutNs = (uint64_t)ms * 1000000ull;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommGetDeviceError(flagcxComm_t comm, int *code, int *peer, int *where, unsigned long long *expected,
                                        unsigned long long *seen) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  FcxDevError e{};
  if (comm->errHost) memcpy(&e, comm->errHost, sizeof e);
  if (code) *code = e.code;
  if (peer) *peer = e.peer;
  if (where) *where = e.where;
  if (expected) *expected = e.expected;
  if (seen) *seen = e.seen;
  return flagcxSuccess;
}

flagcxResult_t flagcxCommClearError(flagcxComm_t comm) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  if (comm->errHost) {
    FCX_CHECK(cudaToResult(cudaDeviceSynchronize(), "clear error"));
    memset(comm->errHost, 0, sizeof(FcxDevError));
    // errClaim and abortSeen live at the start of the local block
    FCX_CHECK(cudaToResult(cudaMemset(comm->heap.base[comm->rank] + FCX_OFF_LOCAL, 0, 16), "clear error"));
  }
  return flagcxSuccess;
}

// Collective re-synchronisation after a collective gave up on some rank.  The ranks may disagree on how many
// collectives completed (a rank that left in its prologue did not count the call, one that left later did),
// and every wait is a ">=" on values built from that count, so carrying on would let the rank that is behind
// pass barriers on flags left by its peers' newer calls.  All ranks therefore agree on a sequence number
// above anything used so far, rewrite their counters to it and clear the control words behind host barriers.
flagcxResult_t flagcxCommRecover(flagcxComm_t comm) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  if (comm->hostOnly || !comm->heap.bytes) return flagcxSuccess;
  FCX_CHECK(cudaToResult(cudaDeviceSynchronize(), "recover"));
  char *base = comm->heap.base[comm->rank];
  // FcxLocal: {ctaDone, errClaim, abortSeen, pad, seq, opCount[][]}
  unsigned long long seq = 0;
  FCX_CHECK(cudaToResult(cudaMemcpy(&seq, base + FCX_OFF_LOCAL + 16, sizeof seq, cudaMemcpyDeviceToHost), "recover: read seq"));
  std::vector<unsigned long long> all(comm->nranks, 0);
  all[comm->rank] = seq;
  FCX_CHECK(comm->bs.allGather(all.data(), sizeof(unsigned long long)));  // also a barrier: every rank's device is idle
  unsigned long long next = 0;
  for (auto v : all) next = std::max(next, v);
  next += 2;
  // nobody launches before everybody has reset, and nobody resets while somebody could still be running
  FCX_CHECK(cudaToResult(cudaMemset(base + FCX_OFF_FLAGS, 0, FCX_OFF_DONE - FCX_OFF_FLAGS), "recover: flags"));
  std::vector<unsigned long long> done(FCX_MAX_RANKS, next);
  FCX_CHECK(cudaToResult(cudaMemcpy(base + FCX_OFF_DONE, done.data(), sizeof(unsigned long long) * FCX_MAX_RANKS, cudaMemcpyHostToDevice),
                         "recover: done words"));
  FCX_CHECK(cudaToResult(cudaMemset(base + FCX_OFF_MAIL, 0, FCX_OFF_P2P - FCX_OFF_MAIL), "recover: mailboxes"));
  FCX_CHECK(cudaToResult(cudaMemset(base + FCX_OFF_P2P, 0, FCX_OFF_LOCAL - FCX_OFF_P2P), "recover: p2p control"));
  FCX_CHECK(cudaToResult(cudaMemset(base + FCX_OFF_LOCAL, 0, FCX_OFF_DEVAPI - FCX_OFF_LOCAL), "recover: local words"));
  FCX_CHECK(cudaToResult(cudaMemcpy(base + FCX_OFF_LOCAL + 16, &next, sizeof next, cudaMemcpyHostToDevice), "recover: seq"));
  FCX_CHECK(cudaToResult(cudaMemset(base + FCX_OFF_LL, 0, 2 * (size_t)FCX_MAX_RANKS * FCX_LL_SLOT_BYTES), "recover: LL lines"));
  memset(comm->sendChunks, 0, sizeof comm->sendChunks);
  memset(comm->recvChunks, 0, sizeof comm->recvChunks);
  comm->seq = next;
  if (comm->errHost) memset(comm->errHost, 0, sizeof(FcxDevError));
  FCX_CHECK(cudaToResult(cudaDeviceSynchronize(), "recover"));
  FCX_CHECK(comm->bs.barrier());
  FCX_INFO(SUB_INIT, "communicator %p re-synchronised at sequence %llu", (void *)comm, next);
  return flagcxSuccess;
}

flagcxResult_t flagcxTunerRecord(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, const char *kind, int nctas, double us) {
  if (!validComm(comm) || !kind) return flagcxInvalidArgument;
  int k = kindFromName(kind);
  if (k < 0) return flagcxInvalidArgument;
  comm->tuner->record(op, bytes, Plan{k, nctas}, us);
  return flagcxSuccess;
}
flagcxResult_t flagcxTunerSave(flagcxComm_t comm, const char *path) {
  if (!validComm(comm) || !path) return flagcxInvalidArgument;
  return comm->tuner->save(path);
}
flagcxResult_t flagcxTunerLoad(flagcxComm_t comm, const char *path) {
  if (!validComm(comm) || !path) return flagcxInvalidArgument;
  return comm->tuner->load(path);
}

}  // extern "C"
