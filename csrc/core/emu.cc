// Single-GPU emulation of a multi-rank communicator (flagcx_ext.h,
// flagcxEmu*).  Every emulated rank gets its own "heap" on the one device and
// all ranks run inside one cooperative launch, so the very kernels that move
// data between GPUs can be checked for protocol errors (flags, parities, unit
// ownership, chunk counters) on a machine with a single GPU.  Kernels that
// wait on one another are never issued as separate launches on one GPU.
#include "comm.h"
#include "hosttypes.h"
#include "log.h"
#include "../kernels/launch.h"

#include <cstring>
#include <cuda_runtime.h>

using namespace fcx;

struct flagcxEmu {
  int n = 0;
  size_t stageBytes = 0, chunk = 0, heapBytes = 0;
  char *heaps[FCX_MAX_RANKS] = {};
  FcxDevComm host[FCX_MAX_RANKS];
  FcxDevComm *dcsDev = nullptr;
  FcxCollArgs *argsDev = nullptr;
  FcxP2pArgs *p2pDev = nullptr;
  FcxDevError *errHost = nullptr;
  uint64_t seq = 0;
  uint64_t sendChunks[FCX_MAX_RANKS][FCX_MAX_RANKS] = {}, recvChunks[FCX_MAX_RANKS][FCX_MAX_RANKS] = {};
};

extern "C" {

flagcxResult_t flagcxEmuCreate(flagcxEmu_t *out, int nranks, size_t stageBytes) {
  if (!out || nranks < 1 || nranks > FCX_MAX_RANKS) return flagcxInvalidArgument;
  flagcxEmu *e = new flagcxEmu;
  e->n = nranks;
  e->stageBytes = (stageBytes + 4095) & ~(size_t)4095;
  e->chunk = 64 << 10;
  size_t p2pOff = FCX_OFF_STAGE + 2 * e->stageBytes;
  e->heapBytes = p2pOff + (size_t)FCX_MAX_RANKS * 2 * e->chunk;
  FCX_CHECK(cudaToResult(cudaHostAlloc((void **)&e->errHost, 4096 * FCX_MAX_RANKS, cudaHostAllocMapped), "emu host alloc"));
  memset(e->errHost, 0, 4096 * FCX_MAX_RANKS);
  for (int r = 0; r < nranks; r++) {
    FCX_CHECK(cudaToResult(cudaMalloc((void **)&e->heaps[r], e->heapBytes), "emu heap"));
    FCX_CHECK(cudaToResult(cudaMemset(e->heaps[r], 0, FCX_OFF_STAGE), "emu heap clear"));
  }
  for (int r = 0; r < nranks; r++) {
    FcxDevComm &d = e->host[r];
    memset(&d, 0, sizeof d);
    d.rank = r;
    d.nranks = nranks;
    for (int p = 0; p < nranks; p++) d.heap[p] = e->heaps[p];
    d.mcHeap = nullptr;
    d.heapBytes = e->heapBytes;
    d.stageBytes = e->stageBytes;
    d.pipeBytes = (unsigned int)std::min<int64_t>(envInt("PIPE_BYTES", 16ll << 20), 1ll << 30);
    d.p2pOff = p2pOff;
    d.p2pChunkBytes = e->chunk;
    d.userOff = e->heapBytes;
    void *dp = nullptr;
    cudaHostGetDevicePointer(&dp, (char *)e->errHost + 4096 * r, 0);
    d.err = (FcxDevError *)dp;
    d.abortWord = (volatile uint32_t *)((char *)dp + 2048);
    d.timeoutNs = (uint64_t)envInt("KERNEL_TIMEOUT_MS", 5000) * 1000000ull;
    d.segs = nullptr;
  }
  FCX_CHECK(cudaToResult(cudaMalloc((void **)&e->dcsDev, sizeof(FcxDevComm) * FCX_MAX_RANKS), "emu alloc"));
  FCX_CHECK(cudaToResult(cudaMalloc((void **)&e->argsDev, sizeof(FcxCollArgs) * FCX_MAX_RANKS), "emu alloc"));
  FCX_CHECK(cudaToResult(cudaMalloc((void **)&e->p2pDev, sizeof(FcxP2pArgs) * FCX_MAX_RANKS), "emu alloc"));
  FCX_CHECK(cudaToResult(cudaMemcpy(e->dcsDev, e->host, sizeof(FcxDevComm) * FCX_MAX_RANKS, cudaMemcpyHostToDevice), "emu copy"));
  *out = e;
  return flagcxSuccess;
}

flagcxResult_t flagcxEmuDestroy(flagcxEmu_t e) {
  if (!e) return flagcxSuccess;
  cudaDeviceSynchronize();
  for (int r = 0; r < e->n; r++) cudaFree(e->heaps[r]);
  cudaFree(e->dcsDev);
  cudaFree(e->argsDev);
  cudaFree(e->p2pDev);
  cudaFreeHost(e->errHost);
  cudaGetLastError();
  delete e;
  return flagcxSuccess;
}

flagcxResult_t flagcxEmuCollective(flagcxEmu_t e, flagcxCommOp_t op, const char *kind, int nctas, void *const *send,
                                   void *const *recv, size_t count, flagcxDataType_t dt, flagcxDataType_t outDt, float scale,
                                   flagcxRedOp_t red, int root, const size_t *tables, void *cudaStream) {
  if (!e || !kind) return flagcxInvalidArgument;
  int k = kindFromName(kind);
  if (k < 0) return flagcxInvalidArgument;
  if (k == FCX_K_AR_NVLS || k == FCX_K_RS_NVLS || k == FCX_K_AG_NVLS) return flagcxNotSupported;  // needs a real switch
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (nctas < 1 || nctas * e->n > sms) {
    FCX_WARN("emulation needs all %d x %d CTAs resident at once (%d SMs)", e->n, nctas, sms);
    return flagcxInvalidArgument;
  }
  const int n = e->n;
  const size_t es = dtypeSize(dt);
  FcxCollArgs as[FCX_MAX_RANKS];
  memset(as, 0, sizeof as);
  uint64_t seq = ++e->seq;
  for (int r = 0; r < n; r++) {
    FcxCollArgs &a = as[r];
    a.kind = k;
    a.dtype = dt;
    a.outDtype = outDt;
    a.redop = red;
    a.root = root;
    a.elemSize = (int)es;
    a.scale = scale;
    a.seq = seq;
    a.send = send ? send[r] : nullptr;
    a.recv = recv ? recv[r] : nullptr;
    a.count = count;
    a.sendHeapOff = a.recvHeapOff = ~0ull;
    a.sendSeg = a.recvSeg = FCX_SEG_NONE;
    if (k == FCX_K_AR_ZC || k == FCX_K_RS_ZC || k == FCX_K_REDUCE_ZC || k == FCX_K_MOVE_ZC) {
      // one device holds every emulated rank's buffers, so a buffer's address is valid for all of them
      a.sendSeg = a.send ? FCX_SEG_ABS : FCX_SEG_NONE;
      a.sendHeapOff = (uint64_t)(uintptr_t)a.send;
      a.recvSeg = a.recv ? FCX_SEG_ABS : FCX_SEG_NONE;
      a.recvHeapOff = (uint64_t)(uintptr_t)a.recv;
    }
    a.moveOp = op == flagcxCommOpAllGather ? FCX_K_AG : op == flagcxCommOpBroadcast ? FCX_K_BCAST : op == flagcxCommOpGather ? FCX_K_GATHER
               : op == flagcxCommOpScatter ? FCX_K_SCATTER : op == flagcxCommOpAlltoAll ? FCX_K_A2A : op == flagcxCommOpAlltoAllv ? FCX_K_A2AV : 0;
    switch (op) {
      case flagcxCommOpAllGather: case flagcxCommOpGather: a.recvStride = count; break;
      case flagcxCommOpReduceScatter: case flagcxCommOpScatter: a.sendStride = count; break;
      case flagcxCommOpAlltoAll: a.sendStride = a.recvStride = count; break;
      case flagcxCommOpAlltoAllv:
        if (!tables) return flagcxInvalidArgument;
        for (int i = 0; i < n; i++) {
          a.scounts[i] = tables[((size_t)r * 4 + 0) * n + i];
          a.sdispls[i] = tables[((size_t)r * 4 + 1) * n + i];
          a.rcounts[i] = tables[((size_t)r * 4 + 2) * n + i];
          a.rdispls[i] = tables[((size_t)r * 4 + 3) * n + i];
        }
        break;
      default: break;
    }
  }
  cudaStream_t st = (cudaStream_t)cudaStream;
  FCX_CHECK(cudaToResult(cudaMemcpyAsync(e->argsDev, as, sizeof(FcxCollArgs) * n, cudaMemcpyHostToDevice, st), "emu args"));
  return cudaToResult(fcxLaunchCollEmu(e->dcsDev, e->argsDev, &as[0], n, nctas, st), "emu launch");
}

flagcxResult_t flagcxEmuSendRecv(flagcxEmu_t e, int nops, const int *srcRank, const int *dstRank, void *const *sendbuf,
                                 void *const *recvbuf, const size_t *bytes, int ctasPerOp, void *cudaStream) {
  if (!e || nops < 1) return flagcxInvalidArgument;
  const int n = e->n;
  std::vector<FcxP2pArgs> gs(n);
  memset(gs.data(), 0, sizeof(FcxP2pArgs) * n);
  int maxOps = 0;
  for (int i = 0; i < nops; i++) {
    int s = srcRank[i], d = dstRank[i];
    if (s < 0 || s >= n || d < 0 || d >= n) return flagcxInvalidArgument;
    uint64_t nch = bytes[i] ? (bytes[i] + e->chunk - 1) / e->chunk : 1;
    if (s == d) {
      FcxP2pOp o{};
      o.isRecv = 2;
      o.peer = s;
      o.buf = recvbuf[i];
      o.bytes = bytes[i];
      o.heapOff = (uint64_t)(uintptr_t)sendbuf[i];
      if (gs[s].nops >= FCX_MAX_GROUP_OPS) return flagcxInvalidArgument;
      gs[s].ops[gs[s].nops++] = o;
    } else {
      FcxP2pOp so{}, ro{};
      so.isRecv = 0; so.peer = d; so.buf = sendbuf[i]; so.bytes = bytes[i]; so.heapOff = ~0ull; so.seg = FCX_SEG_NONE;
      if (envInt("EMU_P2P_ZEROCOPY", 0) != 0 && bytes[i]) {  // the receiver reads the sender's buffer where it lies
        so.seg = FCX_SEG_ABS;
        so.heapOff = (uint64_t)(uintptr_t)sendbuf[i];
      }
      so.firstChunk = e->sendChunks[s][d];
      e->sendChunks[s][d] += nch;
      ro.isRecv = 1; ro.peer = s; ro.buf = recvbuf[i]; ro.bytes = bytes[i]; ro.heapOff = ~0ull;
      ro.firstChunk = e->recvChunks[d][s];
      e->recvChunks[d][s] += nch;
      if (gs[s].nops >= FCX_MAX_GROUP_OPS || gs[d].nops >= FCX_MAX_GROUP_OPS) return flagcxInvalidArgument;
      gs[s].ops[gs[s].nops++] = so;
      gs[d].ops[gs[d].nops++] = ro;
    }
  }
  for (int r = 0; r < n; r++) {
    gs[r].ctasPerOp = ctasPerOp;
    maxOps = std::max(maxOps, gs[r].nops);
  }
  int ctasPerRank = maxOps * ctasPerOp;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (ctasPerRank * n > sms) return flagcxInvalidArgument;
  cudaStream_t st = (cudaStream_t)cudaStream;
  FCX_CHECK(cudaToResult(cudaMemcpyAsync(e->p2pDev, gs.data(), sizeof(FcxP2pArgs) * n, cudaMemcpyHostToDevice, st), "emu args"));
  FCX_CHECK(cudaToResult(cudaStreamSynchronize(st), "emu args"));  // gs is a local
  return cudaToResult(fcxLaunchP2pEmu(e->dcsDev, e->p2pDev, n, ctasPerRank, st), "emu launch");
}

flagcxResult_t flagcxEmuGetError(flagcxEmu_t e, int *code) {
  if (!e || !code) return flagcxInvalidArgument;
  *code = 0;
  for (int r = 0; r < e->n; r++) {
    const volatile FcxDevError *er = (const volatile FcxDevError *)((char *)e->errHost + 4096 * r);
    if (er->code) *code = er->code;
  }
  return flagcxSuccess;
}

}  // extern "C"
