// Public collective entry points, group semantics, and the launch logic that
// turns one API call into kernel launches on the caller's stream.
//
// Each call takes one of four routes (the reference has the same four-way
// split, flagcx/flagcx.cc:699-1848, but its "device" route is a call into the
// vendor library):
//   host     - communicator without a GPU, or FLAGCX_USE_HOST_COMM=1: TCP ring
//              algorithms on host memory (hostcoll.cc);
//   grouped  - between flagcxGroupStart/End: queued, then send/recv are fused
//              into one kernel launch and collectives are issued in order;
//   hybrid   - more than one cluster: the C2C planner (c2c/planner.cc);
//   direct   - a kernel of collectives.cu, variant picked by the tuner.
#include <nvtx3/nvToolsExt.h>
#include "comm.h"
#include "hostcoll.h"
#include "hosttypes.h"
#include "log.h"
#include "../kernels/launch.h"

#include <algorithm>
#include <cstring>
#include <cuda_runtime.h>

namespace fcx {

flagcxResult_t c2cExecute(flagcxComm *c, const PendingOp &op, bool *handled);  // c2c/planner.cc

static thread_local int tGroupDepth = 0;
static thread_local std::vector<flagcxComm *> tGroupComms;
int groupDepth() { return tGroupDepth; }
static thread_local int tInternalDepth = 0;
InternalCallScope::InternalCallScope() { tInternalDepth++; }
InternalCallScope::~InternalCallScope() { tInternalDepth--; }

static cudaStream_t streamOf(flagcxStream_t s) { return s ? s->base : (cudaStream_t)0; }

static void count(flagcxComm *c, flagcxCommOp_t op, size_t bytes) {
  c->counters.calls[op]++;
  c->counters.bytes[op] += bytes;
}

// ------------------------------------------------------------------ host route

flagcxResult_t hostCollective(flagcxComm *c, const PendingOp &o) {
  const int n = c->nranks;
  const size_t es = dtypeSize(o.dt);
  const void *send = o.send;
  void *recv = o.recv;
  std::vector<char> hs, hr;
  size_t sendBytes = 0, recvBytes = 0;
  const size_t *t = o.tables.data();
  switch (o.op) {
    case flagcxCommOpAllReduce: case flagcxCommOpBroadcast: case flagcxCommOpReduce: sendBytes = recvBytes = o.count * es; break;
    case flagcxCommOpAllGather: sendBytes = o.count * es; recvBytes = n * o.count * es; break;
    case flagcxCommOpReduceScatter: sendBytes = n * o.count * es; recvBytes = o.count * es; break;
    case flagcxCommOpGather: sendBytes = o.count * es; recvBytes = c->rank == o.root ? n * o.count * es : 0; break;
    case flagcxCommOpScatter: sendBytes = c->rank == o.root ? n * o.count * es : 0; recvBytes = o.count * es; break;
    case flagcxCommOpAlltoAll: sendBytes = recvBytes = n * o.count * es; break;
    case flagcxCommOpAlltoAllv:
      for (int i = 0; i < n; i++) {
        sendBytes = std::max(sendBytes, (t[n + i] + t[i]) * es);
        recvBytes = std::max(recvBytes, (t[3 * n + i] + t[2 * n + i]) * es);
      }
      break;
    case flagcxCommOpSend: sendBytes = o.count * es; break;
    case flagcxCommOpRecv: recvBytes = o.count * es; break;
    default: break;
  }
  if (o.op == flagcxCommOpBroadcast && c->rank != o.root) sendBytes = 0;
  if (o.op == flagcxCommOpReduce && c->rank != o.root) recvBytes = 0;
  const bool viaCopies = c->hostFallback;
  if (viaCopies) {
    // device buffers: stage through host memory (whole message, synchronous)
    FCX_CHECK(cudaToResult(cudaStreamSynchronize(o.stream), "host path"));
    hs.resize(sendBytes);
    hr.resize(std::max(recvBytes, (size_t)1));
    if (sendBytes) FCX_CHECK(cudaToResult(cudaMemcpy(hs.data(), o.send, sendBytes, cudaMemcpyDefault), "host path D2H"));
    if (o.op == flagcxCommOpAllGather || o.op == flagcxCommOpGather || o.op == flagcxCommOpAlltoAllv) {
      // these may leave parts of recv untouched or are written in place: start from the device contents
      if (recvBytes) FCX_CHECK(cudaToResult(cudaMemcpy(hr.data(), o.recv, recvBytes, cudaMemcpyDefault), "host path D2H"));
    }
    send = hs.data();
    recv = hr.data();
  }
  flagcxResult_t r = flagcxSuccess;
  switch (o.op) {
    case flagcxCommOpAllReduce: r = hostAllReduce(c->bs, send, recv, o.count, o.dt, o.red); break;
    case flagcxCommOpReduceScatter: r = hostReduceScatter(c->bs, send, recv, o.count, o.dt, o.red); break;
    case flagcxCommOpAllGather: r = hostAllGather(c->bs, send, recv, o.count, o.dt); break;
    case flagcxCommOpBroadcast: r = hostBroadcast(c->bs, send, recv, o.count, o.dt, o.root); break;
    case flagcxCommOpReduce: r = hostReduce(c->bs, send, recv, o.count, o.dt, o.red, o.root); break;
    case flagcxCommOpGather: r = hostGather(c->bs, send, recv, o.count, o.dt, o.root); break;
    case flagcxCommOpScatter: r = hostScatter(c->bs, send, recv, o.count, o.dt, o.root); break;
    case flagcxCommOpAlltoAll: r = hostAlltoAll(c->bs, send, recv, o.count, o.dt); break;
    case flagcxCommOpAlltoAllv: r = hostAlltoAllv(c->bs, send, t, t + n, recv, t + 2 * n, t + 3 * n, o.dt); break;
    case flagcxCommOpSend: r = hostSend(c->bs, send, o.count, o.dt, o.root); break;
    case flagcxCommOpRecv: r = hostRecv(c->bs, recv, o.count, o.dt, o.root); break;
    default: r = flagcxInvalidArgument;
  }
  FCX_CHECK(r);
  if (viaCopies && recvBytes) FCX_CHECK(cudaToResult(cudaMemcpy(o.recv, hr.data(), recvBytes, cudaMemcpyDefault), "host path H2D"));
  return flagcxSuccess;
}

// Host-route group: pair the i-th send with the i-th receive so that two
// ranks exchanging large messages progress both directions at once.
static flagcxResult_t hostGroup(flagcxComm *c, std::vector<PendingOp> &ops) {
  std::vector<PendingOp *> sends, recvs;
  for (auto &o : ops) {
    if (o.op == flagcxCommOpSend) sends.push_back(&o);
    else if (o.op == flagcxCommOpRecv) recvs.push_back(&o);
  }
  if (c->hostFallback && (!sends.empty() || !recvs.empty())) {
    // keep it simple on the copy route: receives run on a helper thread
    std::vector<flagcxResult_t> rr(recvs.size(), flagcxSuccess);
    std::thread th([&] { for (size_t i = 0; i < recvs.size(); i++) rr[i] = hostCollective(c, *recvs[i]); });
    flagcxResult_t r = flagcxSuccess;
    for (auto *s : sends) { flagcxResult_t x = hostCollective(c, *s); if (x != flagcxSuccess) r = x; }
    th.join();
    for (auto x : rr) if (x != flagcxSuccess) r = x;
    FCX_CHECK(r);
  } else {
    size_t np = std::min(sends.size(), recvs.size());
    for (size_t i = 0; i < np; i++) {
      PendingOp *s = sends[i], *r = recvs[i];
      FCX_CHECK(c->bs.sendrecv(s->root, 0x170000, s->send, s->count * dtypeSize(s->dt), r->root, 0x170000, r->recv,
                               r->count * dtypeSize(r->dt)));
    }
    for (size_t i = np; i < sends.size(); i++) FCX_CHECK(hostCollective(c, *sends[i]));
    for (size_t i = np; i < recvs.size(); i++) FCX_CHECK(hostCollective(c, *recvs[i]));
  }
  for (auto &o : ops)
    if (o.op != flagcxCommOpSend && o.op != flagcxCommOpRecv) FCX_CHECK(hostCollective(c, o));
  return flagcxSuccess;
}

// ------------------------------------------------------------------ direct route

static uint64_t heapOffOf(flagcxComm *c, const void *p, size_t bytes) {
  const char *base = c->heap.base[c->rank];
  if (p && (const char *)p >= base && (const char *)p + bytes <= base + c->heap.bytes) return (const char *)p - base;
  return ~0ull;
}

// Where `bytes` at `p` live as the peers see them: the symmetric heap, a registered segment, or nowhere.
static void resolveSeg(flagcxComm *c, const void *p, size_t bytes, int *seg, uint64_t *off) {
  *seg = FCX_SEG_NONE;
  *off = ~0ull;
  if (!p) return;
  uint64_t h = heapOffOf(c, p, bytes);
  if (h != ~0ull) { *seg = FCX_SEG_HEAP; *off = h; return; }
  for (int i = 1; i < (int)c->segs.size(); i++) {
    const Segment &sg = c->segs[i];
    if (sg.used && (const char *)p >= sg.localBase && (const char *)p + bytes <= sg.localBase + sg.bytes) {
      *seg = i;
      *off = (const char *)p - sg.localBase;
      return;
    }
  }
}

static bool isZcKind(int k) { return k == FCX_K_AR_ZC || k == FCX_K_RS_ZC || k == FCX_K_REDUCE_ZC || k == FCX_K_MOVE_ZC || k == FCX_K_MOVE_CE; }

// The byte mover a collective stands for when it runs in its LL form.
static int moveKindOf(flagcxCommOp_t op) {
  switch (op) {
    case flagcxCommOpAllGather: return FCX_K_AG;
    case flagcxCommOpBroadcast: return FCX_K_BCAST;
    case flagcxCommOpGather: return FCX_K_GATHER;
    case flagcxCommOpScatter: return FCX_K_SCATTER;
    case flagcxCommOpAlltoAll: return FCX_K_A2A;
    default: return 0;
  }
}

static flagcxResult_t launchOne(flagcxComm *c, FcxCollArgs &a, const Plan &plan, cudaStream_t st, bool timed) {
  a.kind = plan.kind;
  a.seq = ++c->seq;
  int nctas = std::max(1, std::min(plan.nctas, FCX_MAX_CTAS));
  if (timed) c->tuner->beginTiming(st);
  FcxDevComm dev = c->dev;
  if (plan.pipeBytes) dev.pipeBytes = plan.pipeBytes;  // the plan's own sub-chunk size (every rank holds the same plan)
  cudaError_t e = fcxLaunchColl(&dev, &a, nctas, st);
  if (timed) c->tuner->endTiming(st);
  c->counters.launches++;
  if (plan.kind >= 0 && plan.kind < 24) c->counters.kindLaunches[plan.kind]++;
  return cudaToResult(e, "collective kernel launch");
}

flagcxResult_t launchCollective(flagcxComm *c, const PendingOp &o) {
  const int n = c->nranks;
  const size_t es = dtypeSize(o.dt), eso = dtypeSize(o.outDt);
  const size_t stage = c->dev.stageBytes;
  FcxCollArgs a;
  memset(&a, 0, sizeof a);
  a.dtype = o.dt;
  a.outDtype = o.outDt;
  a.redop = o.red;
  a.root = o.root;
  a.elemSize = (int)es;
  a.scale = o.scale;
  a.sendHeapOff = a.recvHeapOff = ~0ull;
  a.useMc = c->dev.mcHeap != nullptr;
  a.moveOp = moveKindOf(o.op);
  const bool cast = o.outDt != o.dt || o.scale != 1.0f;
  const char *send = (const char *)o.send;
  char *recv = (char *)o.recv;

  if (o.op == flagcxCommNoOp) {  // barrier
    a.elemSize = 1;
    Plan p{FCX_K_BARRIER, 1};
    return launchOne(c, a, p, o.stream, false);
  }

  // A stream that is being captured must not see the online search (it synchronises on events).
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(o.stream, &capturing) != cudaSuccess) { cudaGetLastError(); capturing = cudaStreamCaptureStatusNone; }
  const bool maySearch = capturing == cudaStreamCaptureStatusNone;

  // Zero-copy route: the buffer that every rank hands to this collective is peer-visible (the ranks must
  // agree on that; a rank that finds a peer's buffer missing records a bad-argument error, it never guesses).
  static const bool zcEnabled = envInt("ZERO_COPY", 1) != 0;
  // Switch reduction pays from three ranks on: with two, the plain exchange moves S bytes per direction and
  // the switch 1.5 S (measured on two B200s: 404 GB/s through the switch, 526 GB/s without).
  // FLAGCX_ZC_MC: 0 never, 1 from three ranks on (default), 2 always.  FLAGCX_ZC_AG_MC: the same for the
  // multicast store of all-gather.  flagcxCommSetZeroCopyMulticast overrides both per communicator.
  const int zcMcEnv = c->zcMcMode, zcAgEnv = c->zcAgMcMode;
  const int zcMc = ((zcMcEnv == 2 || (zcMcEnv == 1 && n > 2)) ? 1 : 0) | ((zcAgEnv == 2 || (zcAgEnv == 1 && n > 2)) ? 2 : 0);
  a.sendSeg = a.recvSeg = FCX_SEG_NONE;
  bool zc = false;
  if (zcEnabled && n > 1) {
    int sseg, rseg;
    uint64_t soff, roff;
    size_t sspan = 0, rspan = 0;
    bool needS = false, needR = false;
    switch (o.op) {
      case flagcxCommOpAllReduce: needS = needR = true; sspan = o.count * es; rspan = o.count * eso; break;
      case flagcxCommOpReduceScatter: needS = true; sspan = (size_t)n * o.count * es; break;
      case flagcxCommOpReduce: needS = true; sspan = o.count * es; break;
      case flagcxCommOpGather: needS = true; sspan = o.count * es; break;
      case flagcxCommOpAllGather: needR = true; rspan = (size_t)n * o.count * es; break;
      case flagcxCommOpBroadcast: case flagcxCommOpScatter: needR = true; rspan = o.count * es; break;
      case flagcxCommOpAlltoAll: needR = send != recv; rspan = (size_t)n * o.count * es; break;
      case flagcxCommOpAlltoAllv: {
        needS = send != recv;
        const size_t *t = o.tables.data();
        for (int i = 0; i < n; i++) sspan = std::max(sspan, (t[i] + t[n + i]) * es);
        break;
      }
      default: break;
    }
    resolveSeg(c, needS ? send : nullptr, sspan, &sseg, &soff);
    resolveSeg(c, needR ? recv : nullptr, rspan, &rseg, &roff);
    zc = (needS || needR) && (!needS || sseg != FCX_SEG_NONE) && (!needR || rseg != FCX_SEG_NONE);
    if (zc) {
      a.sendSeg = needS ? sseg : FCX_SEG_NONE;
      a.sendHeapOff = needS ? soff : ~0ull;
      a.recvSeg = needR ? rseg : FCX_SEG_NONE;
      a.recvHeapOff = needR ? roff : ~0ull;
      a.useMc = c->dev.mcHeap != nullptr ? zcMc : 0;
    }
  }
  auto launchZc = [&](const Plan &p, bool timed) -> flagcxResult_t {
    a.send = send;
    a.recv = recv;
    a.count = o.count;
    a.sendStride = a.recvStride = o.count;
    if (p.kind != FCX_K_MOVE_CE) return launchOne(c, a, p, o.stream, timed);
    // Copy-engine form (the reference's own transport also moves data with copy engines and leaves the SMs
    // alone, flagcx/core/p2p.cc:73-109; there the CPU drives two staged copies per chunk, here the copies go
    // straight into the peers' receive buffers between two one-CTA kernels).
    if (a.recvSeg != FCX_SEG_HEAP) {  // only symmetric-heap receive buffers: the host must know the peers' addresses
      Plan q{FCX_K_MOVE_ZC, std::max(1, std::min(16, c->tuner->ctaBudget() > 0 ? c->tuner->ctaBudget() : 16))};
      return launchOne(c, a, q, o.stream, timed);
    }
    if (timed) c->tuner->beginTiming(o.stream);
    c->counters.kindLaunches[FCX_K_MOVE_CE]++;
    Plan open{FCX_K_MOVE_ZC, 1};
    a.ceOpen = 1;
    FCX_CHECK(launchOne(c, a, open, o.stream, false));
    a.ceOpen = 0;
    const size_t piece = o.count * es;
    const int me = c->rank;
    auto copy = [&](void *dst, const void *src) -> flagcxResult_t {
      if (dst == src || !piece) return flagcxSuccess;
      return cudaToResult(cudaMemcpyAsync(dst, src, piece, cudaMemcpyDeviceToDevice, o.stream), "copy-engine transfer");
    };
    for (int k = 0; k < n; k++) {
      const int p = (me + k) % n;
      char *peerRecv = p == me ? recv : c->heap.base[p] + a.recvHeapOff;
      switch (o.op) {
        case flagcxCommOpAllGather: FCX_CHECK(copy(peerRecv + (size_t)me * piece, send)); break;
        case flagcxCommOpAlltoAll: FCX_CHECK(copy(peerRecv + (size_t)me * piece, send + (size_t)p * piece)); break;
        case flagcxCommOpBroadcast: if (me == o.root) FCX_CHECK(copy(peerRecv, send)); break;
        case flagcxCommOpScatter: if (me == o.root) FCX_CHECK(copy(peerRecv, send + (size_t)p * piece)); break;
        default: return flagcxInternalError;
      }
    }
    FcxCollArgs b = a;
    b.count = 0;
    Plan close{FCX_K_BARRIER, 1};
    flagcxResult_t r = launchOne(c, b, close, o.stream, false);
    if (timed) c->tuner->endTiming(o.stream);
    return r;
  };

  if (o.op == flagcxCommOpAlltoAllv) {
    const size_t *t = o.tables.data();
    size_t maxPair = 0;
    for (int i = 0; i < n; i++) {
      a.scounts[i] = t[i];
      a.sdispls[i] = t[n + i];
      a.rcounts[i] = t[2 * n + i];
      a.rdispls[i] = t[3 * n + i];
      maxPair = std::max(maxPair, std::max(t[i], t[2 * n + i]) * es);
    }
    a.send = send;
    a.recv = recv;
    if (zc) {
      a.moveOp = FCX_K_A2AV;
      static const int zcCtas = (int)std::max<int64_t>(1, std::min<int64_t>(envInt("A2AV_CTAS", 32), FCX_MAX_CTAS));
      Plan p{FCX_K_MOVE_ZC, c->tuner->ctaBudget() > 0 ? std::min(zcCtas, c->tuner->ctaBudget()) : zcCtas};
      return launchOne(c, a, p, o.stream, false);
    }
    // like the reference (flagcx/flagcx.cc:1613-1616) the variable all-to-all is not searched online
    // The ranks see different counts, so nothing derived from them may shape the launch: every rank must
    // run the same number of CTAs (they pair up across GPUs).
    (void)maxPair;
    static const int a2avCtas = (int)std::max<int64_t>(1, std::min<int64_t>(envInt("A2AV_CTAS", 32), FCX_MAX_CTAS));
    Plan p{FCX_K_A2AV, a2avCtas};
    return launchOne(c, a, p, o.stream, false);
  }

  // Elements one launch can take, limited by the staging area.
  size_t cap;
  switch (o.op) {
    case flagcxCommOpAllReduce:
    case flagcxCommOpReduce: cap = (stage - 256 * (size_t)n) / (es + eso); break;
    case flagcxCommOpBroadcast:
    case flagcxCommOpScatter: cap = (stage - 64) / es; break;
    default: cap = (stage / n - 64) / es; break;  // per-rank piece
  }
  cap &= ~(size_t)63;
  if (zc) {
    // no staging, hence no size limit: the whole message is one launch when the tuner picks a zero-copy kind
    bool timed = false;
    Plan p = c->tuner->choose(o.op, std::max<size_t>(o.count * es, 1), o.dt, o.red, cast, &timed, true, maySearch);
    if (isZcKind(p.kind)) return launchZc(p, timed);
    a.sendSeg = a.recvSeg = FCX_SEG_NONE;
    a.sendHeapOff = a.recvHeapOff = ~0ull;
    a.useMc = c->dev.mcHeap != nullptr;
    if (o.count <= cap) {  // a staged kind won the search or is pinned: the message fits one launch
      a.count = o.count;
      a.send = send;
      a.recv = recv;
      a.sendStride = a.recvStride = o.count;
      return launchOne(c, a, p, o.stream, timed);
    }
  }
  size_t done = 0;
  do {
    size_t cnt = std::min(cap, o.count - done);
    size_t bytes = cnt * es;
    bool timed = false;
    Plan p = c->tuner->choose(o.op, std::max<size_t>(bytes, 1), o.dt, o.red, cast, &timed, false, maySearch);
    a.count = cnt;
    switch (o.op) {
      case flagcxCommOpAllReduce:
      case flagcxCommOpReduce:
      case flagcxCommOpBroadcast:
        a.send = send + done * es;
        a.recv = recv ? recv + done * eso : nullptr;
        break;
      case flagcxCommOpAllGather:
      case flagcxCommOpGather:
        a.send = send + done * es;
        a.recv = recv ? recv + done * es : nullptr;
        a.recvStride = o.count;
        break;
      case flagcxCommOpReduceScatter:
      case flagcxCommOpScatter:
        a.send = send ? send + done * es : nullptr;
        a.recv = recv + done * es;
        a.sendStride = o.count;
        break;
      case flagcxCommOpAlltoAll:
        a.send = send + done * es;
        a.recv = recv + done * es;
        a.sendStride = a.recvStride = o.count;
        break;
      default: return flagcxInvalidArgument;
    }
    FCX_CHECK(launchOne(c, a, p, o.stream, timed));
    done += cnt;
  } while (done < o.count);
  return flagcxSuccess;
}

// One fused launch for a batch of sends and receives.
flagcxResult_t launchP2pBatch(flagcxComm *c, const std::vector<PendingOp> &ops) {
  if (ops.empty()) return flagcxSuccess;
  cudaStream_t st = ops[0].stream;
  // other streams join the first one's timeline and wait for the result
  std::vector<cudaStream_t> others;
  for (auto &o : ops)
    if (o.stream != st && std::find(others.begin(), others.end(), o.stream) == others.end()) others.push_back(o.stream);
  cudaEvent_t ev = nullptr;
  if (!others.empty()) {
    cudaEventCreateWithFlags(&ev, cudaEventDisableTiming);
    for (auto s : others) { cudaEventRecord(ev, s); cudaStreamWaitEvent(st, ev, 0); }
  }
  // match self-sends with self-receives in order
  std::vector<const PendingOp *> selfS, selfR;
  for (auto &o : ops)
    if (o.root == c->rank) (o.op == flagcxCommOpSend ? selfS : selfR).push_back(&o);
  if (selfS.size() != selfR.size()) {
    FCX_WARN("a group holds %zu sends to self but %zu receives from self", selfS.size(), selfR.size());
    return flagcxInvalidUsage;
  }
  std::vector<FcxP2pOp> dops;
  size_t maxBytes = 0;
  for (size_t i = 0; i < selfS.size(); i++) {
    size_t sb = selfS[i]->count * dtypeSize(selfS[i]->dt), rb = selfR[i]->count * dtypeSize(selfR[i]->dt);
    if (sb != rb) { FCX_WARN("self send/recv %zu differ in size (%zu vs %zu bytes)", i, sb, rb); return flagcxInvalidArgument; }
    FcxP2pOp d{};
    d.isRecv = 2;
    d.peer = c->rank;
    d.buf = selfR[i]->recv;
    d.bytes = rb;
    d.heapOff = (uint64_t)(uintptr_t)selfS[i]->send;
    dops.push_back(d);
    maxBytes = std::max(maxBytes, rb);
  }
  const size_t chunk = c->dev.p2pChunkBytes;
  for (auto &o : ops) {
    if (o.root == c->rank) continue;
    FcxP2pOp d{};
    size_t bytes = o.count * dtypeSize(o.dt);
    uint64_t nch = bytes ? (bytes + chunk - 1) / chunk : 1;
    d.peer = o.root;
    d.bytes = bytes;
    if (o.op == flagcxCommOpSend) {
      d.isRecv = 0;
      d.buf = (void *)o.send;
      d.firstChunk = c->sendChunks[o.root];
      c->sendChunks[o.root] += nch;
      static const bool zeroCopy = envInt("P2P_ZEROCOPY", 1) != 0;
      d.heapOff = ~0ull;
      d.seg = FCX_SEG_NONE;
      if (bytes && zeroCopy) {
        resolveSeg(c, o.send, bytes, &d.seg, &d.heapOff);
        if (d.seg == FCX_SEG_NONE) d.heapOff = ~0ull;
      }
    } else {
      d.isRecv = 1;
      d.buf = o.recv;
      d.firstChunk = c->recvChunks[o.root];
      c->recvChunks[o.root] += nch;
      d.heapOff = ~0ull;
    }
    dops.push_back(d);
    maxBytes = std::max(maxBytes, bytes);
  }
  int per = maxBytes <= (64u << 10) ? 1 : maxBytes <= (1u << 20) ? 4 : maxBytes <= (8u << 20) ? 16 : 64;
  per = (int)envInt("P2P_CTAS", per);
  for (size_t i = 0; i < dops.size(); i += FCX_MAX_GROUP_OPS) {
    FcxP2pArgs g;
    memset(&g, 0, sizeof g);
    g.nops = (int)std::min<size_t>(FCX_MAX_GROUP_OPS, dops.size() - i);
    g.ctasPerOp = std::max(1, std::min(per, FCX_MAX_CTAS / g.nops));
    memcpy(g.ops, &dops[i], g.nops * sizeof(FcxP2pOp));
    FCX_CHECK(cudaToResult(fcxLaunchP2p(&c->dev, &g, st), "send/recv kernel launch"));
    c->counters.launches++;
  }
  if (ev) {
    cudaEventRecord(ev, st);
    for (auto s : others) cudaStreamWaitEvent(s, ev, 0);
    cudaEventDestroy(ev);
  }
  return flagcxSuccess;
}

// ------------------------------------------------------------------ dispatch

static flagcxResult_t validate(flagcxComm_t c, const PendingOp &o) {
  if (!validComm(c)) return flagcxInvalidArgument;
  if (!dtypeSize(o.dt) || !dtypeSize(o.outDt)) { FCX_WARN("unknown data type %d", (int)o.dt); return flagcxInvalidArgument; }
  const bool reduces = o.op == flagcxCommOpAllReduce || o.op == flagcxCommOpReduce || o.op == flagcxCommOpReduceScatter;
  if (reduces && (o.red < flagcxSum || o.red > flagcxAvg)) { FCX_WARN("unknown reduction %d", (int)o.red); return flagcxInvalidArgument; }
  const bool rooted = o.op == flagcxCommOpBroadcast || o.op == flagcxCommOpReduce || o.op == flagcxCommOpGather ||
                      o.op == flagcxCommOpScatter || o.op == flagcxCommOpSend || o.op == flagcxCommOpRecv;
  if (rooted && (o.root < 0 || o.root >= c->nranks)) { FCX_WARN("rank %d out of range", o.root); return flagcxInvalidArgument; }
  if (o.count > 0 && o.op != flagcxCommNoOp) {
    bool needSend = o.op != flagcxCommOpRecv && !(o.op == flagcxCommOpScatter && c->rank != o.root) &&
                    !(o.op == flagcxCommOpBroadcast && c->rank != o.root);
    bool needRecv = o.op != flagcxCommOpSend && !(o.op == flagcxCommOpGather && c->rank != o.root) &&
                    !(o.op == flagcxCommOpReduce && c->rank != o.root);
    if ((needSend && !o.send) || (needRecv && !o.recv)) { FCX_WARN("null buffer"); return flagcxInvalidArgument; }
    // element alignment: the kernels load and store whole elements
    const size_t es = dtypeSize(o.dt), eso = dtypeSize(o.outDt), n = (size_t)c->nranks;
    if ((needSend && ((uintptr_t)o.send % es)) || (needRecv && ((uintptr_t)o.recv % eso))) {
      FCX_WARN("buffer not aligned to its element size (%zu / %zu bytes)", es, eso);
      return flagcxInvalidArgument;
    }
    if (o.op == flagcxCommOpAlltoAllv) return flagcxSuccess;  // extents come from the tables
    // count x size x ranks must fit size_t
    const size_t widest = std::max(es, eso);
    if (o.count > (~(size_t)0) / widest / n) { FCX_WARN("count %zu overflows the byte size of the buffer", o.count); return flagcxInvalidArgument; }
    // send and receive ranges: identical or the documented in-place position, otherwise disjoint
    size_t sb = o.count * es, rb = o.count * eso;
    const char *inPlaceSend = (const char *)o.recv;  // where send may sit inside recv
    switch (o.op) {
      case flagcxCommOpAllGather: case flagcxCommOpGather: rb = n * o.count * es; inPlaceSend = (const char *)o.recv + (size_t)c->rank * sb; break;
      case flagcxCommOpReduceScatter: case flagcxCommOpScatter: sb = n * o.count * es; break;
      case flagcxCommOpAlltoAll: sb = rb = n * o.count * es; break;
      default: break;
    }
    if (needSend && needRecv && tInternalDepth == 0) {
      const char *s0 = (const char *)o.send, *r0 = (const char *)o.recv;
      bool inPlace = s0 == inPlaceSend;
      if (o.op == flagcxCommOpReduceScatter || o.op == flagcxCommOpScatter) inPlace = r0 == s0 + (size_t)c->rank * rb;
      const bool overlap = s0 < r0 + rb && r0 < s0 + sb;
      if (overlap && !inPlace) {
        FCX_WARN("send and receive buffers overlap without being the in-place form of the operation");
        return flagcxInvalidArgument;
      }
    }
  }
  return flagcxSuccess;
}

// FLAGCX_NVTX=1: one NVTX range per API call ("flagcx allreduce 1048576 B"), visible in Nsight Systems timelines.
namespace {
const char *const kOpLabel[] = {"send", "recv", "broadcast", "gather", "scatter", "reduce", "allreduce", "allgather",
                                "reducescatter", "alltoall", "alltoallv", "barrier"};
struct NvtxRange {
  bool on;
  NvtxRange(int op, size_t bytes) {
    static const bool enabled = envInt("NVTX", 0) != 0;
    on = enabled;
    if (!on) return;
    char label[96];
    snprintf(label, sizeof label, "flagcx %s %zu B", op >= 0 && op < 12 ? kOpLabel[op] : "op", bytes);
    nvtxRangePushA(label);
  }
  ~NvtxRange() { if (on) nvtxRangePop(); }
};
}  // namespace

static flagcxResult_t submit(flagcxComm_t c, PendingOp &&o) {
  FCX_CHECK(validate(c, o));
  size_t bytes = o.count * dtypeSize(o.dt);
  NvtxRange nvtx((int)o.op, bytes);
  if (o.op != flagcxCommNoOp) count(c, o.op, bytes);
  FCX_TRACE(SUB_CALL, "op %d count %zu dtype %d red %d root %d", (int)o.op, o.count, (int)o.dt, (int)o.red, o.root);
  if (tGroupDepth > 0) {
    if (std::find(tGroupComms.begin(), tGroupComms.end(), c) == tGroupComms.end()) tGroupComms.push_back(c);
    c->pending.push_back(std::move(o));
    return flagcxSuccess;
  }
  if (c->nclusters > 1 && c->nranks > 1 && o.op != flagcxCommNoOp && o.op != flagcxCommOpSend && o.op != flagcxCommOpRecv &&
      o.count > 0) {
    // several clusters: try the hierarchical plan first (its stages come back here on sub-communicators)
    bool handled = false;
    FCX_CHECK(c2cExecute(c, o, &handled));
    if (handled) return flagcxSuccess;
  }
  if (c->hostOnly || c->hostFallback) return hostCollective(c, o);
  if (o.op == flagcxCommOpSend || o.op == flagcxCommOpRecv) return launchP2pBatch(c, {o});
  if (o.count == 0 && o.op != flagcxCommNoOp && o.op != flagcxCommOpAlltoAllv) return flagcxSuccess;
  if (c->nranks == 1) {
    // nothing to exchange: a device copy when the buffers differ
    size_t nb = o.count * dtypeSize(o.dt);
    if (o.op == flagcxCommOpAlltoAllv) {
      const size_t *t = o.tables.data();
      nb = t[0] * dtypeSize(o.dt);
      const char *s = (const char *)o.send + t[1] * dtypeSize(o.dt);
      char *d = (char *)o.recv + t[3] * dtypeSize(o.dt);
      if (s != d && nb) return cudaToResult(cudaMemcpyAsync(d, s, nb, cudaMemcpyDeviceToDevice, o.stream), "single-rank copy");
      return flagcxSuccess;
    }
    if (o.op != flagcxCommNoOp && (o.outDt != o.dt || o.scale != 1.0f || o.red == flagcxAvg)) return launchCollective(c, o);
    if (o.op != flagcxCommNoOp && o.send != o.recv && nb)
      return cudaToResult(cudaMemcpyAsync(o.recv, o.send, nb, cudaMemcpyDeviceToDevice, o.stream), "single-rank copy");
    return flagcxSuccess;
  }
  return launchCollective(c, o);
}

static PendingOp mk(flagcxCommOp_t op, const void *s, void *r, size_t cnt, flagcxDataType_t dt, flagcxRedOp_t red, int root,
                    flagcxStream_t st) {
  PendingOp o;
  o.op = op;
  o.send = s;
  o.recv = r;
  o.count = cnt;
  o.dt = o.outDt = dt;
  o.red = red;
  o.root = root;
  o.scale = 1.0f;
  o.stream = streamOf(st);
  return o;
}

}  // namespace fcx

using namespace fcx;

extern "C" {

flagcxResult_t flagcxBarrier(flagcxComm_t comm, flagcxStream_t stream) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  if (comm->hostOnly || comm->hostFallback) {
    if (comm->hostFallback) cudaStreamSynchronize(streamOf(stream));
    return comm->bs.barrier();
  }
  PendingOp o = mk(flagcxCommNoOp, nullptr, nullptr, 0, flagcxInt8, flagcxSum, 0, stream);
  if (comm->nranks > 1) FCX_CHECK(launchCollective(comm, o));
  // the reference's barrier returns only after the stream has drained (flagcx/flagcx.cc:699-710)
  return cudaToResult(cudaStreamSynchronize(streamOf(stream)), "barrier");
}

flagcxResult_t flagcxReduce(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, flagcxRedOp_t op, int root,
                            flagcxComm_t comm, flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpReduce, sendbuff, recvbuff, count, datatype, op, root, stream));
}
flagcxResult_t flagcxGather(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root,
                            flagcxComm_t comm, flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpGather, sendbuff, recvbuff, count, datatype, flagcxSum, root, stream));
}
flagcxResult_t flagcxScatter(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root,
                             flagcxComm_t comm, flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpScatter, sendbuff, recvbuff, count, datatype, flagcxSum, root, stream));
}
flagcxResult_t flagcxBroadcast(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root,
                               flagcxComm_t comm, flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpBroadcast, sendbuff, recvbuff, count, datatype, flagcxSum, root, stream));
}
flagcxResult_t flagcxAllReduce(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, flagcxRedOp_t op,
                               flagcxComm_t comm, flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpAllReduce, sendbuff, recvbuff, count, datatype, op, 0, stream));
}
flagcxResult_t flagcxAllReduceCast(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t inType,
                                   flagcxDataType_t outType, float scale, flagcxRedOp_t op, flagcxComm_t comm,
                                   flagcxStream_t stream) {
  PendingOp o = mk(flagcxCommOpAllReduce, sendbuff, recvbuff, count, inType, op, 0, stream);
  o.outDt = outType;
  o.scale = scale;
  if (validComm(comm) && (comm->hostOnly || comm->hostFallback) && (outType != inType || scale != 1.0f)) return flagcxNotSupported;
  return submit(comm, std::move(o));
}
flagcxResult_t flagcxReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, flagcxDataType_t datatype, flagcxRedOp_t op,
                                   flagcxComm_t comm, flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpReduceScatter, sendbuff, recvbuff, recvcount, datatype, op, 0, stream));
}
flagcxResult_t flagcxAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, flagcxDataType_t datatype, flagcxComm_t comm,
                               flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpAllGather, sendbuff, recvbuff, sendcount, datatype, flagcxSum, 0, stream));
}
flagcxResult_t flagcxAlltoAll(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, flagcxComm_t comm,
                              flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpAlltoAll, sendbuff, recvbuff, count, datatype, flagcxSum, 0, stream));
}
flagcxResult_t flagcxAlltoAllv(const void *sendbuff, size_t *sendcounts, size_t *sdispls, void *recvbuff, size_t *recvcounts,
                               size_t *rdispls, flagcxDataType_t datatype, flagcxComm_t comm, flagcxStream_t stream) {
  if (!validComm(comm) || !sendcounts || !sdispls || !recvcounts || !rdispls) return flagcxInvalidArgument;
  PendingOp o = mk(flagcxCommOpAlltoAllv, sendbuff, recvbuff, 1, datatype, flagcxSum, 0, stream);
  const int n = comm->nranks;
  o.tables.resize(4 * n);
  size_t total = 0;
  for (int i = 0; i < n; i++) {
    o.tables[i] = sendcounts[i];
    o.tables[n + i] = sdispls[i];
    o.tables[2 * n + i] = recvcounts[i];
    o.tables[3 * n + i] = rdispls[i];
    total += sendcounts[i];
  }
  o.count = total;
  return submit(comm, std::move(o));
}
flagcxResult_t flagcxSend(const void *sendbuff, size_t count, flagcxDataType_t datatype, int peer, flagcxComm_t comm,
                          flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpSend, sendbuff, nullptr, count, datatype, flagcxSum, peer, stream));
}
flagcxResult_t flagcxRecv(void *recvbuff, size_t count, flagcxDataType_t datatype, int peer, flagcxComm_t comm,
                          flagcxStream_t stream) {
  return submit(comm, mk(flagcxCommOpRecv, nullptr, recvbuff, count, datatype, flagcxSum, peer, stream));
}

flagcxResult_t flagcxGroupStart(flagcxComm_t) {
  tGroupDepth++;
  return flagcxSuccess;
}

flagcxResult_t flagcxGroupEnd(flagcxComm_t) {
  if (tGroupDepth <= 0) { FCX_WARN("flagcxGroupEnd without flagcxGroupStart"); return flagcxInvalidUsage; }
  if (--tGroupDepth > 0) return flagcxSuccess;
  std::vector<flagcxComm *> comms;
  comms.swap(tGroupComms);
  flagcxResult_t res = flagcxSuccess;
  for (flagcxComm *c : comms) {
    std::vector<PendingOp> ops;
    ops.swap(c->pending);
    if (res != flagcxSuccess) continue;
    if ((c->hostOnly || c->hostFallback) && c->nclusters == 1) { res = hostGroup(c, ops); continue; }
    if (c->hostOnly || c->hostFallback) {
      // hierarchical host communicator: point-to-point pairs first, then each collective through the planner
      std::vector<PendingOp> p2pOnly, rest;
      for (auto &o : ops) (o.op == flagcxCommOpSend || o.op == flagcxCommOpRecv ? p2pOnly : rest).push_back(o);
      res = hostGroup(c, p2pOnly);
      for (auto &o : rest) {
        if (res != flagcxSuccess) break;
        PendingOp copy = o;
        res = submit(c, std::move(copy));
        c->counters.calls[o.op]--;
        c->counters.bytes[o.op] -= o.count * dtypeSize(o.dt);
      }
      continue;
    }
    std::vector<PendingOp> p2p;
    for (auto &o : ops)
      if (o.op == flagcxCommOpSend || o.op == flagcxCommOpRecv) p2p.push_back(o);
    if (!p2p.empty()) res = launchP2pBatch(c, p2p);
    for (auto &o : ops) {
      if (res != flagcxSuccess) break;
      if (o.op == flagcxCommOpSend || o.op == flagcxCommOpRecv) continue;
      if (o.count == 0 && o.op != flagcxCommOpAlltoAllv) continue;
      if (c->nranks == 1 || c->nclusters > 1) {
        // re-enter the ungrouped path for the special cases
        PendingOp copy = o;
        res = submit(c, std::move(copy));
        c->counters.calls[o.op]--;
        c->counters.bytes[o.op] -= o.count * dtypeSize(o.dt);
      } else {
        res = launchCollective(c, o);
      }
    }
  }
  return res;
}

flagcxResult_t flagcxTunerPin(flagcxComm_t comm, const char *kind, int nctas) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  if (!kind) { comm->tuner->pin(nullptr); return flagcxSuccess; }
  int k = kindFromName(kind);
  if (k < 0) return flagcxInvalidArgument;
  Plan p{k, std::max(1, nctas)};
  comm->tuner->pin(&p);
  return flagcxSuccess;
}

// Every variant that can legally serve a call, best first by the cost model (for tuning tools).
flagcxResult_t flagcxTunerCandidates(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red,
                                     int zeroCopy, int maxOut, int *kinds, int *nctas, int *count) {
  if (!validComm(comm) || !kinds || !nctas || !count || maxOut < 1 || !comm->tuner) return flagcxInvalidArgument;
  std::vector<Plan> c = comm->tuner->candidates(op, std::max<size_t>(bytes, 1), dt, red, false, zeroCopy != 0);
  std::stable_sort(c.begin(), c.end(), [&](const Plan &a, const Plan &b) {
    return comm->tuner->estimate(a, op, bytes, dt) < comm->tuner->estimate(b, op, bytes, dt);
  });
  *count = (int)std::min<size_t>(c.size(), (size_t)maxOut);
  for (int i = 0; i < *count; i++) { kinds[i] = c[i].kind; nctas[i] = c[i].nctas; }
  return flagcxSuccess;
}
const char *flagcxKindName(int kind) { return kindName(kind); }

flagcxResult_t flagcxTunerPinEx(flagcxComm_t comm, const char *kind, int nctas, unsigned int pipeBytes) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  if (!kind) { comm->tuner->pin(nullptr); return flagcxSuccess; }
  int k = kindFromName(kind);
  if (k < 0) return flagcxInvalidArgument;
  Plan p{k, std::max(1, nctas), pipeBytes};
  comm->tuner->pin(&p);
  return flagcxSuccess;
}

flagcxResult_t flagcxTunerRecordEx(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, const char *kind, int nctas, unsigned int pipeBytes,
                                   double us) {
  if (!validComm(comm) || !kind) return flagcxInvalidArgument;
  int k = kindFromName(kind);
  if (k < 0) return flagcxInvalidArgument;
  comm->tuner->record(op, bytes, Plan{k, nctas, pipeBytes}, us);
  return flagcxSuccess;
}

flagcxResult_t flagcxCommSetCtaBudget(flagcxComm_t comm, int maxCtas) {
  if (!validComm(comm) || maxCtas < 0) return flagcxInvalidArgument;
  if (comm->tuner) comm->tuner->setCtaBudget(maxCtas);
  return flagcxSuccess;
}

flagcxResult_t flagcxTunerQuery(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red,
                                char *kindOut, size_t kindOutBytes, int *nctas, double *estimate) {
  return flagcxTunerQueryEx(comm, op, bytes, dt, red, 0, kindOut, kindOutBytes, nctas, estimate);
}

flagcxResult_t flagcxTunerQueryEx(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red,
                                  int zeroCopy, char *kindOut, size_t kindOutBytes, int *nctas, double *estimate) {
  if (!validComm(comm)) return flagcxInvalidArgument;
  Plan p = comm->tuner->peek(op, bytes, dt, red, false, zeroCopy != 0);
  if (kindOut && kindOutBytes) snprintf(kindOut, kindOutBytes, "%s", kindName(p.kind));
  if (nctas) *nctas = p.nctas;
  if (estimate) *estimate = comm->tuner->estimate(p, op, bytes, dt);
  return flagcxSuccess;
}

// The plan the cost-model prior would pick on a machine of `nranks` GPUs, without a communicator (and without a GPU).
flagcxResult_t flagcxTunerPriorPlan(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, int nranks, int multicast, char *kindOut,
                                    size_t kindOutBytes, int *nctas, double *estimate) {
  if (nranks < 1 || nranks > FCX_MAX_RANKS) return flagcxInvalidArgument;
  TunerCaps caps;
  caps.nranks = nranks;
  caps.multicast = multicast != 0;
  caps.stageBytes = (size_t)envInt("STAGE_BYTES", 512ll << 20);
  caps.maxCtas = (int)std::min<int64_t>(envInt("MAX_CTAS", 128), FCX_MAX_CTAS);
  caps.pipeBytes = (size_t)envInt("PIPE_BYTES", 16ll << 20);
  Tuner t(nullptr, caps);
  Plan p = t.peek(op, bytes, dt, flagcxSum, false);
  if (kindOut && kindOutBytes) snprintf(kindOut, kindOutBytes, "%s", kindName(p.kind));
  if (nctas) *nctas = p.nctas;
  if (estimate) *estimate = t.estimate(p, op, bytes, dt);
  return flagcxSuccess;
}

// The same with the caller's buffers taken as peer-visible (zero-copy kinds allowed) and a CTA budget (0 = none).
flagcxResult_t flagcxTunerPriorPlanEx(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, int nranks, int multicast, int zeroCopy,
                                      int ctaBudget, char *kindOut, size_t kindOutBytes, int *nctas, double *estimate) {
  if (nranks < 1 || nranks > FCX_MAX_RANKS) return flagcxInvalidArgument;
  TunerCaps caps;
  caps.nranks = nranks;
  caps.multicast = multicast != 0;
  caps.stageBytes = (size_t)envInt("STAGE_BYTES", 512ll << 20);
  caps.maxCtas = (int)std::min<int64_t>(envInt("MAX_CTAS", 128), FCX_MAX_CTAS);
  caps.pipeBytes = (size_t)envInt("PIPE_BYTES", 16ll << 20);
  Tuner t(nullptr, caps);
  if (ctaBudget > 0) t.setCtaBudget(ctaBudget);
  Plan p = t.peek(op, bytes, dt, flagcxSum, false, zeroCopy != 0);
  if (kindOut && kindOutBytes) snprintf(kindOut, kindOutBytes, "%s", kindName(p.kind));
  if (nctas) *nctas = p.nctas;
  if (estimate) *estimate = t.estimate(p, op, bytes, dt);
  return flagcxSuccess;
}

flagcxResult_t flagcxCommWaitTest(flagcxComm_t comm, flagcxStream_t stream) {
  if (!validComm(comm) || comm->hostOnly || !comm->heap.bytes) return flagcxInvalidArgument;
  return cudaToResult(fcxLaunchWaitTest(&comm->dev, ~0ull, streamOf(stream)), "wait test launch");
}

}  // extern "C"
