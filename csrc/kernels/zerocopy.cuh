// Zero-copy collective kernels: the peers' user buffers are read and written in place.
//
// A buffer qualifies when every rank can reach it: it lies in the symmetric heap (flagcxMemAlloc) or in a
// segment made peer-visible by flagcxCommRegister.  The reference gives registration the same meaning: a
// registered buffer skips the staging copy of its transport (flagcx/core/net.cc:150-168, 234-246) and, on one
// vendor's GPUs, is handed to the vendor library's own registration (flagcx/flagcx.cc:186-201).
//
// Protocol of every kind in this file (one launch, the same CTA count on every rank):
//   1. each CTA writes where its rank's buffers live (segment, offset) into a mailbox on every peer and
//      raises its flag there (release); it then waits for the same from the peers' CTA of the same index.
//      A peer's kernel having started means that everything queued before it on the peer's stream is done,
//      so after this barrier the peers' send buffers hold their data and their recv buffers may be written;
//   2. the data phase: loads from the peers' send buffers and/or stores into the peers' recv buffers, or
//      multimem.ld_reduce / multimem.st on the NVSwitch multicast alias when the buffers sit at the same
//      heap offset on every rank;
//   3. a second barrier: a rank leaves only when no peer CTA still reads or writes its buffers.
// Nothing is staged, so a message makes one pass over NVLink and at most one over local memory, and there
// is no size limit per launch.
//
#pragma once
#include "prims.cuh"

namespace fcxdev {

struct ZcPeers {
  const char *send[FCX_MAX_RANKS];  // rank p's send buffer as this rank addresses it (null: not peer-visible)
  char *recv[FCX_MAX_RANKS];
  const char *mcSend;               // multicast alias of the send buffers, null unless all ranks use one heap offset
  char *mcRecv;
  uint64_t x[FCX_MAX_RANKS], y[FCX_MAX_RANKS];  // two free words per source rank (all-to-all-v: displacement, count)
};

// Step 1 of the protocol.  `needSend` / `needRecv`: which buffers the kind will touch on the peers; a peer
// whose buffer is not visible, or a heap range that leaves the heap, ends the collective with a recorded
// FCX_ERR_BADARG instead of a wild access.  sendSpan / recvSpan are the bytes a peer may touch from the offset.
// xTo[p] / yTo[p]: two words handed to rank p (may be null).
__device__ __forceinline__ bool zcExchange(const FcxDevComm &dc, const FcxCollArgs &a, uint64_t seq, int cta, bool needSend,
                                           bool needRecv, size_t sendSpan, size_t recvSpan, const uint64_t *xTo,
                                           const uint64_t *yTo, ZcPeers *z) {
  const int n = dc.nranks, me = dc.rank, t = threadIdx.x;
  __syncthreads();
  bool ok = true;
  if (t < n && t != me) {
    FcxMail *mb = (FcxMail *)(dc.heap[t] + FCX_OFF_MAIL) + (seq & 1) * FCX_MAX_RANKS + me;
    stRelaxed(&mb->a, (uint64_t)(int64_t)a.sendSeg);
    stRelaxed(&mb->b, a.sendHeapOff);
    stRelaxed(&mb->c, (uint64_t)(int64_t)a.recvSeg);
    stRelaxed(&mb->d, a.recvHeapOff);
    stRelaxed(&mb->e, xTo ? xTo[t] : 0);
    stRelaxed(&mb->f, yTo ? yTo[t] : 0);
    stRelease(flagSlot(dc, t, cta, me), barrierValue(seq, 1));
    ok = waitGe(dc, flagSlot(dc, me, cta, t), barrierValue(seq, 1), t, FCX_WAIT_BARRIER, cta, seq);
  }
  if (!__syncthreads_and(ok)) return false;
  bool symS = a.sendSeg == FCX_SEG_HEAP, symR = a.recvSeg == FCX_SEG_HEAP, bad = false;
  int badPeer = me;
  for (int p = 0; p < n; p++) {
    int sseg, rseg;
    uint64_t soff, roff;
    if (p == me) {
      sseg = a.sendSeg; soff = a.sendHeapOff; rseg = a.recvSeg; roff = a.recvHeapOff;
      z->x[p] = xTo ? xTo[me] : 0;
      z->y[p] = yTo ? yTo[me] : 0;
      // this rank's own buffers are used through the pointers the caller gave
      z->send[p] = (const char *)a.send;
      z->recv[p] = (char *)a.recv;
      if ((needSend && (sseg == FCX_SEG_NONE || !a.send)) || (needRecv && (rseg == FCX_SEG_NONE || !a.recv))) { bad = true; badPeer = p; }
    } else {
      const FcxMail *mb = (const FcxMail *)(dc.heap[me] + FCX_OFF_MAIL) + (seq & 1) * FCX_MAX_RANKS + p;
      sseg = (int)(int64_t)ldRelaxed(&mb->a); soff = ldRelaxed(&mb->b);
      rseg = (int)(int64_t)ldRelaxed(&mb->c); roff = ldRelaxed(&mb->d);
      z->x[p] = ldRelaxed(&mb->e);
      z->y[p] = ldRelaxed(&mb->f);
      z->send[p] = needSend ? zcResolve(dc, sseg, soff, p) : nullptr;
      z->recv[p] = needRecv ? zcResolve(dc, rseg, roff, p) : nullptr;
      if ((needSend && !z->send[p]) || (needRecv && !z->recv[p])) { bad = true; badPeer = p; }
    }
    if (needSend && sseg == FCX_SEG_HEAP && (soff > dc.heapBytes || sendSpan > dc.heapBytes - soff)) { bad = true; badPeer = p; }
    if (needRecv && rseg == FCX_SEG_HEAP && (roff > dc.heapBytes || recvSpan > dc.heapBytes - roff)) { bad = true; badPeer = p; }
    symS = symS && sseg == FCX_SEG_HEAP && soff == a.sendHeapOff;
    symR = symR && rseg == FCX_SEG_HEAP && roff == a.recvHeapOff;
  }
  if (bad) {
    if (t == 0) giveUp(dc, FCX_ERR_BADARG, badPeer, FCX_WAIT_BARRIER, cta, 0, 0, seq);
    return false;
  }
  const bool mc = dc.mcHeap != nullptr && a.useMc;
  z->mcSend = (mc && symS && needSend && (a.sendHeapOff & 15u) == 0) ? dc.mcHeap + a.sendHeapOff : nullptr;
  z->mcRecv = (mc && symR && needRecv && (a.recvHeapOff & 15u) == 0) ? dc.mcHeap + a.recvHeapOff : nullptr;
  return true;
}

// multimem accesses are weak with respect to the generic proxy's ordinary loads and stores of the same
// addresses only through fences; a system-scope fence by every thread before the closing barrier makes the
// multicast stores visible to whatever the peers run next.
__device__ __forceinline__ void zcFenceBeforeClose() { __threadfence_system(); }

// ---------------------------------------------------------------- reducing kinds

// Units [first, first + cnt) of the range, U at a time per thread, for exactly P ranks: all U x P loads are
// issued before anything is combined.  Returns how many units were handled (a multiple of U x gstride); the
// caller finishes the rest.
template <typename TIn, typename TOut, int U, int P>
__device__ __forceinline__ size_t zcReduceBulk(const FcxDevComm &dc, const FcxCollArgs &a, const char *const *src, char *const *dst, int nd,
                                               size_t first, size_t cnt, size_t gtid, size_t gstride) {
  using Acc = typename Elem<TIn>::Acc;
  constexpr int G = 16 / (int)sizeof(TIn);
  const size_t batches = cnt / ((size_t)U * gstride);
  const char *s[P];
#pragma unroll
  for (int p = 0; p < P; p++) s[p] = src[p];
  for (size_t b = 0; b < batches; b++) {
    const size_t u0 = first + b * U * gstride + gtid;
    uint4 raw[U * P];
#pragma unroll
    for (int i = 0; i < U; i++)
#pragma unroll
      for (int p = 0; p < P; p++) raw[i * P + p] = ld16(s[p] + (u0 + i * gstride) * 16);
#pragma unroll
    for (int i = 0; i < U; i++) {
      Acc acc[G];
#pragma unroll
      for (int p = 0; p < P; p++) {
        union { uint4 v; TIn t[G]; } w;
        w.v = raw[i * P + p];
#pragma unroll
        for (int e = 0; e < G; e++) {
          const Acc x = Elem<TIn>::up(w.t[e]);
          acc[e] = p == 0 ? x : applyOp<Acc>(acc[e], x, a.redop);
        }
      }
#pragma unroll
      for (int e = 0; e < G; e++) acc[e] = finish<Acc>(acc[e], a.redop, P, a.scale);
      uint4 packed;
      packUnit<TIn, G>(acc, &packed);
      for (int k = 0; k < nd; k++) st16(dst[k] + (u0 + i * gstride) * 16, packed);
    }
  }
  return batches * U * gstride;
}

// out = finish(x_0 (op) x_1 ... (op) x_{n-1}) for `nElems` elements that start `srcOff` elements into every
// rank's send buffer.  The result goes `dstOff` elements into: this rank's recv buffer (toSelf), every other
// rank's recv buffer (toPeers), or both.  Ranks are combined in rank order, so the owner's result is the one
// every rank receives, bit for bit.
template <typename TIn, typename TOut>
__device__ __forceinline__ void zcReduceRange(const FcxDevComm &dc, const FcxCollArgs &a, const ZcPeers &z, size_t srcOff,
                                              size_t dstOff, size_t nElems, bool toSelf, bool toPeers, size_t gtid,
                                              size_t gstride) {
  using AI = typename Elem<TIn>::Acc;
  using AO = typename Elem<TOut>::Acc;
  constexpr int ESI = (int)sizeof(TIn), ESO = (int)sizeof(TOut);
  constexpr int G = 16 / (ESI < ESO ? ESI : ESO);
  constexpr int INB = G * ESI, OUTB = G * ESO;
  const int n = dc.nranks, me = dc.rank;
  if (!nElems) return;
  const char *src[FCX_MAX_RANKS];
  char *dst[FCX_MAX_RANKS];
  int nd = 0;
  bool alS = true, alD = true;
  for (int p = 0; p < n; p++) {
    src[p] = z.send[p] + srcOff * ESI;
    alS = alS && aligned16(src[p]);
  }
  for (int k = 0; k < n; k++) {
    int p = (me + k) % n;  // own buffer first, then the peers starting with the right-hand neighbour
    if ((p == me && toSelf) || (p != me && toPeers)) {
      dst[nd] = z.recv[p] + dstOff * ESO;
      alD = alD && aligned16(dst[nd]);
      nd++;
    }
  }
  const size_t nunits = (nElems + G - 1) / G;
  size_t firstPlain = 0;  // units below this index are done through the switch

  if constexpr (ESI == ESO && Mm<TIn>::ok) {
    if (z.mcSend != nullptr && alS && alD && Mm<TIn>::opOk(a.redop)) {
      const char *mcs = z.mcSend + srcOff * ESI;
      char *mcd = (toSelf && toPeers && z.mcRecv != nullptr) ? z.mcRecv + dstOff * ESO : nullptr;
      const size_t nfull = nElems / G;
      constexpr int U = 8;
      size_t u = gtid;
      for (; u + (U - 1) * gstride < nfull; u += U * gstride) {
        uint4 r[U];
#pragma unroll
        for (int i = 0; i < U; i++) r[i] = Mm<TIn>::ldReduce(mcs + (u + i * gstride) * 16, a.redop);
#pragma unroll
        for (int i = 0; i < U; i++) {
          const uint4 f = mmFinish<TIn>(r[i], a.redop, n, a.scale);
          const size_t o = (u + i * gstride) * 16;
          if (mcd) mmStore(mcd + o, f);
          else
            for (int k = 0; k < nd; k++) st16(dst[k] + o, f);
        }
      }
      for (; u < nfull; u += gstride) {
        const uint4 f = mmFinish<TIn>(Mm<TIn>::ldReduce(mcs + u * 16, a.redop), a.redop, n, a.scale);
        if (mcd) mmStore(mcd + u * 16, f);
        else
          for (int k = 0; k < nd; k++) st16(dst[k] + u * 16, f);
      }
      firstPlain = nfull;  // at most one ragged unit is left for the plain path
    }
  }

  // Plain loads from peers are latency-bound (a load over NVLink takes microseconds): the aligned bulk of the
  // range keeps U units x P ranks = about sixteen 16-byte loads per thread in flight before it combines any.
  if constexpr (ESI == ESO && Mm<TIn>::ok) {  // the floating-point types of gradients and activations
    if (alS && alD) {
      const size_t nfull = nElems / G;
      if (nfull > firstPlain) {
        const size_t cnt = nfull - firstPlain;
        size_t did = 0;
        if (n == 2) did = zcReduceBulk<TIn, TOut, 8, 2>(dc, a, src, dst, nd, firstPlain, cnt, gtid, gstride);
        else if (n == 4) did = zcReduceBulk<TIn, TOut, 4, 4>(dc, a, src, dst, nd, firstPlain, cnt, gtid, gstride);
        else if (n == 8) did = zcReduceBulk<TIn, TOut, 2, 8>(dc, a, src, dst, nd, firstPlain, cnt, gtid, gstride);
        firstPlain += did;  // whole batches only: the remainder takes the unit-at-a-time path below
      }
    }
  }

  auto gather = [&](size_t u, AI *acc) {
    const int nv = (int)min((size_t)G, nElems - u * G);
    for (int p = 0; p < n; p++) {
      AI in[G];
      loadUnit<TIn, G>(src[p] + u * INB, alS, nv, in);
      if (p == 0) {
#pragma unroll
        for (int i = 0; i < G; i++) acc[i] = in[i];
      } else {
#pragma unroll
        for (int i = 0; i < G; i++) acc[i] = applyOp<AI>(acc[i], in[i], a.redop);
      }
    }
  };
  auto emit = [&](size_t u, const AI *acc) {
    const int nv = (int)min((size_t)G, nElems - u * G);
    AO res[G];
#pragma unroll
    for (int i = 0; i < G; i++) res[i] = accCast<AO, AI>(finish<AI>(acc[i], a.redop, n, a.scale));
    uint4 packed[OUTB / 16];
    packUnit<TOut, G>(res, packed);
    for (int k = 0; k < nd; k++) storeUnit<TOut, G>(dst[k] + u * OUTB, alD, nv, packed);
  };
  size_t u = firstPlain + gtid;
  for (; u + gstride < nunits; u += 2 * gstride) {
    AI acc0[G], acc1[G];
    gather(u, acc0);
    gather(u + gstride, acc1);
    emit(u, acc0);
    emit(u + gstride, acc1);
  }
  for (; u < nunits; u += gstride) {
    AI acc[G];
    gather(u, acc);
    emit(u, acc);
  }
}

template <typename TIn, typename TOut>
__device__ void fcxZcReduceBody(const FcxDevComm &dc, const FcxCollArgs &a, int cta, int nctas) {
  constexpr int ESI = (int)sizeof(TIn), ESO = (int)sizeof(TOut);
  constexpr int G = 16 / (ESI < ESO ? ESI : ESO);
  const int n = dc.nranks, me = dc.rank;
  const uint64_t seq = nextSeq(dc);
  const size_t gtid = (size_t)cta * blockDim.x + threadIdx.x, gstride = (size_t)nctas * blockDim.x;
  if (!prologue(dc, seq, cta)) return;
  ZcPeers z;
  const bool isAR = a.kind == FCX_K_AR_ZC, isRS = a.kind == FCX_K_RS_ZC;
  const size_t sendSpan = (isRS ? (size_t)(n - 1) * a.sendStride + a.count : a.count) * ESI;
  if (zcExchange(dc, a, seq, cta, true, isAR, sendSpan, a.count * ESO, nullptr, nullptr, &z)) {
    if (isAR) {
      // slices in whole units so that every slice starts as aligned as the buffer itself
      const size_t totalUnits = (a.count + G - 1) / G, sliceUnits = (totalUnits + n - 1) / n;
      const size_t lo = min(a.count, (size_t)me * sliceUnits * G), hi = min(a.count, ((size_t)me + 1) * sliceUnits * G);
      zcReduceRange<TIn, TOut>(dc, a, z, lo, lo, hi - lo, true, true, gtid, gstride);
    } else if (isRS) {
      zcReduceRange<TIn, TOut>(dc, a, z, (size_t)me * a.sendStride, 0, a.count, true, false, gtid, gstride);
    } else if (me == a.root) {
      zcReduceRange<TIn, TOut>(dc, a, z, 0, 0, a.count, true, false, gtid, gstride);
    }
    zcFenceBeforeClose();
    ctaBarrier(dc, cta, barrierValue(seq, 2), seq);
  }
  epilogue(dc, seq, nctas);
}

// ---------------------------------------------------------------- byte-moving kinds

// One read of `src`, one store into each of dst[0..nd): used where a rank sends the same bytes to several
// peers, so that local memory is read once whatever the number of peers.
__device__ __forceinline__ void zcCopyMulti(char *const *dst, int nd, const char *src, size_t bytes, size_t gtid, size_t gstride) {
  if (!bytes || !nd) return;
  bool al = aligned16(src);
  for (int k = 0; k < nd; k++) al = al && aligned16(dst[k]);
  if (!al) {
    for (int k = 0; k < nd; k++) copyUnits(dst[k], src, bytes, 16, gtid, gstride);
    return;
  }
  const size_t nfull = bytes / 16;
  size_t u = gtid;
  for (; u + 3 * gstride < nfull; u += 4 * gstride) {
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = ld16(src + (u + i * gstride) * 16);
    for (int k = 0; k < nd; k++) {
#pragma unroll
      for (int i = 0; i < 4; i++) st16(dst[k] + (u + i * gstride) * 16, v[i]);
    }
  }
  for (; u < nfull; u += gstride) {
    const uint4 v = ld16(src + u * 16);
    for (int k = 0; k < nd; k++) st16(dst[k] + u * 16, v);
  }
  const size_t tail = bytes - nfull * 16;
  if (tail && gtid == 0)
    for (int k = 0; k < nd; k++)
      for (size_t i = 0; i < tail; i++) dst[k][nfull * 16 + i] = src[nfull * 16 + i];
}

// Store the 16-byte units of `src` through the multicast alias (every rank of the communicator receives
// them, this one included).  Returns the number of bytes covered; the ragged rest is left to plain stores.
__device__ __forceinline__ size_t zcMcPush(char *mcDst, const char *src, size_t bytes, size_t gtid, size_t gstride) {
  if (!aligned16(src) || !aligned16(mcDst)) return 0;
  const size_t nfull = bytes / 16;
  size_t u = gtid;
  for (; u + 3 * gstride < nfull; u += 4 * gstride) {
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; i++) v[i] = ld16(src + (u + i * gstride) * 16);
#pragma unroll
    for (int i = 0; i < 4; i++) mmStore(mcDst + (u + i * gstride) * 16, v[i]);
  }
  for (; u < nfull; u += gstride) mmStore(mcDst + u * 16, ld16(src + u * 16));
  return nfull * 16;
}

__device__ void fcxZcMoveBody(const FcxDevComm &dc, const FcxCollArgs &a, int cta, int nctas) {
  const int n = dc.nranks, me = dc.rank;
  const uint64_t seq = nextSeq(dc);
  const size_t gtid = (size_t)cta * blockDim.x + threadIdx.x, gstride = (size_t)nctas * blockDim.x;
  const size_t es = a.elemSize, bytes = a.count * es;
  const int mk = a.moveOp;
  if (!prologue(dc, seq, cta)) return;
  const bool pull = mk == FCX_K_GATHER || mk == FCX_K_A2AV;
  size_t sendSpan = 0, recvSpan = 0;
  uint64_t xTo[FCX_MAX_RANKS], yTo[FCX_MAX_RANKS];
  for (int p = 0; p < n; p++) { xTo[p] = 0; yTo[p] = 0; }
  switch (mk) {
    case FCX_K_AG:
    case FCX_K_A2A: recvSpan = ((size_t)(n - 1) * a.recvStride + a.count) * es; break;
    case FCX_K_BCAST:
    case FCX_K_SCATTER: recvSpan = bytes; break;
    case FCX_K_GATHER: sendSpan = bytes; break;
    case FCX_K_A2AV:
      for (int p = 0; p < n; p++) {
        xTo[p] = a.sdispls[p] * es;
        yTo[p] = a.scounts[p] * es;
      }
      break;
    default: break;
  }
  ZcPeers z;
  if (a.ceOpen) {
    // Opening step of the copy-engine form: after this barrier every peer's receive buffer may be written;
    // the host's copies assume one heap offset on all ranks, which is checked here (a mismatch is recorded as a
    // bad argument; the copies then land at this rank's offset inside the peers' heaps, never outside them).
    if (zcExchange(dc, a, seq, cta, false, true, 0, recvSpan, nullptr, nullptr, &z)) {
      bool same = true;
      for (int p = 0; p < n; p++) same = same && (p == me || z.recv[p] == dc.heap[p] + a.recvHeapOff);
      if (!same && threadIdx.x == 0) giveUp(dc, FCX_ERR_BADARG, me, FCX_WAIT_BARRIER, cta, a.recvHeapOff, 0, seq);
    }
    epilogue(dc, seq, nctas);
    return;
  }
  if (zcExchange(dc, a, seq, cta, pull, !pull, sendSpan, recvSpan, xTo, yTo, &z)) {
    const char *send = (const char *)a.send;
    char *recv = (char *)a.recv;
    char *dst[FCX_MAX_RANKS];
    int nd = 0;
    switch (mk) {
      case FCX_K_AG: {
        const size_t off = (size_t)me * a.recvStride * es;
        size_t done = 0;
        if (z.mcRecv && (a.useMc & 2)) done = zcMcPush(z.mcRecv + off, send, bytes, gtid, gstride);
        // a multicast store reaches this rank too, so everybody, this rank included, still needs [done, bytes)
        if (recv + off != send) dst[nd++] = recv + off;
        for (int k = 1; k < n; k++) dst[nd++] = z.recv[(me + k) % n] + off;
        if (done < bytes) {
          char *d2[FCX_MAX_RANKS];
          for (int k = 0; k < nd; k++) d2[k] = dst[k] + done;
          zcCopyMulti(d2, nd, send + done, bytes - done, gtid, gstride);
        }
        break;
      }
      case FCX_K_BCAST: {
        if (me != a.root) break;
        size_t done = 0;
        if (z.mcRecv) done = zcMcPush(z.mcRecv, send, bytes, gtid, gstride);
        if (recv != send) dst[nd++] = recv;
        for (int k = 1; k < n; k++) dst[nd++] = z.recv[(me + k) % n];
        if (done < bytes) {
          char *d2[FCX_MAX_RANKS];
          for (int k = 0; k < nd; k++) d2[k] = dst[k] + done;
          zcCopyMulti(d2, nd, send + done, bytes - done, gtid, gstride);
        }
        break;
      }
      case FCX_K_SCATTER: {
        if (me != a.root) break;
        for (int k = 0; k < n; k++) {
          const int p = (me + k) % n;
          const char *s = send + (size_t)p * a.sendStride * es;
          char *d = p == me ? recv : z.recv[p];
          if (d != s) copyUnits(d, s, bytes, 16, gtid, gstride);
        }
        break;
      }
      case FCX_K_A2A: {
        for (int k = 0; k < n; k++) {
          const int p = (me + k) % n;
          const char *s = send + (size_t)p * a.sendStride * es;
          char *d = (p == me ? recv : z.recv[p]) + (size_t)me * a.recvStride * es;
          if (d != s) copyUnits(d, s, bytes, 16, gtid, gstride);
        }
        break;
      }
      case FCX_K_GATHER: {
        if (me != a.root) break;
        for (int k = 0; k < n; k++) {
          const int p = (me + k) % n;
          const char *s = p == me ? send : z.send[p];
          char *d = recv + (size_t)p * a.recvStride * es;
          if (d != s) copyUnits(d, s, bytes, 16, gtid, gstride);
        }
        break;
      }
      case FCX_K_A2AV: {
        for (int k = 0; k < n; k++) {
          const int p = (me + k) % n;
          const char *s = (p == me ? send : z.send[p]) + z.x[p];
          const size_t nb = min((size_t)z.y[p], (size_t)(a.rcounts[p] * es));
          char *d = recv + a.rdispls[p] * es;
          if (nb && d != s) copyUnits(d, s, nb, 16, gtid, gstride);
        }
        break;
      }
      default: break;
    }
    zcFenceBeforeClose();
    ctaBarrier(dc, cta, barrierValue(seq, 2), seq);
  }
  epilogue(dc, seq, nctas);
}

}  // namespace fcxdev
