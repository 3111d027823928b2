// The collective kernels.
//
// One templated body, fcxCollBody<TIn,TOut>, implements every collective as a
// sequence of at most three phases separated by cross-GPU CTA barriers.  The
// data path is "push": a rank stores its contribution straight into the
// staging area of the peer that needs it (NVLink stores from the SMs), the
// barrier publishes it, and the receiver combines or copies it out of its own
// HBM.  The NVLS kinds replace the push by multimem.ld_reduce / multimem.st on
// the NVSwitch multicast alias of the heaps.  In the reference these
// operations are calls into the vendor library
// (flagcx/adaptor/ccl/nccl_adaptor.cc:92-256); nothing here calls it.
//
// Work is cut into "units" of G elements (16 bytes of the narrower of the two
// element types).  Unit u of any buffer is always handled by the same thread
// of the same CTA index on every rank and in every phase, which is what lets a
// per-CTA barrier (instead of a grid-wide one) order the phases.
//
// The body takes the CTA index and CTA count as arguments so that the very
// same code can run as one real rank per GPU (fcxCollKernel) or as several
// emulated ranks inside one cooperative launch on a single GPU
// (fcxCollEmuKernel), which is how the protocol is tested without NVLink.
#include "prims.cuh"
#include "launch.h"
#include "dispatch.h"

#include <cuda_runtime.h>

namespace fcxdev {

__device__ __forceinline__ char *stagePtr(const FcxDevComm &dc, int r, uint64_t seq) {
  return dc.heap[r] + FCX_OFF_STAGE + (size_t)(seq & 1) * dc.stageBytes;
}

__device__ __forceinline__ void copyToSlot(char *slot, const char *user, size_t bytes, int unitBytes, size_t gtid,
                                           size_t gstride) {
  copyUnits(slot, user, bytes, unitBytes, gtid, gstride);
}
__device__ __forceinline__ void copyFromSlot(char *user, const char *slot, size_t bytes, int unitBytes, size_t gtid,
                                             size_t gstride) {
  copyUnits(user, slot, bytes, unitBytes, gtid, gstride);
}


// ---------------------------------------------------------------- software pipeline over sub-chunks
//
// Large messages are cut into sub-chunks so that the phases of a collective overlap: while sub-chunk i is
// pushed over NVLink, sub-chunk i-1 is reduced or copied out of local memory (and i-2 copied out, for the
// three-phase kinds).  One cross-GPU CTA barrier per iteration orders phase k of a sub-chunk before phase
// k+1 of the same sub-chunk.  Sixteen CTAs saturate a direction of NVLink; the rest of the grid hides the
// local traffic behind it.
__device__ __forceinline__ size_t subLen(size_t total, size_t sub, int c, size_t *lo) {
  *lo = (size_t)c * sub;
  return *lo < total ? min(sub, total - *lo) : 0;
}
__device__ __forceinline__ size_t pipeBytesOf(const FcxDevComm &dc) { return dc.pipeBytes ? (size_t)dc.pipeBytes : ((size_t)16 << 20); }

// The barrier between iterations is split: a CTA posts "iteration i done" to its peers at the end of the
// iteration and only checks the peers' post after it has issued the next sub-chunk's pushes, so the link
// never idles while flags travel, and the release that precedes a post finds the pushes long acknowledged
// (the local phases run in between).
__device__ __forceinline__ void postPeers(const FcxDevComm &dc, int cta, uint64_t value, bool selfToo = false) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < dc.nranks && (t != dc.rank || selfToo)) stRelease(flagSlot(dc, t, cta, dc.rank), value);
}
__device__ __forceinline__ bool waitPeers(const FcxDevComm &dc, int cta, uint64_t value, uint64_t seq) {
  bool ok = true;
  const int t = threadIdx.x;
  if (t < dc.nranks && t != dc.rank) ok = waitGe(dc, flagSlot(dc, dc.rank, cta, t), value, t, FCX_WAIT_BARRIER, cta, seq);
  return __syncthreads_and(ok);
}

// ---- role split -----------------------------------------------------------------------------------------
// With two or more CTAs the grid is split into "link" CTAs, which only stream sub-chunks to the peers (each
// one a contiguous share, back to back, never waiting for anybody), and "local" CTAs, which copy, reduce and
// copy out inside this GPU as the sub-chunks arrive.  A link CTA raises its own flag on every peer after
// each sub-chunk; a consumer waits for the flags of all link CTAs of the ranks it expects data from.  The
// link therefore stays busy from the first to the last byte while local memory traffic runs beside it.
__device__ __forceinline__ int linkCtasOf(int nctas) { return nctas < 2 ? 0 : (nctas < 8 ? 1 : min(32, nctas / 4)); }

// Contiguous share of [0, len) for worker x of L, in multiples of `unit` bytes.
__device__ __forceinline__ size_t shareOf(size_t len, int x, int L, size_t unit, size_t *lo) {
  const size_t units = (len + unit - 1) / unit, per = (units + L - 1) / L;
  *lo = min(len, (size_t)x * per * unit);
  return min(len - *lo, per * unit);
}

// All threads of the CTA.  Wait until CTAs [first, first+count) of every rank in `srcMask` have posted `value`.
__device__ __forceinline__ bool waitChunk(const FcxDevComm &dc, int cta, int first, int count, unsigned srcMask, uint64_t value,
                                          uint64_t seq) {
  bool ok = true;
  const int n = dc.nranks;
  for (int t = threadIdx.x; t < count * n && ok; t += blockDim.x) {
    const int x = first + t / n, p = t % n;
    if ((srcMask >> p) & 1u) ok = waitGe(dc, flagSlot(dc, dc.rank, x, p), value, p, FCX_WAIT_BARRIER, cta, seq);
  }
  return __syncthreads_and(ok);
}

template <int DEPTH, class FA, class FB, class FC>
__device__ __forceinline__ bool pipelined(const FcxDevComm &dc, int cta, uint64_t seq, int chunks, FA stageA, FB stageB, FC stageC) {
  const int iters = chunks + DEPTH - 1;
  for (int i = 0; i < iters; i++) {
    if (i < chunks) stageA(i);                                              // needs nothing from the peers
    if (i >= 1 && !waitPeers(dc, cta, barrierValue(seq, (unsigned)i), seq)) return false;  // peers finished iteration i-1
    if (i >= 1 && i - 1 < chunks) stageB(i - 1);
    if (DEPTH == 3 && i >= 2 && i - 2 < chunks) stageC(i - 2);
    if (i + 1 < iters) postPeers(dc, cta, barrierValue(seq, 1 + (unsigned)i));
  }
  return true;
}

// ---------------------------------------------------------------- LL one-shot all-reduce

// A 16-byte LL line carries 8 payload bytes and two copies of the 32-bit
// sequence tag: {d0, tag, d1, tag}.  Each 8-byte half is written atomically,
// so a reader that sees the tag in a half also sees that half's payload.
__device__ __forceinline__ void llStore(char *line, uint32_t d0, uint32_t d1, uint32_t tag) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(line), "r"(d0), "r"(tag), "r"(d1), "r"(tag)
               : "memory");
}
__device__ __forceinline__ uint4 llLoad(const char *line) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(line) : "memory");
  return v;
}

// mode 0: all-reduce (everybody sends its whole vector to everybody and reduces);
// mode 1: reduce-scatter (piece p goes to rank p, every rank reduces the pieces it received and its own);
// mode 2: reduce (everybody sends its whole vector to the root, which reduces).
template <typename T>
__device__ void arLL(const FcxDevComm &dc, const FcxCollArgs &a, uint64_t seq, int cta, int nctas, int mode = 0) {
  using Acc = typename Elem<T>::Acc;
  constexpr int G = 16 / (int)sizeof(T);
  const int n = dc.nranks, me = dc.rank;
  const uint32_t tag = (uint32_t)seq;
  const size_t gtid = (size_t)cta * blockDim.x + threadIdx.x, gstride = (size_t)nctas * blockDim.x;
  const size_t nunits = (a.count + G - 1) / G;
  const size_t pieceBytes = mode == 1 ? a.sendStride * sizeof(T) : 0;  // distance between the pieces of a reduce-scatter
  const char *send = (const char *)a.send + (size_t)me * pieceBytes;    // what this rank contributes to its own result
  const bool reduces = mode != 2 || me == a.root;
  const bool alS = aligned16(send), alR = aligned16(a.recv);
  const size_t llOff = FCX_OFF_LL + (size_t)(seq & 1) * FCX_MAX_RANKS * FCX_LL_SLOT_BYTES;
  bool ok = true;
  for (size_t u = gtid; u < nunits; u += gstride) {
    int nv = (int)min((size_t)G, a.count - u * G);
    Acc mine[G];
    loadUnit<T, G>(send + u * 16, alS, nv, mine);
    for (int k = 1; k < n; k++) {
      int p = (me + k) % n;
      if (mode == 2 && p != a.root) continue;
      uint4 raw;
      if (mode == 1) {
        const char *src = (const char *)a.send + (size_t)p * pieceBytes + u * 16;
        Acc theirs[G];
        loadUnit<T, G>(src, aligned16(src), nv, theirs);
        packUnit<T, G>(theirs, &raw);
      } else {
        packUnit<T, G>(mine, &raw);
      }
      char *line = dc.heap[p] + llOff + (size_t)me * FCX_LL_SLOT_BYTES + u * 32;
      llStore(line, raw.x, raw.y, tag);
      llStore(line + 16, raw.z, raw.w, tag);
    }
    if (!reduces) continue;
    Acc acc[G];
    bool first = true;
    for (int p = 0; p < n; p++) {
      Acc in[G];
      if (p == me) {
#pragma unroll
        for (int i = 0; i < G; i++) in[i] = mine[i];
      } else {
        const char *line = dc.heap[me] + llOff + (size_t)p * FCX_LL_SLOT_BYTES + u * 32;
        uint4 lo = llLoad(line), hi = llLoad(line + 16);
        if (!(lo.y == tag && lo.w == tag && hi.y == tag && hi.w == tag)) {
          uint64_t t0 = globalTimerNs();
          unsigned spins = 0;
          for (;;) {
            lo = llLoad(line);
            hi = llLoad(line + 16);
            if (lo.y == tag && lo.w == tag && hi.y == tag && hi.w == tag) break;
            if ((++spins & 63u) == 0u) {
              if (*(volatile unsigned int *)&localOf(dc)->abortSeen) { ok = false; break; }
              if (globalTimerNs() - t0 > dc.timeoutNs) {
                giveUp(dc, FCX_ERR_TIMEOUT, p, FCX_WAIT_LL, cta, tag, lo.y, seq);
                ok = false;
                break;
              }
              if ((spins & 1023u) == 0u && *dc.abortWord) {
                giveUp(dc, FCX_ERR_ABORT, p, FCX_WAIT_LL, cta, tag, lo.y, seq);
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
        }
        union { uint4 v; T t[G]; } w;
        w.v = make_uint4(lo.x, lo.z, hi.x, hi.z);
#pragma unroll
        for (int i = 0; i < G; i++) in[i] = Elem<T>::up(w.t[i]);
      }
      if (first) {
#pragma unroll
        for (int i = 0; i < G; i++) acc[i] = in[i];
        first = false;
      } else {
#pragma unroll
        for (int i = 0; i < G; i++) acc[i] = applyOp<Acc>(acc[i], in[i], a.redop);
      }
    }
    if (!ok) break;
#pragma unroll
    for (int i = 0; i < G; i++) acc[i] = finish<Acc>(acc[i], a.redop, n, a.scale);
    uint4 outv;
    packUnit<T, G>(acc, &outv);
    storeUnit<T, G>((char *)a.recv + u * 16, alR, nv, &outv);
  }
}

// ---------------------------------------------------------------- reductions out of staging

// out[u] = finish( x_0[u] (op) x_1[u] ... x_{n-1}[u] ) over the ranks in rank
// order, where x_own comes from `own` (user memory) and the others from the
// local staging slots.  The result unit goes to `dstUser` (user memory, may
// be null) and, as a full 16-byte-multiple unit, to every pointer in dstSlots.
template <typename TIn, typename TOut, int G>
__device__ __forceinline__ void reduceUnits(const FcxDevComm &dc, const FcxCollArgs &a, const char *own, bool ownAligned,
                                            const char *slotBase, size_t slotStride, size_t nElems, char *dstUser,
                                            bool dstAligned, char *const *dstSlots, int nDstSlots, size_t gtid,
                                            size_t gstride) {
  using AI = typename Elem<TIn>::Acc;
  using AO = typename Elem<TOut>::Acc;
  constexpr int INB = G * (int)sizeof(TIn), OUTB = G * (int)sizeof(TOut);
  const int n = dc.nranks, me = dc.rank;
  const size_t nunits = (nElems + G - 1) / G;
  // all loads of a unit, combined in rank order (no stores in here, so the
  // compiler may overlap the loads of two units)
  auto gather = [&](size_t u, AI *acc) {
    int nv = (int)min((size_t)G, nElems - u * G);
    for (int p = 0; p < n; p++) {
      AI in[G];
      if (p == me) loadUnit<TIn, G>(own + u * INB, ownAligned, nv, in);
      else loadUnit<TIn, G>(slotBase + (size_t)p * slotStride + u * INB, true, G, in);
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
    int nv = (int)min((size_t)G, nElems - u * G);
    AO res[G];
#pragma unroll
    for (int i = 0; i < G; i++) res[i] = accCast<AO, AI>(finish<AI>(acc[i], a.redop, n, a.scale));
    uint4 packed[OUTB / 16];
    packUnit<TOut, G>(res, packed);
    if (dstUser) storeUnit<TOut, G>(dstUser + u * OUTB, dstAligned, nv, packed);
    for (int k = 0; k < nDstSlots; k++) storeUnit<TOut, G>(dstSlots[k] + u * OUTB, true, G, packed);
  };
  size_t u = gtid;
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

// ---------------------------------------------------------------- the body

template <typename TIn, typename TOut>
__device__ void fcxCollBody(const FcxDevComm &dc, const FcxCollArgs &a, int cta, int nctas) {
  constexpr int ESI = (int)sizeof(TIn), ESO = (int)sizeof(TOut);
  constexpr int G = 16 / (ESI < ESO ? ESI : ESO);
  constexpr int INB = G * ESI, OUTB = G * ESO;
  const int n = dc.nranks, me = dc.rank;
  const uint64_t seq = nextSeq(dc);
  const size_t gtid = (size_t)cta * blockDim.x + threadIdx.x, gstride = (size_t)nctas * blockDim.x;

  if (!prologue(dc, seq, cta)) return;

  const char *send = (const char *)a.send;
  char *recv = (char *)a.recv;

  // Bounds of the staging area: the host cuts a message so that one launch fits, and the kernel checks it
  // again, because a launch that does not fit would write into the other parity's half or past the heap.
  {
    size_t need = 0;
    const size_t units = (a.count + G - 1) / G, sliceUnits = (units + n - 1) / n;
    switch (a.kind) {
      case FCX_K_AR_ONESHOT:
      case FCX_K_RS: need = (size_t)n * units * INB; break;
      case FCX_K_AR_TWOSHOT:
      case FCX_K_REDUCE: need = (size_t)n * sliceUnits * (INB + OUTB); break;
      case FCX_K_AR_NVLS: need = (size_t)n * sliceUnits * 16; break;
      case FCX_K_RS_NVLS: need = (size_t)n * ((a.count * ESI + 15) / 16 * 16); break;
      case FCX_K_AR_LL: case FCX_K_REDUCE_LL: need = a.count * ESI > FCX_LL_MAX_PAYLOAD ? ~(size_t)0 : 0; break;
      case FCX_K_RS_LL: need = a.count * ESI > FCX_LL_MAX_PAYLOAD ? ~(size_t)0 : 0; break;
      default: break;
    }
    if (need > dc.stageBytes) {
      if (threadIdx.x == 0) giveUp(dc, FCX_ERR_BADARG, me, FCX_WAIT_BARRIER, cta, dc.stageBytes, need, seq);
      epilogue(dc, seq, nctas);
      return;
    }
  }

  switch (a.kind) {
    case FCX_K_BARRIER: {
      if (cta == 0) ctaBarrier(dc, 0, barrierValue(seq, 1), seq);
      break;
    }

    case FCX_K_AR_LL: {
      if constexpr (ESI == ESO) arLL<TIn>(dc, a, seq, cta, nctas);
      break;
    }
    case FCX_K_RS_LL: {
      if constexpr (ESI == ESO) arLL<TIn>(dc, a, seq, cta, nctas, 1);
      break;
    }
    case FCX_K_REDUCE_LL: {
      if constexpr (ESI == ESO) arLL<TIn>(dc, a, seq, cta, nctas, 2);
      break;
    }

    case FCX_K_AR_ONESHOT: {
      // every rank receives every other rank's whole vector
      const size_t bytes = a.count * ESI;
      const size_t slot = (bytes + INB - 1) / INB * INB;
      for (int k = 1; k < n; k++) {
        int p = (me + k) % n;
        copyToSlot(stagePtr(dc, p, seq) + (size_t)me * slot, send, bytes, INB, gtid, gstride);
      }
      if (!ctaBarrier(dc, cta, barrierValue(seq, 1), seq)) break;
      reduceUnits<TIn, TOut, G>(dc, a, send, aligned16(send), stagePtr(dc, me, seq), slot, a.count, recv,
                                aligned16(recv), nullptr, 0, gtid, gstride);
      break;
    }

    case FCX_K_AR_TWOSHOT:
    case FCX_K_REDUCE: {
      const bool toRootOnly = a.kind == FCX_K_REDUCE;
      const size_t totalUnits = (a.count + G - 1) / G;
      const size_t sliceUnits = (totalUnits + n - 1) / n;
      const size_t sliceElems = sliceUnits * G;
      const size_t slotA = sliceUnits * INB, slotB = sliceUnits * OUTB;
      auto elemsOf = [&](int p) -> size_t {
        size_t lo = (size_t)p * sliceElems;
        return lo >= a.count ? 0 : min(sliceElems, a.count - lo);
      };
      // sub-chunks of every slice, in units
      const size_t cu = max((size_t)1024, pipeBytesOf(dc) / (size_t)max(1, n - 1) / 16);
      const int chunks = (int)max((size_t)1, (sliceUnits + cu - 1) / cu);
      auto rangeOf = [&](int p, int c, size_t *loU) -> size_t {  // elements of slice p that fall into sub-chunk c
        *loU = (size_t)c * cu;
        size_t ne = elemsOf(p), lo = *loU * G;
        return lo >= ne ? 0 : min(cu * G, ne - lo);
      };
      // phase 1: slice p of my vector goes to rank p (units [uLo, uLo+uCnt) of sub-chunk c, relative to the sub-chunk)
      auto pushW = [&](int c, size_t tid0, size_t stride, int x, int L) {
        for (int k = 1; k < n; k++) {
          int p = (me + k) % n;
          size_t loU, ne = rangeOf(p, c, &loU);
          if (!ne) continue;
          size_t slo, slen = shareOf(ne * ESI, x, L, INB, &slo);  // bytes of this worker's share
          if (slen)
            copyToSlot(stagePtr(dc, p, seq) + (size_t)me * slotA + loU * INB + slo,
                       send + ((size_t)p * sliceElems + loU * G) * ESI + slo, slen, INB, tid0, stride);
        }
      };
      // phase 2: combine my slice, hand the result to whoever needs it
      auto combineW = [&](int c, size_t tid0, size_t stride) {
        size_t loU, ne = rangeOf(me, c, &loU);
        if (!ne) return;
        char *dstSlots[FCX_MAX_RANKS];
        int nd = 0;
        char *dstUser = nullptr;
        if (toRootOnly) {
          if (me == a.root) dstUser = recv + ((size_t)me * sliceElems + loU * G) * ESO;
          else dstSlots[nd++] = stagePtr(dc, a.root, seq) + (size_t)n * slotA + (size_t)me * slotB + loU * OUTB;
        } else {
          dstUser = recv + ((size_t)me * sliceElems + loU * G) * ESO;
          for (int k = 1; k < n; k++) {
            int p = (me + k) % n;
            dstSlots[nd++] = stagePtr(dc, p, seq) + (size_t)n * slotA + (size_t)me * slotB + loU * OUTB;
          }
        }
        const char *own = send + ((size_t)me * sliceElems + loU * G) * ESI;
        reduceUnits<TIn, TOut, G>(dc, a, own, aligned16(own), stagePtr(dc, me, seq) + loU * INB, slotA, ne, dstUser,
                                  dstUser && aligned16(dstUser), dstSlots, nd, tid0, stride);
      };
      // phase 3: collect the other ranks' finished slices
      auto collectW = [&](int c, size_t tid0, size_t stride) {
        if (toRootOnly && me != a.root) return;
        for (int k = 1; k < n; k++) {
          int p = (me + k) % n;
          size_t loU, ne = rangeOf(p, c, &loU);
          if (ne)
            copyFromSlot(recv + ((size_t)p * sliceElems + loU * G) * ESO,
                         stagePtr(dc, me, seq) + (size_t)n * slotA + (size_t)p * slotB + loU * OUTB, ne * ESO, OUTB, tid0, stride);
        }
      };
      const int L = linkCtasOf(nctas);
      if (L > 0) {
        const unsigned all = ((1u << n) - 1u) & ~(1u << me);
        if (cta < L) {
          for (int c = 0; c < chunks; c++) {
            pushW(c, threadIdx.x, blockDim.x, cta, L);
            postPeers(dc, cta, barrierValue(seq, 1 + (unsigned)c));
          }
        } else {
          const int NL = nctas - L;
          const size_t tid0 = (size_t)(cta - L) * blockDim.x + threadIdx.x, stride = (size_t)NL * blockDim.x;
          // results travel to: everybody (all-reduce) or the root (reduce)
          const bool collects = !toRootOnly || me == a.root;
          bool ok = true;
          for (int c = 0; c < chunks && ok; c++) {
            ok = waitChunk(dc, cta, 0, L, all, barrierValue(seq, 1 + (unsigned)c), seq);
            if (!ok) break;
            combineW(c, tid0, stride);
            postPeers(dc, cta, barrierValue(seq, 1 + (unsigned)c));
            if (c >= 1 && collects) {
              ok = waitChunk(dc, cta, L, NL, all, barrierValue(seq, (unsigned)c), seq);
              if (ok) collectW(c - 1, tid0, stride);
            }
          }
          if (ok && collects && waitChunk(dc, cta, L, NL, all, barrierValue(seq, (unsigned)chunks), seq)) collectW(chunks - 1, tid0, stride);
        }
        break;
      }
      auto push = [&](int c) { pushW(c, gtid, gstride, 0, 1); };
      auto combine = [&](int c) { combineW(c, gtid, gstride); };
      auto collect = [&](int c) { collectW(c, gtid, gstride); };
      pipelined<3>(dc, cta, seq, chunks, push, combine, collect);
      break;
    }

    case FCX_K_AR_NVLS:
    case FCX_K_RS_NVLS: {
      if constexpr (ESI == ESO && Mm<TIn>::ok) {
        // copy in (local), switch-reduce my slice, multicast it back (all-reduce)
        // or keep it (reduce-scatter), copy out (local).  Copies are indexed
        // relative to the slice so that the unit-ownership rule holds between
        // the rank that wrote a line and the rank that reads it through the switch.
        const bool isRS = a.kind == FCX_K_RS_NVLS;
        size_t sliceElems, sliceBytes;
        if (isRS) {
          sliceElems = a.count;
          sliceBytes = (a.count * ESI + 15) / 16 * 16;
        } else {
          size_t totalUnits = (a.count + G - 1) / G;
          size_t sliceUnits = (totalUnits + n - 1) / n;
          sliceElems = sliceUnits * G;
          sliceBytes = sliceUnits * 16;
        }
        auto elemsOf = [&](int p) -> size_t {
          if (isRS) return a.count;
          size_t lo = (size_t)p * sliceElems;
          return lo >= a.count ? 0 : min(sliceElems, a.count - lo);
        };
        const size_t srcStride = isRS ? a.sendStride : sliceElems;
        const size_t cu = max((size_t)1024, pipeBytesOf(dc) / (size_t)max(1, n - 1) / 16);  // units of a slice per sub-chunk
        const int chunks = (int)max((size_t)1, (sliceBytes / 16 + cu - 1) / cu);
        auto rangeOf = [&](int p, int c, size_t *loU) -> size_t {
          *loU = (size_t)c * cu;
          size_t ne = elemsOf(p), lo = *loU * G;
          return lo >= ne ? 0 : min(cu * G, ne - lo);
        };
        const size_t stageOff = FCX_OFF_STAGE + (size_t)(seq & 1) * dc.stageBytes;
        char *mcSlice = dc.mcHeap + stageOff + (size_t)me * sliceBytes;
        const bool alR = aligned16(recv);
        auto copyIn = [&](int c) {
          for (int p = 0; p < n; p++) {
            size_t loU, ne = rangeOf(p, c, &loU);
            if (ne)
              copyToSlot(stagePtr(dc, me, seq) + (size_t)p * sliceBytes + loU * 16, send + ((size_t)p * srcStride + loU * G) * ESI, ne * ESI,
                         16, gtid, gstride);
          }
        };
        auto reduce = [&](int c) {
          size_t loU, ne = rangeOf(me, c, &loU);
          if (!ne) return;
          const size_t myUnits = (ne + G - 1) / G;
          char *mcp = mcSlice + loU * 16;
          if (isRS) {
            char *out = recv + loU * 16;
            size_t u = gtid;
            for (; u + 3 * gstride < myUnits; u += 4 * gstride) {
              uint4 r[4];
#pragma unroll
              for (int i = 0; i < 4; i++) r[i] = Mm<TIn>::ldReduce(mcp + (u + i * gstride) * 16, a.redop);
#pragma unroll
              for (int i = 0; i < 4; i++) {
                size_t uu = u + i * gstride;
                uint4 f = mmFinish<TIn>(r[i], a.redop, n, a.scale);
                storeUnit<TIn, G>(out + uu * 16, alR, (int)min((size_t)G, ne - uu * G), &f);
              }
            }
            for (; u < myUnits; u += gstride) {
              uint4 f = mmFinish<TIn>(Mm<TIn>::ldReduce(mcp + u * 16, a.redop), a.redop, n, a.scale);
              storeUnit<TIn, G>(out + u * 16, alR, (int)min((size_t)G, ne - u * G), &f);
            }
            return;
          }
          size_t u = gtid;
          for (; u + 3 * gstride < myUnits; u += 4 * gstride) {
            uint4 r[4];
#pragma unroll
            for (int i = 0; i < 4; i++) r[i] = Mm<TIn>::ldReduce(mcp + (u + i * gstride) * 16, a.redop);
#pragma unroll
            for (int i = 0; i < 4; i++) mmStore(mcp + (u + i * gstride) * 16, mmFinish<TIn>(r[i], a.redop, n, a.scale));
          }
          for (; u < myUnits; u += gstride)
            mmStore(mcp + u * 16, mmFinish<TIn>(Mm<TIn>::ldReduce(mcp + u * 16, a.redop), a.redop, n, a.scale));
        };
        auto copyOut = [&](int c) {
          for (int p = 0; p < n; p++) {
            size_t loU, ne = rangeOf(p, c, &loU);
            if (ne)
              copyFromSlot(recv + ((size_t)p * sliceElems + loU * G) * ESI, stagePtr(dc, me, seq) + (size_t)p * sliceBytes + loU * 16,
                           ne * ESI, 16, gtid, gstride);
          }
        };
        if (isRS) pipelined<2>(dc, cta, seq, chunks, copyIn, reduce, copyOut);
        else pipelined<3>(dc, cta, seq, chunks, copyIn, reduce, copyOut);
      }
      break;
    }

    case FCX_K_RS: {
      const size_t bytes = a.count * ESI;
      const size_t slot = (bytes + INB - 1) / INB * INB;
      const size_t units = (a.count + G - 1) / G;
      const size_t cu = max((size_t)1024, pipeBytesOf(dc) / (size_t)max(1, n - 1) / INB);
      const int chunks = (int)max((size_t)1, (units + cu - 1) / cu);
      auto rangeOf = [&](int c, size_t *loU) -> size_t {
        *loU = (size_t)c * cu;
        size_t lo = *loU * G;
        return lo >= a.count ? 0 : min(cu * G, a.count - lo);
      };
      auto pushW = [&](int c, size_t tid0, size_t stride, int x, int L) {
        size_t loU, ne = rangeOf(c, &loU);
        if (!ne) return;
        size_t slo, slen = shareOf(ne * ESI, x, L, INB, &slo);
        if (!slen) return;
        for (int k = 1; k < n; k++) {
          int p = (me + k) % n;
          copyToSlot(stagePtr(dc, p, seq) + (size_t)me * slot + loU * INB + slo, send + ((size_t)p * a.sendStride + loU * G) * ESI + slo, slen,
                     INB, tid0, stride);
        }
      };
      auto combineW = [&](int c, size_t tid0, size_t stride) {
        size_t loU, ne = rangeOf(c, &loU);
        if (!ne) return;
        const char *own = send + ((size_t)me * a.sendStride + loU * G) * ESI;
        char *out = recv + loU * G * ESO;
        reduceUnits<TIn, TOut, G>(dc, a, own, aligned16(own), stagePtr(dc, me, seq) + loU * INB, slot, ne, out, aligned16(out), nullptr, 0,
                                  tid0, stride);
      };
      const int L = linkCtasOf(nctas);
      if (L > 0) {
        if (cta < L) {
          for (int c = 0; c < chunks; c++) {
            pushW(c, threadIdx.x, blockDim.x, cta, L);
            postPeers(dc, cta, barrierValue(seq, 1 + (unsigned)c));
          }
        } else {
          const size_t tid0 = (size_t)(cta - L) * blockDim.x + threadIdx.x, stride = (size_t)(nctas - L) * blockDim.x;
          for (int c = 0; c < chunks; c++) {
            if (!waitChunk(dc, cta, 0, L, ((1u << n) - 1u) & ~(1u << me), barrierValue(seq, 1 + (unsigned)c), seq)) break;
            combineW(c, tid0, stride);
          }
        }
        break;
      }
      auto push = [&](int c) { pushW(c, gtid, gstride, 0, 1); };
      auto combine = [&](int c) { combineW(c, gtid, gstride); };
      pipelined<2>(dc, cta, seq, chunks, push, combine, combine);
      break;
    }

    default:
      break;
  }

  epilogue(dc, seq, nctas);
}

// ---------------------------------------------------------------- LL byte mover
//
// Small fixed-size exchanges without any barrier: every 8 payload bytes travel in one 16-byte line
// {lo, tag, hi, tag} whose halves are written atomically, so a reader that sees the tag in both halves
// has the payload.  The tag is the collective's sequence number; the slots are parity double-buffered
// like the staging area.  One line slot per source rank on every receiver (FCX_LL_SLOT_BYTES each).
__device__ __forceinline__ void ld8(const char *p, size_t valid, uint32_t *lo, uint32_t *hi) {
  if (valid >= 8 && ((uintptr_t)p & 7u) == 0) {
    uint2 v = *(const uint2 *)p;
    *lo = v.x;
    *hi = v.y;
  } else {
    union { uint2 v; char c[8]; } w;
    w.v = make_uint2(0, 0);
    for (size_t i = 0; i < valid && i < 8; i++) w.c[i] = p[i];
    *lo = w.v.x;
    *hi = w.v.y;
  }
}
__device__ __forceinline__ void st8(char *p, size_t valid, uint32_t lo, uint32_t hi) {
  if (valid >= 8 && ((uintptr_t)p & 7u) == 0) {
    *(uint2 *)p = make_uint2(lo, hi);
  } else {
    union { uint2 v; char c[8]; } w;
    w.v = make_uint2(lo, hi);
    for (size_t i = 0; i < valid && i < 8; i++) p[i] = w.c[i];
  }
}
// Bounded wait for one line carrying `tag`; false = gave up.
__device__ __forceinline__ bool llWaitLine(const FcxDevComm &dc, const char *line, uint32_t tag, int peer, int cta, uint64_t seq,
                                           uint4 *out) {
  uint4 v = llLoad(line);
  if (v.y == tag && v.w == tag) { *out = v; return true; }
  const uint64_t t0 = globalTimerNs();
  unsigned spins = 0;
  for (;;) {
    v = llLoad(line);
    if (v.y == tag && v.w == tag) { *out = v; return true; }
    if ((++spins & 63u) == 0u) {
      if (*(volatile unsigned int *)&localOf(dc)->abortSeen) return false;
      if (globalTimerNs() - t0 > dc.timeoutNs) {
        giveUp(dc, FCX_ERR_TIMEOUT, peer, FCX_WAIT_LL, cta, tag, v.y, seq);
        return false;
      }
      if ((spins & 1023u) == 0u && *dc.abortWord) {
        giveUp(dc, FCX_ERR_ABORT, peer, FCX_WAIT_LL, cta, tag, v.y, seq);
        return false;
      }
    }
  }
}

// Byte-moving collectives need no element type.
__device__ void fcxMoveBody(const FcxDevComm &dc, const FcxCollArgs &a, int cta, int nctas) {
  const int n = dc.nranks, me = dc.rank;
  const uint64_t seq = nextSeq(dc);
  const size_t gtid = (size_t)cta * blockDim.x + threadIdx.x, gstride = (size_t)nctas * blockDim.x;
  const size_t es = a.elemSize;
  if (!prologue(dc, seq, cta)) return;
  const char *send = (const char *)a.send;
  char *recv = (char *)a.recv;
  const size_t bytes = a.count * es;
  const size_t slot = (bytes + 15) / 16 * 16;

  {  // the pieces of one launch must fit the staging half (or the LL slots) they travel through
    size_t need = 0;
    const int mk0 = a.kind == FCX_K_MOVE_LL ? a.moveOp : a.kind;
    if (a.kind == FCX_K_MOVE_LL) need = bytes > FCX_LL_MAX_PAYLOAD ? ~(size_t)0 : 0;
    else if (mk0 == FCX_K_BCAST || mk0 == FCX_K_SCATTER) need = slot;
    else if (a.kind != FCX_K_A2AV) need = (size_t)n * slot;
    if (need > dc.stageBytes) {
      if (threadIdx.x == 0) giveUp(dc, FCX_ERR_BADARG, me, FCX_WAIT_BARRIER, cta, dc.stageBytes, need, seq);
      epilogue(dc, seq, nctas);
      return;
    }
  }

  if (a.kind != FCX_K_A2AV) {
    const int mk = a.kind == FCX_K_MOVE_LL ? a.moveOp : a.kind;  // the LL form moves the same pieces
    // Every fixed-size byte mover is one exchange: piece out[p] goes into a slot of rank p's staging area,
    // piece in[p] arrives in a slot of this rank's staging area and is copied to its place, and the piece a
    // rank keeps for itself is copied locally.  With the multicast alias one store reaches every rank.
    const char *outSrc[FCX_MAX_RANKS];
    char *outDst[FCX_MAX_RANKS];
    const char *inSrc[FCX_MAX_RANKS];
    char *inDst[FCX_MAX_RANKS];
    for (int p = 0; p < n; p++) { outSrc[p] = nullptr; outDst[p] = nullptr; inSrc[p] = nullptr; inDst[p] = nullptr; }
    const char *selfSrc = nullptr, *mcSrc = nullptr;
    char *selfDst = nullptr, *mcDst = nullptr;
    const size_t stageOff = FCX_OFF_STAGE + (size_t)(seq & 1) * dc.stageBytes;
    char *myStage = stagePtr(dc, me, seq);
    switch (mk) {
      case FCX_K_AG:
      case FCX_K_AG_NVLS:
        for (int p = 0; p < n; p++)
          if (p != me) {
            if (mk == FCX_K_AG) { outSrc[p] = send; outDst[p] = stagePtr(dc, p, seq) + (size_t)me * slot; }
            inSrc[p] = myStage + (size_t)p * slot;
            inDst[p] = recv + (size_t)p * a.recvStride * es;
          }
        if (mk == FCX_K_AG_NVLS) { mcSrc = send; mcDst = dc.mcHeap + stageOff + (size_t)me * slot; }
        selfSrc = send;
        selfDst = recv + (size_t)me * a.recvStride * es;
        break;
      case FCX_K_BCAST:
        if (me == a.root) {
          if (dc.mcHeap != nullptr && a.useMc && n > 2) { mcSrc = send; mcDst = dc.mcHeap + stageOff; }  // two ranks: a plain store does the same
          else
            for (int p = 0; p < n; p++)
              if (p != me) { outSrc[p] = send; outDst[p] = stagePtr(dc, p, seq); }
          selfSrc = send;
          selfDst = recv;
        } else {
          inSrc[a.root] = myStage;
          inDst[a.root] = recv;
        }
        break;
      case FCX_K_GATHER:
        if (me != a.root) { outSrc[a.root] = send; outDst[a.root] = stagePtr(dc, a.root, seq) + (size_t)me * slot; }
        else {
          for (int p = 0; p < n; p++)
            if (p != me) { inSrc[p] = myStage + (size_t)p * slot; inDst[p] = recv + (size_t)p * a.recvStride * es; }
          selfSrc = send;
          selfDst = recv + (size_t)me * a.recvStride * es;
        }
        break;
      case FCX_K_SCATTER:
        if (me == a.root) {
          for (int p = 0; p < n; p++)
            if (p != me) { outSrc[p] = send + (size_t)p * a.sendStride * es; outDst[p] = stagePtr(dc, p, seq); }
          selfSrc = send + (size_t)me * a.sendStride * es;
          selfDst = recv;
        } else {
          inSrc[a.root] = myStage;
          inDst[a.root] = recv;
        }
        break;
      case FCX_K_A2A:
        for (int p = 0; p < n; p++)
          if (p != me) {
            outSrc[p] = send + (size_t)p * a.sendStride * es;
            outDst[p] = stagePtr(dc, p, seq) + (size_t)me * slot;
            inSrc[p] = myStage + (size_t)p * slot;
            inDst[p] = recv + (size_t)p * a.recvStride * es;
          }
        selfSrc = send + (size_t)me * a.sendStride * es;
        selfDst = recv + (size_t)me * a.recvStride * es;
        break;
      default: break;
    }
    if (a.kind == FCX_K_MOVE_LL) {
      const uint32_t tag = (uint32_t)seq;
      const size_t llOff = FCX_OFF_LL + (size_t)(seq & 1) * FCX_MAX_RANKS * FCX_LL_SLOT_BYTES;
      const size_t nwords = (bytes + 7) / 8;
      for (size_t w = gtid; w < nwords; w += gstride) {
        const size_t valid = min((size_t)8, bytes - w * 8);
        for (int k = 1; k < n; k++) {
          int p = (me + k) % n;
          if (!outSrc[p] && !(mcSrc && mk == FCX_K_BCAST)) continue;
          const char *src = outSrc[p] ? outSrc[p] : mcSrc;  // a multicast broadcast falls back to unicast lines here
          uint32_t lo, hi;
          ld8(src + w * 8, valid, &lo, &hi);
          llStore(dc.heap[p] + llOff + (size_t)me * FCX_LL_SLOT_BYTES + w * 16, lo, hi, tag);
        }
      }
      if (selfSrc && selfSrc != selfDst) copyUnits(selfDst, selfSrc, bytes, 16, gtid, gstride);
      bool ok = true;
      for (size_t w = gtid; w < nwords && ok; w += gstride) {
        const size_t valid = min((size_t)8, bytes - w * 8);
        for (int k = 1; k < n && ok; k++) {
          int p = (me + k) % n;
          if (!inSrc[p]) continue;
          uint4 v;
          ok = llWaitLine(dc, dc.heap[me] + llOff + (size_t)p * FCX_LL_SLOT_BYTES + w * 16, tag, p, cta, seq, &v);
          if (ok) st8(inDst[p] + w * 8, valid, v.x, v.z);
        }
      }
      epilogue(dc, seq, nctas);
      return;
    }
    const size_t sub = max((size_t)16384, (pipeBytesOf(dc) / (size_t)max(1, n - 1)) & ~(size_t)15);
    const int chunks = (int)max((size_t)1, (bytes + sub - 1) / sub);
    // remote part of sub-chunk c: bytes [off, off+len) of every outgoing piece, worked on by threads (tid0, stride)
    auto pushRange = [&](size_t off, size_t len, size_t tid0, size_t stride) {
      if (!len) return;
      if (mcDst) {
        const bool al = aligned16(mcSrc);
        const size_t nunits = (len + 15) / 16;
        for (size_t u = tid0; u < nunits; u += stride) {
          int nv = (int)min((size_t)16, len - u * 16);
          uint4 v;
          if (al && nv == 16) v = ld16(mcSrc + off + u * 16);
          else {
            union { uint4 q; char c[16]; } w;
            w.q = make_uint4(0, 0, 0, 0);
            for (int i = 0; i < nv; i++) w.c[i] = mcSrc[off + u * 16 + i];
            v = w.q;
          }
          mmStore(mcDst + off + u * 16, v);
        }
      }
      for (int k = 1; k < n; k++) {
        int p = (me + k) % n;
        if (outSrc[p]) copyToSlot(outDst[p] + off, outSrc[p] + off, len, 16, tid0, stride);
      }
    };
    auto selfRange = [&](size_t off, size_t len, size_t tid0, size_t stride) {
      if (len && selfSrc && selfSrc != selfDst) copyUnits(selfDst + off, selfSrc + off, len, 16, tid0, stride);
    };
    auto pullRange = [&](size_t off, size_t len, size_t tid0, size_t stride) {
      if (!len) return;
      for (int k = 1; k < n; k++) {
        int p = (me + k) % n;
        if (inSrc[p]) copyFromSlot(inDst[p] + off, inSrc[p] + off, len, 16, tid0, stride);
      }
    };
    // Link CTAs of this rank and of the ranks it receives from.  Rooted kinds are lopsided: the sending side
    // puts almost the whole grid on the link and the receiving side has no link work at all.
    int L = linkCtasOf(nctas), Lsrc = L;
    if (nctas >= 2) {
      const int most = nctas - max(1, nctas / 8);
      if (a.kind == FCX_K_BCAST || a.kind == FCX_K_SCATTER) { Lsrc = most; L = me == a.root ? most : 0; }
      if (a.kind == FCX_K_GATHER) { Lsrc = nctas; L = me == a.root ? 0 : nctas; }
    }
    if (nctas >= 2) {
      unsigned inMask = 0;
      bool sends = mcDst != nullptr;
      for (int p = 0; p < n; p++) {
        if (inSrc[p]) inMask |= 1u << p;
        if (outSrc[p]) sends = true;
      }
      // all-to-all in place: a piece may only be overwritten once this rank's own link CTAs have sent it
      const bool aliased = a.kind == FCX_K_A2A && send == recv;
      if (aliased && inMask) inMask |= 1u << me;
      if (cta < L) {
        for (int c = 0; c < chunks; c++) {
          size_t lo, len = subLen(bytes, sub, c, &lo), slo, slen = shareOf(len, cta, L, 16, &slo);
          if (sends) pushRange(lo + slo, slen, threadIdx.x, blockDim.x);
          postPeers(dc, cta, barrierValue(seq, 1 + (unsigned)c), aliased);
        }
      } else {
        const size_t tid0 = (size_t)(cta - L) * blockDim.x + threadIdx.x, stride = (size_t)(nctas - L) * blockDim.x;
        for (int c = 0; c < chunks; c++) {
          size_t lo, len = subLen(bytes, sub, c, &lo);
          selfRange(lo, len, tid0, stride);
          if (inMask) {
            if (!waitChunk(dc, cta, 0, Lsrc, inMask, barrierValue(seq, 1 + (unsigned)c), seq)) break;
            pullRange(lo, len, tid0, stride);
          }
        }
      }
      epilogue(dc, seq, nctas);
      return;
    }
    auto push = [&](int c) {
      size_t lo, len = subLen(bytes, sub, c, &lo);
      pushRange(lo, len, gtid, gstride);
      selfRange(lo, len, gtid, gstride);
    };
    auto pull = [&](int c) {
      size_t lo, len = subLen(bytes, sub, c, &lo);
      pullRange(lo, len, gtid, gstride);
    };
    pipelined<2>(dc, cta, seq, chunks, push, pull, pull);
    epilogue(dc, seq, nctas);
    return;
  }

  switch (a.kind) {
    case FCX_K_A2AV: {
      // Variable blocks move in rounds through per-source slots that are cut
      // in two halves, so that round k+1 can be pushed while the receiver
      // still copies round k-1 out... the barrier of round k orders them.
      // Ranks first agree on the number of rounds through the mailboxes.
      const size_t slotBytes = (dc.stageBytes / n / 2) & ~(size_t)15;
      uint64_t myRounds = 1;
      for (int p = 0; p < n; p++) {
        uint64_t r1 = (a.scounts[p] * es + slotBytes - 1) / slotBytes, r2 = (a.rcounts[p] * es + slotBytes - 1) / slotBytes;
        myRounds = max(myRounds, max(r1, r2));
      }
      if (threadIdx.x < n && threadIdx.x != me) {
        FcxMail *mb = (FcxMail *)(dc.heap[threadIdx.x] + FCX_OFF_MAIL) + (seq & 1) * FCX_MAX_RANKS + me;
        stRelaxed(&mb->a, myRounds);
      }
      if (!ctaBarrier(dc, cta, barrierValue(seq, 1), seq)) break;
      uint64_t rounds = myRounds;
      for (int p = 0; p < n; p++)
        if (p != me) {
          const FcxMail *mb = (const FcxMail *)(dc.heap[me] + FCX_OFF_MAIL) + (seq & 1) * FCX_MAX_RANKS + p;
          rounds = max(rounds, ldRelaxed(&mb->a));
        }
      {
        const char *s = send + a.sdispls[me] * es;
        char *d = recv + a.rdispls[me] * es;
        size_t b = a.scounts[me] * es;
        if (s != d && b) copyUnits(d, s, b, 16, gtid, gstride);
      }
      bool ok = true;
      for (uint64_t r = 0; r < rounds && ok; r++) {
        const size_t half = (r & 1) * slotBytes;
        for (int k = 1; k < n; k++) {
          int p = (me + k) % n;
          size_t tot = a.scounts[p] * es, lo = r * slotBytes;
          if (lo < tot)
            copyToSlot(stagePtr(dc, p, seq) + (size_t)me * 2 * slotBytes + half, send + a.sdispls[p] * es + lo,
                       min(slotBytes, tot - lo), 16, gtid, gstride);
        }
        ok = ctaBarrier(dc, cta, barrierValue(seq, 2 + (unsigned)r), seq);
        if (!ok) break;
        for (int k = 1; k < n; k++) {
          int p = (me + k) % n;
          size_t tot = a.rcounts[p] * es, lo = r * slotBytes;
          if (lo < tot)
            copyFromSlot(recv + a.rdispls[p] * es + lo, stagePtr(dc, me, seq) + (size_t)p * 2 * slotBytes + half,
                         min(slotBytes, tot - lo), 16, gtid, gstride);
        }
      }
      break;
    }

    default:
      break;
  }
  epilogue(dc, seq, nctas);
}

// ---------------------------------------------------------------- grouped send/recv

// Each op owns `ctasPerOp` consecutive CTAs.  A send pushes its data chunk by
// chunk straight from the user buffer into the receiver's staging slots
// (NVLink stores) and raises `ready` on the receiver; the receiver copies the
// chunk out of its own memory and raises `consumed` on the sender, which
// frees the slot.  Two slots per (receiver, sender) pair keep both sides busy.
// A send whose buffer is peer-visible (symmetric heap or registered segment)
// publishes where it lives instead, and the receiver reads it directly into
// the user's receive buffer: one pass over NVLink, nothing staged
// (FLAGCX_P2P_ZEROCOPY=0 turns that off).
__device__ __forceinline__ FcxP2pCtl *p2pCtl(const FcxDevComm &dc, int onRank, int dir, int peer) {
  return (FcxP2pCtl *)(dc.heap[onRank] + FCX_OFF_P2P) + dir * FCX_MAX_RANKS + peer;
}

// Arrive at the op's counter; returns true in every thread of the last CTA.
// The fences are system-wide because the data written before arriving may
// live in a peer's memory and is published by the last CTA's release store.
__device__ __forceinline__ bool opArrive(const FcxDevComm &dc, int op, int slot, int ctasPerOp) {
  __shared__ unsigned int isLast;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    unsigned int *c = &localOf(dc)->opCount[op][slot];
    unsigned int old = atomicAdd(c, 1u);
    isLast = (old == (unsigned)ctasPerOp - 1u);
    if (isLast) { *c = 0; __threadfence_system(); }
  }
  __syncthreads();
  return isLast != 0;
}

__device__ void fcxP2pBody(const FcxDevComm &dc, const FcxP2pArgs &g, int cta) {
  const int opIdx = cta / g.ctasPerOp, sub = cta % g.ctasPerOp;
  if (opIdx >= g.nops) return;
  if (*(volatile unsigned int *)&localOf(dc)->abortSeen) return;
  const FcxP2pOp &op = g.ops[opIdx];
  const int me = dc.rank, peer = op.peer;
  const size_t gtid = (size_t)sub * blockDim.x + threadIdx.x, gstride = (size_t)g.ctasPerOp * blockDim.x;
  const size_t chunk = dc.p2pChunkBytes;
  const uint64_t nchunks = op.bytes ? (op.bytes + chunk - 1) / chunk : 1;

  if (op.isRecv == 2) {  // local copy (send to self matched with recv from self); heapOff carries the source pointer
    const char *s = (const char *)(uintptr_t)op.heapOff;
    char *d = (char *)op.buf;
    copyUnits(d, s, op.bytes, 16, gtid, gstride);
    return;
  }

  if (!op.isRecv) {
    // ---- sender
    FcxP2pCtl *theirs = p2pCtl(dc, peer, 0, me);  // on the receiver: what I (sender) publish
    FcxP2pCtl *mine = p2pCtl(dc, me, 1, peer);    // on me: what the receiver publishes
    const bool zeroCopy = op.heapOff != ~0ull;
    if (zeroCopy) {
      if (sub == 0 && threadIdx.x == 0) {
        stRelaxed(&theirs->srcOff, op.heapOff);
        stRelaxed(&theirs->srcSeg, (uint64_t)(int64_t)op.seg);
        stRelease(&theirs->ready, op.firstChunk + nchunks);
      }
      // the buffer stays in use until the receiver has read all of it
      bool ok = true;
      if (threadIdx.x == 0)
        ok = waitGe(dc, &mine->consumed, op.firstChunk + nchunks, peer, FCX_WAIT_P2P_CONSUMED, cta, op.firstChunk);
      __syncthreads_and(ok);
      return;
    }
    for (uint64_t c = 0; c < nchunks; c++) {
      uint64_t gidx = op.firstChunk + c;
      int slot = (int)(gidx & 1);
      bool ok = true;
      if (gidx >= 2 && threadIdx.x == 0)
        ok = waitGe(dc, &mine->consumed, gidx - 1, peer, FCX_WAIT_P2P_CONSUMED, cta, gidx);
      if (!__syncthreads_and(ok)) return;
      size_t lo = c * chunk, nb = op.bytes > lo ? min(chunk, op.bytes - lo) : 0;
      char *st = dc.heap[peer] + dc.p2pOff + ((size_t)me * 2 + slot) * chunk;  // the receiver's slot for this sender
      if (nb) copyUnits(st, (const char *)op.buf + lo, nb, 16, gtid, gstride);
      if (opArrive(dc, opIdx, slot, g.ctasPerOp) && threadIdx.x == 0) {
        if (c == 0) stRelaxed(&theirs->srcOff, ~0ull);
        stRelease(&theirs->ready, gidx + 1);
      }
    }
    return;
  }

  // ---- receiver
  FcxP2pCtl *mine = p2pCtl(dc, me, 0, peer);    // on me: what the sender publishes
  FcxP2pCtl *theirs = p2pCtl(dc, peer, 1, me);  // on the sender: what I (receiver) publish
  {
    bool ok = true;
    if (threadIdx.x == 0) ok = waitGe(dc, &mine->ready, op.firstChunk + 1, peer, FCX_WAIT_P2P_READY, cta, op.firstChunk);
    if (!__syncthreads_and(ok)) return;
  }
  const uint64_t srcOff = ldRelaxed(&mine->srcOff);
  if (srcOff != ~0ull) {
    const char *src = zcResolve(dc, (int)(int64_t)ldRelaxed(&mine->srcSeg), srcOff, peer);
    if (op.bytes && src) copyUnits((char *)op.buf, src, op.bytes, 16, gtid, gstride);
    if (op.bytes && !src && gtid == 0) giveUp(dc, FCX_ERR_BADARG, peer, FCX_WAIT_P2P_READY, cta, 0, srcOff, op.firstChunk);
    if (opArrive(dc, opIdx, 0, g.ctasPerOp) && threadIdx.x == 0) stRelease(&theirs->consumed, op.firstChunk + nchunks);
    return;
  }
  for (uint64_t c = 0; c < nchunks; c++) {
    uint64_t gidx = op.firstChunk + c;
    int slot = (int)(gidx & 1);
    if (c > 0) {
      bool ok = true;
      if (threadIdx.x == 0) ok = waitGe(dc, &mine->ready, gidx + 1, peer, FCX_WAIT_P2P_READY, cta, gidx);
      if (!__syncthreads_and(ok)) return;
    }
    size_t lo = c * chunk, nb = op.bytes > lo ? min(chunk, op.bytes - lo) : 0;
    const char *st = dc.heap[me] + dc.p2pOff + ((size_t)peer * 2 + slot) * chunk;  // my slot for that sender
    if (nb) copyUnits((char *)op.buf + lo, st, nb, 16, gtid, gstride);
    if (opArrive(dc, opIdx, slot, g.ctasPerOp) && threadIdx.x == 0) stRelease(&theirs->consumed, gidx + 1);
  }
}

// ---------------------------------------------------------------- global entry points

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxCollKernel(FcxDevComm dc, FcxCollArgs a) {
  fcxCollBody<TIn, TOut>(dc, a, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxMoveKernel(FcxDevComm dc, FcxCollArgs a) {
  fcxMoveBody(dc, a, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxP2pKernel(FcxDevComm dc, FcxP2pArgs g) {
  fcxP2pBody(dc, g, blockIdx.x);
}

// Emulation: rank = blockIdx.x / ctasPerRank.  Launched cooperatively so that
// all emulated ranks are resident at once and may wait on one another.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxCollEmuKernel(const FcxDevComm *dcs, const FcxCollArgs *as, int ctasPerRank) {
  int r = blockIdx.x / ctasPerRank;
  fcxCollBody<TIn, TOut>(dcs[r], as[r], blockIdx.x % ctasPerRank, ctasPerRank);
}
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxMoveEmuKernel(const FcxDevComm *dcs, const FcxCollArgs *as, int ctasPerRank) {
  int r = blockIdx.x / ctasPerRank;
  fcxMoveBody(dcs[r], as[r], blockIdx.x % ctasPerRank, ctasPerRank);
}
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxP2pEmuKernel(const FcxDevComm *dcs, const FcxP2pArgs *gs, int ctasPerRank) {
  int r = blockIdx.x / ctasPerRank;
  fcxP2pBody(dcs[r], gs[r], blockIdx.x % ctasPerRank);
}

// A wait that nothing satisfies, used to test the time-out path: returns
// after dc.timeoutNs with the error record filled in.
__global__ void fcxWaitTestKernel(FcxDevComm dc, uint64_t want) {
  if (threadIdx.x == 0) {
    const uint64_t *f = (const uint64_t *)(dc.heap[dc.rank] + FCX_OFF_DEVAPI) + (FCX_DEVAPI_SIGNALS - 1) * FCX_MAX_RANKS;
    waitGe(dc, f, want, dc.rank, FCX_WAIT_TEST, 0, 0);
  }
}

}  // namespace fcxdev

// ---------------------------------------------------------------- host launchers

using namespace fcxdev;

namespace {

template <typename TIn, typename TOut>
cudaError_t launchTyped(const FcxDevComm &dc, const FcxCollArgs &a, int nctas, cudaStream_t s) {
  fcxCollKernel<TIn, TOut><<<nctas, FCX_THREADS, 0, s>>>(dc, a);
  return cudaGetLastError();
}

template <typename TIn, typename TOut>
cudaError_t launchTypedEmu(const FcxDevComm *dcs, const FcxCollArgs *as, int nranks, int nctas, cudaStream_t s) {
  void *params[] = {(void *)&dcs, (void *)&as, (void *)&nctas};
  return cudaLaunchCooperativeKernel((const void *)fcxCollEmuKernel<TIn, TOut>, dim3(nranks * nctas), dim3(FCX_THREADS),
                                     params, 0, s);
}

}  // namespace

// kinds that move bytes without looking at the element type
static bool isMoveKind(int k) {
  return (k >= FCX_K_AG && k <= FCX_K_MOVE_LL && k != FCX_K_REDUCE) || k == FCX_K_MOVE_ZC;
}
static bool isZcReduceKind(int k) { return k == FCX_K_AR_ZC || k == FCX_K_RS_ZC || k == FCX_K_REDUCE_ZC; }

// A kind that cannot serve the call's element types or reduction must never be launched: its body would
// be empty and recv would silently keep its old contents.
static bool kindServes(const FcxCollArgs *a) {
  const bool same = a->outDtype == a->dtype && a->scale == 1.0f;
  switch (a->kind) {
    case FCX_K_AR_LL: case FCX_K_RS_LL: case FCX_K_REDUCE_LL: return same;
    case FCX_K_AR_NVLS: case FCX_K_RS_NVLS: {
      if (a->outDtype != a->dtype) return false;
      if (a->dtype == 7) return a->redop == 0 || a->redop == 4;               // fp32: the switch only adds
      if (a->dtype == 6 || a->dtype == 9) return a->redop != 1;               // fp16 / bf16: add, min, max
      return false;
    }
    default: return true;
  }
}

extern "C" cudaError_t fcxLaunchColl(const FcxDevComm *dc, const FcxCollArgs *a, int nctas, cudaStream_t s) {
  if (a->kind < 0 || a->kind >= FCX_K_NUM || !kindServes(a)) return cudaErrorInvalidValue;
  if (a->kind == FCX_K_MOVE_ZC || isZcReduceKind(a->kind)) return fcxLaunchZc(dc, a, nctas, s);
  if (isMoveKind(a->kind)) {
    fcxMoveKernel<<<nctas, FCX_THREADS, 0, s>>>(*dc, *a);
    return cudaGetLastError();
  }
  if (a->kind == FCX_K_BARRIER) return launchTyped<uint8_t, uint8_t>(*dc, *a, 1, s);
#define CALL(TI, TO) launchTyped<TI, TO>(*dc, *a, nctas, s)
  FCX_DISPATCH_ALL(a, CALL);
#undef CALL
}

extern "C" cudaError_t fcxLaunchP2p(const FcxDevComm *dc, const FcxP2pArgs *g, cudaStream_t s) {
  fcxP2pKernel<<<g->nops * g->ctasPerOp, FCX_THREADS, 0, s>>>(*dc, *g);
  return cudaGetLastError();
}

extern "C" cudaError_t fcxLaunchWaitTest(const FcxDevComm *dc, uint64_t want, cudaStream_t s) {
  fcxWaitTestKernel<<<1, 32, 0, s>>>(*dc, want);
  return cudaGetLastError();
}

// dcs/as/gs are device arrays with one entry per emulated rank.
extern "C" cudaError_t fcxLaunchCollEmu(const FcxDevComm *dcs, const FcxCollArgs *as, const FcxCollArgs *hostArgs0,
                                        int nranks, int nctas, cudaStream_t s) {
  const FcxCollArgs *a = hostArgs0;
  if (a->kind < 0 || a->kind >= FCX_K_NUM || !kindServes(a)) return cudaErrorInvalidValue;
  void *params[] = {(void *)&dcs, (void *)&as, (void *)&nctas};
  if (a->kind == FCX_K_MOVE_ZC || isZcReduceKind(a->kind)) return fcxLaunchZcEmu(dcs, as, hostArgs0, nranks, nctas, s);
  if (isMoveKind(a->kind))
    return cudaLaunchCooperativeKernel((const void *)fcxMoveEmuKernel, dim3(nranks * nctas), dim3(FCX_THREADS), params, 0, s);
  if (a->kind == FCX_K_BARRIER) return launchTypedEmu<uint8_t, uint8_t>(dcs, as, nranks, nctas, s);
#define CALL(TI, TO) launchTypedEmu<TI, TO>(dcs, as, nranks, nctas, s)
  FCX_DISPATCH_ALL(a, CALL);
#undef CALL
}

extern "C" cudaError_t fcxLaunchP2pEmu(const FcxDevComm *dcs, const FcxP2pArgs *gs, int nranks, int ctasPerRank,
                                       cudaStream_t s) {
  void *params[] = {(void *)&dcs, (void *)&gs, (void *)&ctasPerRank};
  return cudaLaunchCooperativeKernel((const void *)fcxP2pEmuKernel, dim3(nranks * ctasPerRank), dim3(FCX_THREADS), params, 0, s);
}
