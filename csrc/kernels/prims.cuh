// Device-side building blocks of the collective kernels: system-scope
// flag accesses, bounded waits, the cross-GPU CTA barrier, and unit-wise
// load/convert/store helpers for every element type.
#pragma once
#include "devcomm.h"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

namespace fcxdev {

// ------------------------------------------------------------------ flags

__device__ __forceinline__ void stRelease(uint64_t *p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void stRelaxed(uint64_t *p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ldAcquire(const uint64_t *p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ldRelaxed(const uint64_t *p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t globalTimerNs() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Local words of the control block that only this rank's kernels touch.
struct FcxLocal {
  unsigned int ctaDone;        // CTAs of the running collective that reached the epilogue
  unsigned int errClaim;       // first waiter to give up owns the host error record
  unsigned int abortSeen;      // set once any waiter gave up; later waits leave at once
  unsigned int pad;
  unsigned long long seq;      // collectives completed by this rank; the next one runs as seq + 1
  unsigned int opCount[FCX_MAX_GROUP_OPS][2];  // arrivals per grouped p2p op and staging slot
};

__device__ __forceinline__ FcxLocal *localOf(const FcxDevComm &dc) {
  return (FcxLocal *)(dc.heap[dc.rank] + FCX_OFF_LOCAL);
}

// Record why a wait ended without its condition.  Never traps: the kernel
// keeps running valid code and returns; the host reads the record.
static __device__ __noinline__ void giveUp(const FcxDevComm &dc, uint32_t code, int peer, int where, int cta,
                                    uint64_t expected, uint64_t seen, uint64_t seq) {
  FcxLocal *loc = localOf(dc);
  if (atomicCAS(&loc->errClaim, 0u, 1u) == 0u) {
    volatile FcxDevError *e = dc.err;
    e->peer = peer;
    e->where = where;
    e->cta = cta;
    e->expected = expected;
    e->seen = seen;
    e->seq = seq;
    __threadfence_system();
    e->code = code;
    __threadfence_system();
  }
  atomicExch(&loc->abortSeen, 1u);
}

// Spin until *flag >= want.  Bounded three ways: the communicator's time-out
// (measured with %globaltimer), the host's abort word, and a local word set
// by the first waiter that gave up.  Returns false when the wait was cut short.
__device__ __forceinline__ bool waitGe(const FcxDevComm &dc, const uint64_t *flag, uint64_t want, int peer,
                                       int where, int cta, uint64_t seq) {
  uint64_t v = ldAcquire(flag);
  if (v >= want) return true;
  FcxLocal *loc = localOf(dc);
  uint64_t t0 = globalTimerNs();
  unsigned int spins = 0;
  for (;;) {
    v = ldAcquire(flag);
    if (v >= want) return true;
    spins++;
    if (spins > 64) __nanosleep(spins > 4096 ? 400 : 40);
    if ((spins & 63u) == 0u) {
      if (*(volatile unsigned int *)&loc->abortSeen) return false;
      if (globalTimerNs() - t0 > dc.timeoutNs) {
        giveUp(dc, FCX_ERR_TIMEOUT, peer, where, cta, want, v, seq);
        return false;
      }
      if ((spins & 1023u) == 0u && *dc.abortWord) {
        giveUp(dc, FCX_ERR_ABORT, peer, where, cta, want, v, seq);
        return false;
      }
    }
  }
}

__device__ __forceinline__ uint64_t *flagSlot(const FcxDevComm &dc, int onRank, int cta, int fromRank) {
  return (uint64_t *)(dc.heap[onRank] + FCX_OFF_FLAGS) + (size_t)cta * FCX_MAX_RANKS + fromRank;
}

// Barrier between CTA `cta` of every rank.  All threads of the CTA call it.
// Writes made by this CTA before the call are visible to the peers' CTA
// `cta` after their call returns (release store after the CTA-wide sync;
// acquire load before the second sync).
__device__ __forceinline__ bool ctaBarrier(const FcxDevComm &dc, int cta, uint64_t value, uint64_t seq) {
  __syncthreads();
  bool ok = true;
  int t = threadIdx.x;
  if (t < dc.nranks && t != dc.rank) {
    stRelease(flagSlot(dc, t, cta, dc.rank), value);
    ok = waitGe(dc, flagSlot(dc, dc.rank, cta, t), value, t, FCX_WAIT_BARRIER, cta, seq);
  }
  return __syncthreads_and(ok);
}

// Flag value of phase `phase` of collective `seq`.  The phase field is 24 bits wide: the pipelined kinds count one
// phase per sub-chunk, and a launch never holds more than stageBytes / 16 KiB sub-chunks (the host caps the
// staging area at 2^24 sub-chunks of the smallest size), so a phase can never carry into the sequence number.
#define FCX_PHASE_BITS 24
__device__ __forceinline__ uint64_t barrierValue(uint64_t seq, unsigned phase) {
  return (seq << FCX_PHASE_BITS) | (uint64_t)(phase & ((1u << FCX_PHASE_BITS) - 1u));
}

// The sequence number of the collective that is starting.  It lives in device
// memory (not in the launch arguments) so that a captured CUDA graph can be
// replayed: every replay advances it exactly as a fresh launch would.
__device__ __forceinline__ uint64_t nextSeq(const FcxDevComm &dc) {
  return *(volatile unsigned long long *)&localOf(dc)->seq + 1;
}

// Before writing into a peer's parity-selected buffers for collective `seq`,
// the peer must have finished collective seq-2 (which used the same parity).
__device__ __forceinline__ bool prologue(const FcxDevComm &dc, uint64_t seq, int cta) {
  if (*(volatile unsigned int *)&localOf(dc)->abortSeen) return false;
  bool ok = true;
  int t = threadIdx.x;
  if (seq >= 2 && t < dc.nranks && t != dc.rank) {
    const uint64_t *d = (const uint64_t *)(dc.heap[dc.rank] + FCX_OFF_DONE) + t;
    ok = waitGe(dc, d, seq - 2, t, FCX_WAIT_DONE, cta, seq);
  }
  return __syncthreads_and(ok);
}

// The last CTA of this rank to finish tells every peer that collective `seq`
// no longer reads this rank's parity buffers.
__device__ __forceinline__ void epilogue(const FcxDevComm &dc, uint64_t seq, int nctas) {
  __syncthreads();
  __shared__ unsigned int last;
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned int old = atomicAdd(&localOf(dc)->ctaDone, 1u);
    last = (old == (unsigned)nctas - 1u);
    if (last) {
      localOf(dc)->ctaDone = 0;
      localOf(dc)->seq = seq;
    }
  }
  __syncthreads();
  if (last && threadIdx.x < dc.nranks && threadIdx.x != dc.rank) {
    uint64_t *d = (uint64_t *)(dc.heap[threadIdx.x] + FCX_OFF_DONE) + dc.rank;
    stRelease(d, seq);
  }
}

// Rank p's copy of a peer-visible buffer, as this rank addresses it (FCX_SEG_* in devcomm.h); null when the
// segment is unknown.
__device__ __forceinline__ char *zcResolve(const FcxDevComm &dc, int seg, uint64_t off, int p) {
  if (seg == FCX_SEG_HEAP) return dc.heap[p] + off;
  if (seg == FCX_SEG_ABS) return (char *)(uintptr_t)off;
  if (seg > 0 && seg < FCX_MAX_SEGS && dc.segs != nullptr) {
    char *b = dc.segs[seg][p];
    return b ? b + off : nullptr;
  }
  return nullptr;
}

// ------------------------------------------------------------------ element types

struct F8E4 { uint8_t v; };
struct F8E5 { uint8_t v; };

template <typename T> struct Elem { using Acc = T;
  static __device__ __forceinline__ Acc up(T x) { return x; }
  static __device__ __forceinline__ T down(Acc a) { return a; } };
template <> struct Elem<__half> { using Acc = float;
  static __device__ __forceinline__ float up(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half down(float a) { return __float2half_rn(a); } };
template <> struct Elem<__nv_bfloat16> { using Acc = float;
  static __device__ __forceinline__ float up(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 down(float a) { return __float2bfloat16_rn(a); } };
template <> struct Elem<F8E4> { using Acc = float;
  static __device__ __forceinline__ float up(F8E4 x) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(x.v, __NV_E4M3))); }
  static __device__ __forceinline__ F8E4 down(float a) {
    F8E4 r; r.v = (uint8_t)__nv_cvt_float_to_fp8(a, __NV_SATFINITE, __NV_E4M3); return r; } };
template <> struct Elem<F8E5> { using Acc = float;
  static __device__ __forceinline__ float up(F8E5 x) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(x.v, __NV_E5M2))); }
  static __device__ __forceinline__ F8E5 down(float a) {
    F8E5 r; r.v = (uint8_t)__nv_cvt_float_to_fp8(a, __NV_SATFINITE, __NV_E5M2); return r; } };

// redop values follow flagcxRedOp_t: 0 sum, 1 prod, 2 max, 3 min, 4 avg
template <typename A> __device__ __forceinline__ A applyOp(A a, A b, int op) {
  switch (op) {
    case 1: return a * b;
    case 2: return a > b ? a : b;
    case 3: return a < b ? a : b;
    default: return a + b;
  }
}

// Result of an accumulator type converted to the accumulator type of the
// output element (identity unless a cast is fused into the all-reduce).
template <typename AO, typename AI> __device__ __forceinline__ AO accCast(AI a) { return (AO)a; }

template <typename A> __device__ __forceinline__ A finish(A a, int op, int nranks, float scale) {
  if (op == 4) a = a / (A)nranks;
  return a;
}
template <> __device__ __forceinline__ float finish<float>(float a, int op, int nranks, float scale) {
  if (op == 4) a = a / (float)nranks;
  if (scale != 1.0f) a *= scale;
  return a;
}

// ------------------------------------------------------------------ 16-byte accesses

__device__ __forceinline__ uint4 ld16(const void *p) { return *(const uint4 *)p; }
__device__ __forceinline__ void st16(void *p, uint4 v) { *(uint4 *)p = v; }

// Copy `n` (<= unitBytes) bytes; `aligned` says that both pointers are 16-byte aligned.
__device__ __forceinline__ void copyUnit(char *dst, const char *src, int unitBytes, int n, bool aligned) {
  if (aligned && n == unitBytes) {
#pragma unroll 4
    for (int i = 0; i < unitBytes; i += 16) st16(dst + i, ld16(src + i));
  } else {
    for (int i = 0; i < n; i++) dst[i] = src[i];
  }
}

// Load G elements of T (nvalid of them meaningful) and widen.
template <typename T, int G>
__device__ __forceinline__ void loadUnit(const char *p, bool aligned, int nvalid, typename Elem<T>::Acc *out) {
  constexpr int BYTES = G * (int)sizeof(T);
  if (aligned && nvalid == G) {
    union { uint4 v[BYTES / 16]; T t[G]; } u;
#pragma unroll
    for (int i = 0; i < BYTES / 16; i++) u.v[i] = ld16(p + 16 * i);
#pragma unroll
    for (int i = 0; i < G; i++) out[i] = Elem<T>::up(u.t[i]);
  } else {
    const T *e = (const T *)p;
#pragma unroll
    for (int i = 0; i < G; i++) out[i] = i < nvalid ? Elem<T>::up(e[i]) : typename Elem<T>::Acc(0);
  }
}

template <typename T, int G>
__device__ __forceinline__ void packUnit(const typename Elem<T>::Acc *in, uint4 *v) {
  union { uint4 v[G * sizeof(T) / 16]; T t[G]; } u;
#pragma unroll
  for (int i = 0; i < G; i++) u.t[i] = Elem<T>::down(in[i]);
#pragma unroll
  for (int i = 0; i < (int)(G * sizeof(T) / 16); i++) v[i] = u.v[i];
}

template <typename T, int G>
__device__ __forceinline__ void storeUnit(char *p, bool aligned, int nvalid, const uint4 *packed) {
  constexpr int BYTES = G * (int)sizeof(T);
  if (aligned && nvalid == G) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; i++) st16(p + 16 * i, packed[i]);
  } else {
    const T *src = (const T *)packed;
    T *e = (T *)p;
    for (int i = 0; i < nvalid; i++) e[i] = src[i];
  }
}

__device__ __forceinline__ bool aligned16(const void *p) { return (((uintptr_t)p) & 15u) == 0; }

// ------------------------------------------------------------------ multimem (NVSwitch)

template <typename T> struct Mm { static constexpr bool ok = false; };
template <> struct Mm<float> {
  static constexpr bool ok = true;
  static __device__ __forceinline__ uint4 ldReduce(const void *mc, int op) {
    uint4 r;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    return r;
  }
  static __device__ __forceinline__ bool opOk(int op) { return op == 0 || op == 4; }
};
template <> struct Mm<__nv_bfloat16> {
  static constexpr bool ok = true;
  static __device__ __forceinline__ uint4 ldReduce(const void *mc, int op) {
    uint4 r;
    if (op == 2)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    else if (op == 3)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    else
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    return r;
  }
  static __device__ __forceinline__ bool opOk(int op) { return op == 0 || op == 2 || op == 3 || op == 4; }
};
template <> struct Mm<__half> {
  static constexpr bool ok = true;
  static __device__ __forceinline__ uint4 ldReduce(const void *mc, int op) {
    uint4 r;
    if (op == 2)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.max.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    else if (op == 3)
      asm volatile("multimem.ld_reduce.relaxed.sys.global.min.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    else
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                   : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc) : "memory");
    return r;
  }
  static __device__ __forceinline__ bool opOk(int op) { return op == 0 || op == 2 || op == 3 || op == 4; }
};

__device__ __forceinline__ void mmStore(void *mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w) : "memory");
}

// ---------------------------------------------------------------- plain copies

// Copy `bytes` between two buffers in units of `unitBytes` (a multiple of 16).
// Unit u always belongs to thread (u mod gstride), whatever the alignment, so
// the same thread that wrote a unit into a slot is the one that reads it back
// on the other side of a barrier.  When both pointers are 16-byte aligned the
// loop keeps four independent 16-byte loads in flight per thread.
__device__ __forceinline__ void copyUnits(char *dst, const char *src, size_t bytes, int unitBytes, size_t gtid,
                                          size_t gstride) {
  const size_t nfull = bytes / unitBytes;
  const int tail = (int)(bytes - nfull * unitBytes);
  uintptr_t both = (uintptr_t)dst | (uintptr_t)src;
  if ((both & 15u) == 0) {
    size_t u = gtid;
    if (unitBytes == 16) {
      // eight independent 16-byte loads in flight per thread, then eight stores
      for (; u + 7 * gstride < nfull; u += 8 * gstride) {
        uint4 v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = ld16(src + (u + i * gstride) * 16);
#pragma unroll
        for (int i = 0; i < 8; i++) st16(dst + (u + i * gstride) * 16, v[i]);
      }
      for (; u + 3 * gstride < nfull; u += 4 * gstride) {
        uint4 v0 = ld16(src + u * 16), v1 = ld16(src + (u + gstride) * 16), v2 = ld16(src + (u + 2 * gstride) * 16),
              v3 = ld16(src + (u + 3 * gstride) * 16);
        st16(dst + u * 16, v0);
        st16(dst + (u + gstride) * 16, v1);
        st16(dst + (u + 2 * gstride) * 16, v2);
        st16(dst + (u + 3 * gstride) * 16, v3);
      }
      for (; u < nfull; u += gstride) st16(dst + u * 16, ld16(src + u * 16));
    } else {
      const int lines = unitBytes / 16;
      for (; u < nfull; u += gstride) {
        uint4 v[4];
        const char *s = src + u * unitBytes;
        char *d = dst + u * unitBytes;
        for (int l0 = 0; l0 < lines; l0 += 4) {
#pragma unroll
          for (int l = 0; l < 4; l++)
            if (l0 + l < lines) v[l] = ld16(s + (l0 + l) * 16);
#pragma unroll
          for (int l = 0; l < 4; l++)
            if (l0 + l < lines) st16(d + (l0 + l) * 16, v[l]);
        }
      }
    }
  } else if ((both & 3u) == 0 && (bytes & 3u) == 0) {
    for (size_t u = gtid; u < nfull; u += gstride) {
      const uint32_t *s = (const uint32_t *)(src + u * unitBytes);
      uint32_t *d = (uint32_t *)(dst + u * unitBytes);
      for (int i = 0; i < unitBytes / 4; i++) d[i] = s[i];
    }
  } else {
    for (size_t u = gtid; u < nfull; u += gstride) {
      const char *s = src + u * unitBytes;
      char *d = dst + u * unitBytes;
      for (int i = 0; i < unitBytes; i++) d[i] = s[i];
    }
  }
  if (tail && (nfull % gstride) == gtid) {
    const char *s = src + nfull * unitBytes;
    char *d = dst + nfull * unitBytes;
    for (int i = 0; i < tail; i++) d[i] = s[i];
  }
}

// ---------------------------------------------------------------- NVLS helpers

template <typename T>
__device__ __forceinline__ uint4 mmFinish(uint4 r, int op, int nranks, float scale) {
  // avg and scale need arithmetic on the switch's result
  if (op != 4 && scale == 1.0f) return r;
  using Acc = typename Elem<T>::Acc;
  constexpr int G = 16 / (int)sizeof(T);
  union { uint4 v; T t[G]; } w;
  w.v = r;
  Acc x[G];
#pragma unroll
  for (int i = 0; i < G; i++) x[i] = finish<Acc>(Elem<T>::up(w.t[i]), op, nranks, scale);
  uint4 o;
  packUnit<T, G>(x, &o);
  return o;
}


}  // namespace fcxdev
