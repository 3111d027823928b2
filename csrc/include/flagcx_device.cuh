/*
 * flagcx_device.cuh - communication from inside a kernel.
 *
 * A kernel that receives a `FcxDevComm` by value (flagcxCommDeviceDescriptor
 * on the host) can read and write the symmetric heap of every rank of the
 * communicator directly over NVLink, raise and await signals, and use the
 * NVSwitch multicast alias, with no CPU thread in the loop.  This is what the
 * library's own fused kernels are written with.  The reference's "device
 * API" (flagcx/kernels/flagcx_kernel_device.cu:67-124) only queues requests for
 * a host thread; that form is kept for compatibility in flagcx_kernel.h.
 *
 * Memory: buffers obtained from flagcxMemAlloc(comm) live in the heap;
 * flagcxHeapOffset gives their offset, which is what these calls take.
 *
 * Signals: flagcxCommAllocSignals reserves slots.  Slot s on rank r has one
 * 64-bit word per source rank; `fcx_signal(dc, peer, s, v)` stores v into
 * this rank's word of slot s on `peer` with release semantics (everything
 * this CTA wrote before - after a __syncthreads - is visible to whoever
 * acquires the value), and `fcx_wait(dc, s, from, v)` spins until the word
 * written by `from` is >= v.  Values must grow monotonically; the wait is
 * bounded by the communicator's time-out and returns false when it gives up
 * (the host then sees flagcxRemoteError from flagcxCommGetAsyncError).
 *
 * All calls marked "CTA" must be made by every thread of the block.
 */
#pragma once
#include "../kernels/prims.cuh"

namespace flagcx {

using DevComm = FcxDevComm;

__device__ __forceinline__ char *fcx_ptr(const DevComm &dc, int rank, size_t heapOffset) { return dc.heap[rank] + heapOffset; }
__device__ __forceinline__ char *fcx_mc_ptr(const DevComm &dc, size_t heapOffset) { return dc.mcHeap ? dc.mcHeap + heapOffset : nullptr; }

__device__ __forceinline__ uint64_t *fcx_signal_word(const DevComm &dc, int onRank, int slot, int fromRank) {
  return (uint64_t *)(dc.heap[onRank] + FCX_OFF_DEVAPI) + (size_t)slot * FCX_MAX_RANKS + fromRank;
}

// One thread: publish `value` in slot `slot` of `peer`.
__device__ __forceinline__ void fcx_signal(const DevComm &dc, int peer, int slot, uint64_t value) {
  fcxdev::stRelease(fcx_signal_word(dc, peer, slot, dc.rank), value);
}
// One thread: atomically add to the word (several producers may share it).
__device__ __forceinline__ void fcx_signal_add(const DevComm &dc, int peer, int slot, uint64_t delta) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(fcx_signal_word(dc, peer, slot, dc.rank)), "l"(delta) : "memory");
}
// One thread: wait for the word that `from` writes into this rank's slot.
__device__ __forceinline__ bool fcx_wait(const DevComm &dc, int slot, int from, uint64_t value) {
  return fcxdev::waitGe(dc, fcx_signal_word(dc, dc.rank, slot, from), value, from, FCX_WAIT_DEVAPI, blockIdx.x, value);
}

// CTA: copy `bytes` from local memory into `peer`'s heap at `dstOffset` (both 16-byte aligned for full speed).
__device__ __forceinline__ void fcx_put(const DevComm &dc, int peer, size_t dstOffset, const void *src, size_t bytes) {
  const uint4 *s = (const uint4 *)src;
  uint4 *d = (uint4 *)fcx_ptr(dc, peer, dstOffset);
  const size_t n = bytes / 16;
  size_t i = threadIdx.x;
  for (; i + 3 * blockDim.x < n; i += 4 * blockDim.x) {
    uint4 a = s[i], b = s[i + blockDim.x], c = s[i + 2 * blockDim.x], e = s[i + 3 * blockDim.x];
    d[i] = a; d[i + blockDim.x] = b; d[i + 2 * blockDim.x] = c; d[i + 3 * blockDim.x] = e;
  }
  for (; i < n; i += blockDim.x) d[i] = s[i];
  for (size_t b = n * 16 + threadIdx.x; b < bytes; b += blockDim.x) ((char *)d)[b] = ((const char *)s)[b];
}
// CTA: copy from `peer`'s heap into local memory.
__device__ __forceinline__ void fcx_get(const DevComm &dc, int peer, size_t srcOffset, void *dst, size_t bytes) {
  const uint4 *s = (const uint4 *)fcx_ptr(dc, peer, srcOffset);
  uint4 *d = (uint4 *)dst;
  const size_t n = bytes / 16;
  size_t i = threadIdx.x;
  for (; i + 3 * blockDim.x < n; i += 4 * blockDim.x) {
    uint4 a = s[i], b = s[i + blockDim.x], c = s[i + 2 * blockDim.x], e = s[i + 3 * blockDim.x];
    d[i] = a; d[i + blockDim.x] = b; d[i + 2 * blockDim.x] = c; d[i + 3 * blockDim.x] = e;
  }
  for (; i < n; i += blockDim.x) d[i] = s[i];
  for (size_t b = n * 16 + threadIdx.x; b < bytes; b += blockDim.x) ((char *)d)[b] = ((const char *)s)[b];
}
// CTA: put, then signal once the whole block's stores are ordered before the flag.
__device__ __forceinline__ void fcx_put_signal(const DevComm &dc, int peer, size_t dstOffset, const void *src, size_t bytes, int slot,
                                               uint64_t value) {
  fcx_put(dc, peer, dstOffset, src, bytes);
  __syncthreads();
  if (threadIdx.x == 0) fcx_signal(dc, peer, slot, value);
}
// CTA: barrier between the calling block of every rank (same blockIdx everywhere), on slot `slot`.
__device__ __forceinline__ bool fcx_barrier(const DevComm &dc, int slot, uint64_t epoch) {
  __syncthreads();
  bool ok = true;
  int t = threadIdx.x;
  if (t < dc.nranks && t != dc.rank) {
    fcx_signal(dc, t, slot, epoch);
    ok = fcx_wait(dc, slot, t, epoch);
  }
  return __syncthreads_and(ok);
}

// ---------------------------------------------------------------- bulk-copy engine (TMA) transfers
//
// One thread streams a large block between this GPU's memory and a peer's through a ring in shared memory:
// cp.async.bulk global -> shared (completion on an mbarrier), then cp.async.bulk shared -> global (bulk groups).
// No load is multicast.  The other threads of the CTA stay free (or idle): one SM sustains a high NVLink rate
// without spending its load/store units.  Requirements: both addresses 16-byte aligned, `bytes` a multiple of 16.
//
//   __shared__ (or dynamic) ring of FCX_BULK_STAGES x FCX_BULK_CHUNK bytes, 128-byte aligned, and FCX_BULK_STAGES mbarriers;
//   fcx_bulk_init(ring) once by one thread, then __syncthreads();
//   fcx_bulk_copy(ring, dst, src, bytes, &err) by that thread, as often as needed;
//   the data is complete at the destination when the call returns; publish with fcx_bulk_release_fence() + fcx_signal.
#define FCX_BULK_STAGES 6
#define FCX_BULK_CHUNK 32768

struct fcx_bulk_ring {
  unsigned char *buf;   // FCX_BULK_STAGES * FCX_BULK_CHUNK bytes of shared memory
  uint64_t *bars;       // FCX_BULK_STAGES mbarriers in shared memory
  uint32_t phases;      // bit s: parity of the next completion on stage s
};

__device__ __forceinline__ uint32_t fcx_smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void fcx_bulk_init(fcx_bulk_ring &r, void *buf, uint64_t *bars) {
  r.buf = (unsigned char *)buf;
  r.bars = bars;
  r.phases = 0;
  for (int s = 0; s < FCX_BULK_STAGES; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(fcx_smem_addr(&bars[s])));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fcx_bulk_load_(fcx_bulk_ring &r, int stage, const char *src, uint32_t bytes) {
  const uint32_t bar = fcx_smem_addr(&r.bars[stage]), dst = fcx_smem_addr(r.buf + (size_t)stage * FCX_BULK_CHUNK);
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
               "r"(bar) : "memory");
}

// Bounded wait on a stage's mbarrier; false = gave up (sets *err).
__device__ __forceinline__ bool fcx_bulk_wait_(fcx_bulk_ring &r, int stage, volatile int *err) {
  const uint32_t bar = fcx_smem_addr(&r.bars[stage]), parity = (r.phases >> stage) & 1u;
  uint32_t done = 0;
  for (uint32_t spin = 0; spin < (1u << 26); spin++) {
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) { r.phases ^= 1u << stage; return true; }
  }
  *err = 1;
  return false;
}

// One thread.  Copies src -> dst through the ring; either side may be a peer's memory.
__device__ __forceinline__ bool fcx_bulk_copy(fcx_bulk_ring &r, void *dst, const void *src, size_t bytes, volatile int *err) {
  const char *s = (const char *)src;
  char *d = (char *)dst;
  const int n = (int)((bytes + FCX_BULK_CHUNK - 1) / FCX_BULK_CHUNK);
  auto sizeOf = [&](int c) { return (uint32_t)min((size_t)FCX_BULK_CHUNK, bytes - (size_t)c * FCX_BULK_CHUNK); };
  int ld = 0;
  bool ok = true;
  for (; ld < n && ld < FCX_BULK_STAGES - 2; ld++) fcx_bulk_load_(r, ld % FCX_BULK_STAGES, s + (size_t)ld * FCX_BULK_CHUNK, sizeOf(ld));
  for (int c = 0; c < n; c++) {
    const int st = c % FCX_BULK_STAGES;
    if (!fcx_bulk_wait_(r, st, err)) { ok = false; break; }
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(d + (size_t)c * FCX_BULK_CHUNK),
                 "r"(fcx_smem_addr(r.buf + (size_t)st * FCX_BULK_CHUNK)), "r"(sizeOf(c)) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    if (ld < n) {
      // the stage about to be refilled belongs to chunk c-2, whose store has been read once at most one group is pending
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      fcx_bulk_load_(r, ld % FCX_BULK_STAGES, s + (size_t)ld * FCX_BULK_CHUNK, sizeOf(ld));
      ld++;
    }
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  return ok;
}
// Orders the bulk engine's writes before a following release store of the same thread.
__device__ __forceinline__ void fcx_bulk_release_fence() { asm volatile("fence.proxy.async;" ::: "memory"); }

// NVSwitch: sum the same 16 bytes of every rank's heap (4 floats / 8 bf16) and broadcast 16 bytes to all.
__device__ __forceinline__ uint4 fcx_multimem_sum_f32x4(const DevComm &dc, size_t heapOffset) {
  return fcxdev::Mm<float>::ldReduce(dc.mcHeap + heapOffset, 0);
}
__device__ __forceinline__ uint4 fcx_multimem_sum_bf16x8(const DevComm &dc, size_t heapOffset) {
  return fcxdev::Mm<__nv_bfloat16>::ldReduce(dc.mcHeap + heapOffset, 0);
}
__device__ __forceinline__ void fcx_multimem_store(const DevComm &dc, size_t heapOffset, uint4 v) { fcxdev::mmStore(dc.mcHeap + heapOffset, v); }
// Add 16 bytes (4 floats) into every rank's heap at once.
__device__ __forceinline__ void fcx_multimem_red_f32x4(const DevComm &dc, size_t heapOffset, float4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(dc.mcHeap + heapOffset), "f"(v.x), "f"(v.y), "f"(v.z),
               "f"(v.w) : "memory");
}

}  // namespace flagcx
