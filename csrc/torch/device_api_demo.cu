// Ring exchange written with the in-kernel communication API
// (flagcx_device.cuh): every rank puts its block into the next rank's heap
// buffer and signals; it then waits for the previous rank's signal and copies
// what arrived into the output.  This is the building block of ring attention
// (rotating K/V blocks) and of pipeline-parallel hand-offs; the reference
// offers it only through host-driven send/recv (test/perf/test_sendrecv.cpp:110-113).
#include "flagcx_device.cuh"
#include <cuda_runtime.h>

__global__ void __launch_bounds__(512) fcxRingExchangeKernel(FcxDevComm dc, const char *src, size_t inboxOffset, char *dst, size_t bytes,
                                                             int slot, unsigned long long epoch, int *status) {
  using namespace flagcx;
  const int next = (dc.rank + 1) % dc.nranks, prev = (dc.rank + dc.nranks - 1) % dc.nranks;
  // each block moves a contiguous share of the message (16-byte granules)
  const size_t granules = (bytes + 15) / 16, per = (granules + gridDim.x - 1) / gridDim.x;
  const size_t lo = min(bytes, (size_t)blockIdx.x * per * 16), hi = min(bytes, lo + per * 16);
  fcx_put(dc, next, inboxOffset + lo, src + lo, hi - lo);
  __syncthreads();
  // every block signals its own word by adding one; the consumer waits for gridDim.x arrivals of this epoch
  if (threadIdx.x == 0) fcx_signal_add(dc, next, slot, 1);
  bool ok = true;
  if (threadIdx.x == 0) ok = fcx_wait(dc, slot, prev, epoch * gridDim.x);
  ok = __syncthreads_and(ok);
  if (!ok) { if (threadIdx.x == 0) *status = 1; return; }
  fcx_get(dc, dc.rank, inboxOffset + lo, dst + lo, hi - lo);
}

extern "C" cudaError_t fcxRingExchange(const FcxDevComm *dc, const void *src, size_t inboxOffset, void *dst, size_t bytes, int slot,
                                       unsigned long long epoch, int *status, int nblocks, cudaStream_t s) {
  fcxRingExchangeKernel<<<nblocks, 512, 0, s>>>(*dc, (const char *)src, inboxOffset, (char *)dst, bytes, slot, epoch, status);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- copy-rate probe
// Moves `bytes` between this rank's `local` buffer and `peer`'s heap at `peerOffset`, split over the CTAs:
//   mode 0  every thread loads and stores 16 bytes at a time (fcx_put)
//   mode 1  bulk-copy engine, local -> peer (one thread per CTA drives a shared-memory ring)
//   mode 2  bulk-copy engine, peer -> local
// Used to choose between the two transfer styles per message size and CTA budget.
__global__ void __launch_bounds__(512) fcxCopyProbeKernel(FcxDevComm dc, char *local, size_t peerOffset, size_t bytes, int mode, int peer,
                                                          int *status) {
  using namespace flagcx;
  extern __shared__ __align__(128) unsigned char probeSmem[];
  const size_t granules = bytes / 16, per = (granules + gridDim.x - 1) / gridDim.x;
  const size_t lo = min(bytes, (size_t)blockIdx.x * per * 16), hi = min(bytes, lo + per * 16);
  if (mode == 0) {
    fcx_put(dc, peer, peerOffset + lo, local + lo, hi - lo);
    return;
  }
  if (threadIdx.x == 0 && hi > lo) {
    fcx_bulk_ring ring;
    fcx_bulk_init(ring, probeSmem, (uint64_t *)(probeSmem + (size_t)FCX_BULK_STAGES * FCX_BULK_CHUNK));
    char *remote = fcx_ptr(dc, peer, peerOffset + lo);
    if (mode == 1) fcx_bulk_copy(ring, remote, local + lo, hi - lo, status);
    else fcx_bulk_copy(ring, local + lo, remote, hi - lo, status);
  }
}

extern "C" cudaError_t fcxCopyProbe(const FcxDevComm *dc, void *local, size_t peerOffset, size_t bytes, int mode, int peer, int *status,
                                    int nblocks, cudaStream_t s) {
  if (bytes % 16 || ((uintptr_t)local & 15) || (peerOffset & 15)) return cudaErrorInvalidValue;
  const int smem = mode ? FCX_BULK_STAGES * FCX_BULK_CHUNK + 64 : 0;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fcxCopyProbeKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FCX_BULK_STAGES * FCX_BULK_CHUNK + 64);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  fcxCopyProbeKernel<<<nblocks, mode ? 32 : 512, smem, s>>>(*dc, (char *)local, peerOffset, bytes, mode, peer, status);
  return cudaGetLastError();
}
