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
  // Flow control: the caller alternates between two inboxes, so the put of epoch e lands where epoch e-2 was
  // read from.  In a ring of three or more a rank can run ahead of its right-hand neighbour (it only waits for
  // its left-hand one), so the neighbour acknowledges every epoch it has copied out (signal slot + 1) and the
  // sender waits for the acknowledgement of epoch e-2 before it overwrites that inbox.
  bool ok = true;
  if (epoch > 2 && threadIdx.x == 0) ok = fcx_wait(dc, slot + 1, next, (epoch - 2) * gridDim.x);
  ok = __syncthreads_and(ok);
  if (!ok) { if (threadIdx.x == 0) *status = 1; return; }
  fcx_put(dc, next, inboxOffset + lo, src + lo, hi - lo);
  __syncthreads();
  // every block signals its own word by adding one; the consumer waits for gridDim.x arrivals of this epoch
  if (threadIdx.x == 0) fcx_signal_add(dc, next, slot, 1);
  if (threadIdx.x == 0) ok = fcx_wait(dc, slot, prev, epoch * gridDim.x);
  ok = __syncthreads_and(ok);
  if (!ok) { if (threadIdx.x == 0) *status = 1; return; }
  fcx_get(dc, dc.rank, inboxOffset + lo, dst + lo, hi - lo);
  __syncthreads();
  if (threadIdx.x == 0) fcx_signal_add(dc, prev, slot + 1, 1);  // this block's share of the inbox may be reused
}

// `slot` and `slot + 1` must both be reserved (flagcxCommAllocSignals(comm, 2, &slot)); `epoch` counts the calls from 1
// and the caller alternates between two inboxes (epoch & 1).
extern "C" cudaError_t fcxRingExchange(const FcxDevComm *dc, const void *src, size_t inboxOffset, void *dst, size_t bytes, int slot,
                                       unsigned long long epoch, int *status, int nblocks, cudaStream_t s) {
  fcxRingExchangeKernel<<<nblocks, 512, 0, s>>>(*dc, (const char *)src, inboxOffset, (char *)dst, bytes, slot, epoch, status);
  return cudaGetLastError();
}
