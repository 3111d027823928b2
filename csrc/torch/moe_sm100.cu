// Expert-parallel mixture-of-experts: dispatch and combine without a host
// round trip (one or several experts per rank).
//
//   fcxMoeDispatch  one cooperative kernel: counts the tokens bound for every
//                   expert, exchanges the count matrix with all ranks through
//                   the symmetric heap, derives this rank's write offsets on
//                   every expert, pushes each token's hidden vector straight
//                   into the expert rank's input buffer over NVLink together
//                   with a (source rank, token, choice) record, and returns
//                   once every source has finished writing into this rank.
//                   The number of rows received stays on the device.
//   (expert MLP)    tcgen05 GEMMs with a device-resident row count
//                   (gemm_sm100.cu); the down projection runs in ROWMAP mode:
//                   its epilogue stores every output row directly into the
//                   combine buffer of the rank the token came from.
//   fcxMoeCombine   waits for every CTA of every expert to report, then
//                   out[t] = sum_k w[t,k] * returned[t,k].
//
// With the reference a MoE layer needs flagcxAlltoAllv twice, whose counts and
// displacements are host arrays (flagcx/include/flagcx.h:397-401): the router
// result has to be copied to the host and the stream synchronised before the
// dispatch can even be issued.
#include "../kernels/prims.cuh"

#include <algorithm>
#include <cooperative_groups.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "moe_sm100.h"

namespace cg = cooperative_groups;

namespace {

constexpr int THREADS = 512;

__global__ void __launch_bounds__(THREADS, 1) moeDispatchKernel(const FcxDevComm dc, const FcxMoeParams p) {
  cg::grid_group grid = cg::this_grid();
  const int n = dc.nranks, me = dc.rank, L = p.L, E = n * L, capL = p.cap / L;
  const int entries = p.T * p.K;
  __shared__ int warpTotals[THREADS / 32];
  __shared__ int running;
  volatile int *err = p.errFlag;

  // ---- phase 1: CTA e numbers, in token order, the entries routed to expert e
  if ((int)blockIdx.x < E) {
    const int e = blockIdx.x;
    if (threadIdx.x == 0) running = 0;
    __syncthreads();
    for (int base = 0; base < entries; base += THREADS) {
      const int i = base + threadIdx.x;
      const int hit = (i < entries && p.topkIdx[i] == e) ? 1 : 0;
      const unsigned ballot = __ballot_sync(0xffffffffu, hit);
      const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
      const int before = __popc(ballot & ((1u << lane) - 1));
      if (lane == 0) warpTotals[warp] = __popc(ballot);
      __syncthreads();
      int warpBase = 0, total = 0;
      for (int w = 0; w < THREADS / 32; w++) {
        if (w < warp) warpBase += warpTotals[w];
        total += warpTotals[w];
      }
      if (hit) p.slot[i] = running + warpBase + before;
      __syncthreads();
      if (threadIdx.x == 0) running += total;
      __syncthreads();
    }
    if (threadIdx.x == 0) p.localCounts[e] = running;
  }
  __threadfence();
  grid.sync();

  // ---- phase 2: every rank learns the whole count matrix [source][expert]
  if (blockIdx.x == 0 && (int)threadIdx.x < n) {
    const int r = threadIdx.x;
    int *mat = (int *)(dc.heap[r] + p.countMatOff) + me * E;
    for (int e = 0; e < E; e++) mat[e] = p.localCounts[e];
    __threadfence_system();
    fcxdev::stRelease((uint64_t *)(dc.heap[r] + p.countFlagOff) + me, p.epoch);
  }
  __shared__ int baseOf[64];  // where this rank's tokens start in expert e's segment
  {
    bool ok = true;
    if ((int)threadIdx.x < n)
      ok = fcxdev::waitGe(dc, (const uint64_t *)(dc.heap[me] + p.countFlagOff) + threadIdx.x, p.epoch, threadIdx.x, FCX_WAIT_DEVAPI,
                          blockIdx.x, p.epoch);
    if (!__syncthreads_and(ok)) { if (threadIdx.x == 0) *err = 1; }
    const int *mat = (const int *)(dc.heap[me] + p.countMatOff);
    if ((int)threadIdx.x < E) {
      int b = 0, tot = 0;
      for (int r = 0; r < n; r++) {
        int c = mat[r * E + threadIdx.x];
        if (r < me) b += c;
        tot += c;
      }
      baseOf[threadIdx.x] = b;
      if (tot > capL && blockIdx.x == 0) *err = 2;  // an expert's segment would overflow: tokens beyond the capacity are dropped
    }
    __syncthreads();
  }

  // ---- phase 3: one warp per (token, choice): push the hidden vector and its return address
  {
    const int warpsPerGrid = gridDim.x * (THREADS / 32);
    const int gw = blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const int vecs = p.H / 8;  // 16-byte vectors per token
    for (int i = gw; i < entries; i += warpsPerGrid) {
      const int e = p.topkIdx[i];
      if (e < 0 || e >= E) continue;
      const int inSeg = baseOf[e] + p.slot[i];
      if (inSeg >= capL) continue;
      const int dstRank = e / L, pos = (e % L) * capL + inSeg;
      const int t = i / p.K, k = i % p.K;
      const uint4 *src = (const uint4 *)((const __nv_bfloat16 *)p.x + (size_t)t * p.H);
      uint4 *dst = (uint4 *)(dc.heap[dstRank] + p.recvOff + (size_t)pos * p.H * 2);
      int v = lane;
      for (; v + 96 < vecs; v += 128) {
        uint4 a = src[v], b = src[v + 32], c = src[v + 64], d = src[v + 96];
        dst[v] = a; dst[v + 32] = b; dst[v + 64] = c; dst[v + 96] = d;
      }
      for (; v < vecs; v += 32) dst[v] = src[v];
      if (lane == 0) ((int4 *)(dc.heap[dstRank] + p.infoOff))[pos] = make_int4(me, t, k, 0);
    }
  }
  __threadfence_system();
  grid.sync();

  // ---- phase 4: tell every expert that this source is done; wait for all sources of this expert
  if (blockIdx.x == 0) {
    if ((int)threadIdx.x < n) fcxdev::stRelease((uint64_t *)(dc.heap[threadIdx.x] + p.doneOff) + me, p.epoch);
    bool ok = true;
    if ((int)threadIdx.x < n)
      ok = fcxdev::waitGe(dc, (const uint64_t *)(dc.heap[me] + p.doneOff) + threadIdx.x, p.epoch, threadIdx.x, FCX_WAIT_DEVAPI, 0, p.epoch);
    if (!__syncthreads_and(ok)) { if (threadIdx.x == 0) *err = 1; }
    if ((int)threadIdx.x < L) {
      const int *mat = (const int *)(dc.heap[me] + p.countMatOff);
      int tot = 0;
      for (int r = 0; r < n; r++) tot += mat[r * E + me * L + threadIdx.x];
      p.recvTotal[threadIdx.x] = min(tot, capL);
    }
  }
}

// h[r, f] = silu(g[r, f]) * u[r, f] with gu = [g | u] of width 2F; rows beyond *rows are skipped
__global__ void __launch_bounds__(256) siluMulKernel(const __nv_bfloat16 *__restrict__ gu, __nv_bfloat16 *__restrict__ h, const int *rows,
                                                     int maxRows, int F) {
  const int R = rows ? min(*rows, maxRows) : maxRows;
  const size_t vecPerRow = F / 8, total = (size_t)R * vecPerRow;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / vecPerRow, c = i % vecPerRow;
    uint4 gv = *(const uint4 *)(gu + r * 2 * F + c * 8), uv = *(const uint4 *)(gu + r * 2 * F + F + c * 8);
    const __nv_bfloat162 *g2 = (const __nv_bfloat162 *)&gv, *u2 = (const __nv_bfloat162 *)&uv;
    uint4 o;
    __nv_bfloat162 *o2 = (__nv_bfloat162 *)&o;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
      float a = g.x / (1.f + __expf(-g.x)) * u.x, b = g.y / (1.f + __expf(-g.y)) * u.y;
      o2[j] = __floats2bfloat162_rn(a, b);
    }
    *(uint4 *)(h + r * F + c * 8) = o;
  }
}

// out[t] = sum_k w[t,k] * ret[t,k], after every CTA of every expert's output GEMM has reported
__global__ void __launch_bounds__(256) moeCombineKernel(const FcxDevComm dc, const __nv_bfloat16 *__restrict__ ret, const float *__restrict__ w,
                                                        __nv_bfloat16 *__restrict__ out, int T, int H, int K, size_t doneOff, uint64_t want,
                                                        int *errFlag) {
  bool ok = true;
  if (threadIdx.x == 0) {
    ok = fcxdev::waitGe(dc, (const uint64_t *)(dc.heap[dc.rank] + doneOff), want, -1, FCX_WAIT_DEVAPI, blockIdx.x, want);
    if (!ok) *errFlag = 1;
  }
  if (!__syncthreads_and(ok)) return;
  const size_t vecPerRow = H / 8, total = (size_t)T * vecPerRow, stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (K <= 4) {
    // two output vectors per thread and step, every choice's row loaded before the first is used: up to eight
    // 16-byte loads in flight per thread (the kernel is bound by load latency, not by bytes)
    for (; i < total; i += 2 * stride) {
      const size_t pos[2] = {i, i + stride};
      uint4 v[2][4];
      float wk[2][4];
#pragma unroll
      for (int u = 0; u < 2; u++) {
        const bool live = pos[u] < total;
        const size_t t = live ? pos[u] / vecPerRow : 0, c = live ? pos[u] % vecPerRow : 0;
#pragma unroll
        for (int k = 0; k < 4; k++) {
          wk[u][k] = (live && k < K) ? w[t * K + k] : 0.f;
          // a choice that was not dispatched (expert id out of range, capacity overflow) has weight 0 and no row
          v[u][k] = wk[u][k] != 0.f ? *(const uint4 *)(ret + ((t * K + k) * H) + c * 8) : make_uint4(0, 0, 0, 0);
        }
      }
#pragma unroll
      for (int u = 0; u < 2; u++) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const __nv_bfloat162 *h2 = (const __nv_bfloat162 *)&v[u][k];
#pragma unroll
          for (int j = 0; j < 4; j++) {
            float2 f = __bfloat1622float2(h2[j]);
            acc[2 * j] += wk[u][k] * f.x;
            acc[2 * j + 1] += wk[u][k] * f.y;
          }
        }
        uint4 o;
        __nv_bfloat162 *o2 = (__nv_bfloat162 *)&o;
#pragma unroll
        for (int j = 0; j < 4; j++) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
        if (pos[u] < total) {
          const size_t t = pos[u] / vecPerRow, c = pos[u] % vecPerRow;
          *(uint4 *)(out + t * H + c * 8) = o;
        }
      }
    }
    return;
  }
  for (; i < total; i += stride) {
    const size_t t = i / vecPerRow, c = i % vecPerRow;
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int k = 0; k < K; k++) {
      const float wk = w[t * K + k];
      if (wk == 0.f) continue;  // a choice that was not dispatched (expert id out of range, capacity overflow) has no row
      uint4 v = *(const uint4 *)(ret + ((t * K + k) * H) + c * 8);
      const __nv_bfloat162 *h2 = (const __nv_bfloat162 *)&v;
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 f = __bfloat1622float2(h2[j]);
        acc[2 * j] += wk * f.x;
        acc[2 * j + 1] += wk * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162 *o2 = (__nv_bfloat162 *)&o;
#pragma unroll
    for (int j = 0; j < 4; j++) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    *(uint4 *)(out + t * H + c * 8) = o;
  }
}

}  // namespace

extern "C" cudaError_t fcxMoeDispatch(const FcxDevComm *dc, const FcxMoeParams *p, int ctas, cudaStream_t s) {
  if (p->H % 8 || p->K < 1 || dc->nranks > FCX_MAX_RANKS || p->L < 1 || dc->nranks * p->L > 64 || p->cap % p->L) return cudaErrorInvalidValue;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  ctas = std::max(dc->nranks * p->L, std::min(ctas, sms));  // one CTA per expert at least; all resident: the kernel synchronises the grid
  void *args[] = {(void *)dc, (void *)p};
  return cudaLaunchCooperativeKernel((const void *)moeDispatchKernel, dim3(ctas), dim3(THREADS), args, 0, s);
}

extern "C" cudaError_t fcxSiluMul(const void *gu, void *h, const int *rows, int maxRows, int F, cudaStream_t s) {
  if (F % 8) return cudaErrorInvalidValue;
  siluMulKernel<<<592, 256, 0, s>>>((const __nv_bfloat16 *)gu, (__nv_bfloat16 *)h, rows, maxRows, F);
  return cudaGetLastError();
}

extern "C" cudaError_t fcxMoeCombine(const FcxDevComm *dc, const void *ret, const float *w, void *out, int T, int H, int K, size_t doneOff,
                                     uint64_t want, int *errFlag, cudaStream_t s) {
  if (H % 8) return cudaErrorInvalidValue;
  moeCombineKernel<<<296, 256, 0, s>>>(*dc, (const __nv_bfloat16 *)ret, w, (__nv_bfloat16 *)out, T, H, K, doneOff, want, errFlag);
  return cudaGetLastError();
}
