// Fused element-wise / normalisation / loss / optimiser kernels of the
// training step (GPT-2-style decoder, bf16 activations, fp32 arithmetic).
// The reference library has no model code at all; these kernels exist so
// that the data-parallel benchmark spends its non-GEMM time in a handful of
// bandwidth-bound passes instead of dozens of eager element-wise launches.
//
// All kernels are plain sm_100a CUDA C++: 16-byte vector accesses, one warp
// per row for the row-wise ops, grid sized as a multiple of the SM count.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <algorithm>

#include "train_ops.h"
#include "train_ops_noalloc.h"

#include <mutex>

namespace {

using bf16 = __nv_bfloat16;

__device__ __forceinline__ float warpSum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warpMax(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

struct alignas(16) Bf8 { bf16 v[8]; };

// Eight bf16 <-> eight floats.  The 16 bytes move as ONE 128-bit access wherever they live (global or shared memory:
// read field by field, a vector in shared memory turns into eight 2-byte loads); a bf16 is the upper half of a float.
__device__ __forceinline__ void unpack8(const Bf8 &p, float *f) {
  const uint4 u = *reinterpret_cast<const uint4 *>(&p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; i++) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ Bf8 pack8(const float *f) {
  uint4 u;
  uint32_t *w = reinterpret_cast<uint32_t *>(&u);
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    w[i] = *reinterpret_cast<const uint32_t *>(&h);
  }
  Bf8 p;
  *reinterpret_cast<uint4 *>(&p) = u;
  return p;
}

// Tickets of the one-launch reductions (colSumFusedKernel, lnBwdParamKernel): one counter per 64-column block.
__device__ unsigned int gColTickets[1024];
__device__ unsigned int gLnTickets[1024];

// ---------------------------------------------------------------- LayerNorm
// One warp per row, persistent over rows, 16 warps per SM (8 for rows wider than 1024).  The rows a warp will work on
// are streamed into a private three-deep ring in shared memory with cp.async two rows ahead, so that every SM keeps
// ~128 KB of loads in flight whatever the warps are computing; a lane copies exactly the 16-byte vectors that it later reads, so
// the ring needs no barrier, only cp.async.wait_group.  C is a multiple of 256 and at most 256 * MAXV.
__device__ __forceinline__ void cpAsync16(void *smemDst, const void *gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smemDst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cpAsyncCommit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cpAsyncWait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int MAXV, int STAGES, int LN_WARPS>
__global__ void __launch_bounds__(LN_WARPS * 32, 1) lnFwdKernel(const bf16 *__restrict__ x, const bf16 *__restrict__ delta,
                                                                const bf16 *__restrict__ gamma, const bf16 *__restrict__ beta,
                                                                bf16 *__restrict__ resOut, bf16 *__restrict__ y,
                                                                float *__restrict__ mean, float *__restrict__ rstd, int M, int C,
                                                                float eps) {
  extern __shared__ __align__(16) uint8_t lnSmem[];
  const int warpInCta = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp = blockIdx.x * LN_WARPS + warpInCta, nwarps = gridDim.x * LN_WARPS;
  const int nv = C / 256;  // 16-byte vectors per lane and row
  const int narr = delta ? 2 : 1;
  const size_t rowBytes = (size_t)C * 2;
  uint8_t *ring = lnSmem + (size_t)warpInCta * STAGES * 2 * rowBytes;
  auto issue = [&](int row, int st) {
    if (row < M) {
      uint8_t *dst = ring + (size_t)st * 2 * rowBytes;
#pragma unroll
      for (int i = 0; i < MAXV; i++)
        if (i < nv) {
          cpAsync16(dst + (i * 32 + lane) * 16, (const uint8_t *)(x + (size_t)row * C) + (i * 32 + lane) * 16);
          if (narr == 2) cpAsync16(dst + rowBytes + (i * 32 + lane) * 16, (const uint8_t *)(delta + (size_t)row * C) + (i * 32 + lane) * 16);
        }
    }
    cpAsyncCommit();  // an empty group past the last row keeps the group count uniform
  };
#pragma unroll
  for (int st = 0; st < STAGES - 1; st++) issue(warp + st * nwarps, st);
  int k = 0;
  for (int row = warp; row < M; row += nwarps, k++) {
    issue(row + (STAGES - 1) * nwarps, (k + STAGES - 1) % STAGES);
    cpAsyncWait<STAGES - 1>();
    const Bf8 *xr = (const Bf8 *)(ring + (size_t)(k % STAGES) * 2 * rowBytes);
    const Bf8 *dr = (const Bf8 *)((const uint8_t *)xr + rowBytes);
    float v[MAXV][8];
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; i++)
      if (i < nv) {
        unpack8(xr[i * 32 + lane], v[i]);
        if (narr == 2) {
          float d[8];
          unpack8(dr[i * 32 + lane], d);
#pragma unroll
          for (int j = 0; j < 8; j++) v[i][j] += d[j];
          // the residual stream is kept in bf16: round it here so that the
          // statistics see what the next layer will read
          Bf8 r = pack8(v[i]);
          ((Bf8 *)(resOut + (size_t)row * C))[i * 32 + lane] = r;
          unpack8(r, v[i]);
        }
#pragma unroll
        for (int j = 0; j < 8; j++) s += v[i][j];
      }
    const float mu = warpSum(s) / C;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; i++)
      if (i < nv) {
#pragma unroll
        for (int j = 0; j < 8; j++) { float d = v[i][j] - mu; q += d * d; }
      }
    const float rs = rsqrtf(warpSum(q) / C + eps);
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
#pragma unroll
    for (int i = 0; i < MAXV; i++)
      if (i < nv) {
        float g[8], b[8], o[8];
        unpack8(((const Bf8 *)gamma)[i * 32 + lane], g);
        unpack8(((const Bf8 *)beta)[i * 32 + lane], b);
#pragma unroll
        for (int j = 0; j < 8; j++) o[j] = (v[i][j] - mu) * rs * g[j] + b[j];
        ((Bf8 *)(y + (size_t)row * C))[i * 32 + lane] = pack8(o);
      }
  }
  cpAsyncWait<0>();
}

// Backward, part 1: dx = rstd * (g*dy - mean(g*dy) - xhat * mean(g*dy*xhat)) [+ dres].
// Same streaming scheme for dy and x; the residual gradient, needed only for the last step of a row, is loaded into
// registers when the row's turn begins.
template <int MAXV, int STAGES, int LN_WARPS>
__global__ void __launch_bounds__(LN_WARPS * 32, 1) lnBwdDxKernel(const bf16 *__restrict__ dy, const bf16 *__restrict__ x,
                                                                  const bf16 *__restrict__ gamma, const float *__restrict__ mean,
                                                                  const float *__restrict__ rstd, const bf16 *__restrict__ dres,
                                                                  bf16 *__restrict__ dx, int M, int C) {
  extern __shared__ __align__(16) uint8_t lnSmem[];
  const int warpInCta = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warp = blockIdx.x * LN_WARPS + warpInCta, nwarps = gridDim.x * LN_WARPS;
  const int nv = C / 256;
  const size_t rowBytes = (size_t)C * 2;
  uint8_t *ring = lnSmem + (size_t)warpInCta * STAGES * 2 * rowBytes;
  auto issue = [&](int row, int st) {
    if (row < M) {
      uint8_t *dst = ring + (size_t)st * 2 * rowBytes;
#pragma unroll
      for (int i = 0; i < MAXV; i++)
        if (i < nv) {
          const size_t off = (size_t)(i * 32 + lane) * 16;
          cpAsync16(dst + off, (const uint8_t *)(dy + (size_t)row * C) + off);
          cpAsync16(dst + rowBytes + off, (const uint8_t *)(x + (size_t)row * C) + off);
        }
    }
    cpAsyncCommit();
  };
#pragma unroll
  for (int st = 0; st < STAGES - 1; st++) issue(warp + st * nwarps, st);
  float muN = warp < M ? mean[warp] : 0.f, rsN = warp < M ? rstd[warp] : 0.f;  // statistics one row ahead
  int k = 0;
  for (int row = warp; row < M; row += nwarps, k++) {
    issue(row + (STAGES - 1) * nwarps, (k + STAGES - 1) % STAGES);
    const float mu = muN, rs = rsN;
    if (row + nwarps < M) { muN = mean[row + nwarps]; rsN = rstd[row + nwarps]; }
    Bf8 dr[MAXV];
    if (dres) {
#pragma unroll
      for (int i = 0; i < MAXV; i++)
        if (i < nv) dr[i] = ((const Bf8 *)(dres + (size_t)row * C))[i * 32 + lane];
    }
    cpAsyncWait<STAGES - 1>();
    const uint8_t *base = ring + (size_t)(k % STAGES) * 2 * rowBytes;
    const Bf8 *dyr = (const Bf8 *)base, *xr = (const Bf8 *)(base + rowBytes);
    float gy[MAXV][8], xh[MAXV][8];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < MAXV; i++)
      if (i < nv) {
        float d[8], xv[8], g[8];
        unpack8(dyr[i * 32 + lane], d);
        unpack8(xr[i * 32 + lane], xv);
        unpack8(((const Bf8 *)gamma)[i * 32 + lane], g);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          xh[i][j] = (xv[j] - mu) * rs;
          gy[i][j] = g[j] * d[j];
          s1 += gy[i][j];
          s2 += gy[i][j] * xh[i][j];
        }
      }
    s1 = warpSum(s1) / C;
    s2 = warpSum(s2) / C;
#pragma unroll
    for (int i = 0; i < MAXV; i++)
      if (i < nv) {
        float o[8];
        if (dres) unpack8(dr[i], o);
#pragma unroll
        for (int j = 0; j < 8; j++) {
          float t = rs * (gy[i][j] - s1 - xh[i][j] * s2);
          o[j] = dres ? o[j] + t : t;
        }
        ((Bf8 *)(dx + (size_t)row * C))[i * 32 + lane] = pack8(o);
      }
  }
  cpAsyncWait<0>();
}

// Backward, part 2: dgamma[c] = sum_r dy[r,c] * xhat[r,c], dbeta[c] = sum_r dy[r,c].
// A CTA owns 64 columns and one slice of the rows; partial sums go to
// `partial` ([gridDim.y][2][C], fp32 scratch); the CTA that finishes a column block last folds them into dgamma / dbeta.
__global__ void __launch_bounds__(256) lnBwdParamKernel(const bf16 *__restrict__ dy, const bf16 *__restrict__ x,
                                                        const float *__restrict__ mean, const float *__restrict__ rstd,
                                                        float *__restrict__ partial, int M, int C, bf16 *__restrict__ dgamma,
                                                        bf16 *__restrict__ dbeta, int accumulate) {
  __shared__ float redG[32][64 + 1], redB[32][64 + 1];
  const int col0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  float dg[8] = {0, 0, 0, 0, 0, 0, 0, 0}, db[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int rowsPer = (M + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * rowsPer, r1 = min(M, r0 + rowsPer);
  int r = r0 + ty;
  for (; r + 96 < r1; r += 128) {  // four rows (eight 16-byte loads) in flight per thread
    Bf8 pd[4], px[4];
    float m[4], sd[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      pd[u] = *(const Bf8 *)(dy + (size_t)(r + 32 * u) * C + col0 + tx * 8);
      px[u] = *(const Bf8 *)(x + (size_t)(r + 32 * u) * C + col0 + tx * 8);
      m[u] = mean[r + 32 * u];
      sd[u] = rstd[r + 32 * u];
    }
#pragma unroll
    for (int u = 0; u < 4; u++) {
      float d0[8], x0[8];
      unpack8(pd[u], d0);
      unpack8(px[u], x0);
#pragma unroll
      for (int k = 0; k < 8; k++) {
        dg[k] += d0[k] * (x0[k] - m[u]) * sd[u];
        db[k] += d0[k];
      }
    }
  }
  for (; r < r1; r += 32) {
    float d0[8], x0[8];
    unpack8(*(const Bf8 *)(dy + (size_t)r * C + col0 + tx * 8), d0);
    unpack8(*(const Bf8 *)(x + (size_t)r * C + col0 + tx * 8), x0);
    const float m0 = mean[r], s0 = rstd[r];
#pragma unroll
    for (int k = 0; k < 8; k++) {
      dg[k] += d0[k] * (x0[k] - m0) * s0;
      db[k] += d0[k];
    }
  }
#pragma unroll
  for (int k = 0; k < 8; k++) { redG[ty][tx * 8 + k] = dg[k]; redB[ty][tx * 8 + k] = db[k]; }
  __syncthreads();
  if (threadIdx.x < 128) {
    const int c = threadIdx.x & 63;
    const bool isB = threadIdx.x >= 64;
    float s = 0.f;
#pragma unroll 8
    for (int j = 0; j < 32; j++) s += isB ? redB[j][c] : redG[j][c];
    partial[((size_t)blockIdx.y * 2 + (isB ? 1 : 0)) * C + col0 + c] = s;
    __threadfence();
  }
  if (dgamma == nullptr) return;  // partial sums only
  // the CTA that finishes this 64-column block last folds them (ticket scheme of colSumFusedKernel)
  __shared__ unsigned int ticket;
  __syncthreads();
  if (threadIdx.x == 0) ticket = atomicAdd(&gLnTickets[blockIdx.x], 1u);
  __syncthreads();
  if (ticket != gridDim.y - 1) return;
  __threadfence();
  {
    // 128 outputs (64 dgamma, 64 dbeta), two halves of the partial sums per output
    const int o = threadIdx.x & 127, half = threadIdx.x >> 7, c = o & 63;
    const bool isB = o >= 64;
    float s = 0.f;
    for (int p = half; p < (int)gridDim.y; p += 2) s += __ldcg(partial + ((size_t)p * 2 + (isB ? 1 : 0)) * C + col0 + c);
    __syncthreads();
    float *fold = &redB[0][0];
    fold[half * 128 + o] = s;
    __syncthreads();
    if (threadIdx.x < 128) {
      s = fold[o] + fold[128 + o];
      bf16 *dst = isB ? dbeta + col0 + c : dgamma + col0 + c;
      if (accumulate) s += __bfloat162float(*dst);
      *dst = __float2bfloat16_rn(s);
    }
  }
  if (threadIdx.x == 0) gLnTickets[blockIdx.x] = 0;
}

// ---------------------------------------------------------------- bias + GELU (tanh form)
__device__ __forceinline__ float fastTanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float geluF(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  return 0.5f * x * (1.f + fastTanh(k0 * (x + k1 * x * x * x)));
}
__device__ __forceinline__ float geluGrad(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x), t = fastTanh(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k0 * (1.f + 3.f * k1 * x * x);
}

// y = gelu(x + bias); x is [M, C].  Each thread keeps four 16-byte loads in flight.
__global__ void __launch_bounds__(256) biasGeluFwdKernel(const bf16 *__restrict__ x, const bf16 *__restrict__ bias,
                                                         bf16 *__restrict__ y, size_t nvec, int C) {
  const int cv = C / 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < nvec; i += 4 * stride) {
    Bf8 v[4];
#pragma unroll
    for (int j = 0; j < 4; j++) v[j] = ((const Bf8 *)x)[i + j * stride];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float a[8], b[8];
      unpack8(v[j], a);
      unpack8(((const Bf8 *)bias)[(i + j * stride) % cv], b);
#pragma unroll
      for (int k = 0; k < 8; k++) a[k] = geluF(a[k] + b[k]);
      ((Bf8 *)y)[i + j * stride] = pack8(a);
    }
  }
  for (; i < nvec; i += stride) {
    float a[8], b[8];
    unpack8(((const Bf8 *)x)[i], a);
    unpack8(((const Bf8 *)bias)[i % cv], b);
#pragma unroll
    for (int k = 0; k < 8; k++) a[k] = geluF(a[k] + b[k]);
    ((Bf8 *)y)[i] = pack8(a);
  }
}

// dx = dy * gelu'(x + bias)
__global__ void __launch_bounds__(256) biasGeluBwdKernel(const bf16 *__restrict__ dy, const bf16 *__restrict__ x,
                                                         const bf16 *__restrict__ bias, bf16 *__restrict__ dx, size_t nvec, int C) {
  const int cv = C / 8;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + stride < nvec; i += 2 * stride) {
    Bf8 xv[2], dv[2];
#pragma unroll
    for (int j = 0; j < 2; j++) { xv[j] = ((const Bf8 *)x)[i + j * stride]; dv[j] = ((const Bf8 *)dy)[i + j * stride]; }
#pragma unroll
    for (int j = 0; j < 2; j++) {
      float a[8], b[8], d[8];
      unpack8(xv[j], a);
      unpack8(dv[j], d);
      unpack8(((const Bf8 *)bias)[(i + j * stride) % cv], b);
#pragma unroll
      for (int k = 0; k < 8; k++) d[k] *= geluGrad(a[k] + b[k]);
      ((Bf8 *)dx)[i + j * stride] = pack8(d);
    }
  }
  for (; i < nvec; i += stride) {
    float a[8], b[8], d[8];
    unpack8(((const Bf8 *)x)[i], a);
    unpack8(((const Bf8 *)bias)[i % cv], b);
    unpack8(((const Bf8 *)dy)[i], d);
#pragma unroll
    for (int k = 0; k < 8; k++) d[k] *= geluGrad(a[k] + b[k]);
    ((Bf8 *)dx)[i] = pack8(d);
  }
}

// Column sums of a [M, C] bf16 matrix (bias gradients).  Each CTA owns 64
// columns and a slice of rows; partials go to fp32 scratch [gridDim.y][C].
__global__ void __launch_bounds__(256) colSumKernel(const bf16 *__restrict__ a, float *__restrict__ partial, int M, int C) {
  const int col0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;  // 8 vector columns x 32 row lanes
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int rowsPer = (M + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * rowsPer, r1 = min(M, r0 + rowsPer);
  int r = r0 + ty;
  for (; r + 96 < r1; r += 128) {  // four rows in flight per thread
    Bf8 p[4];
#pragma unroll
    for (int u = 0; u < 4; u++) p[u] = *(const Bf8 *)(a + (size_t)(r + 32 * u) * C + col0 + tx * 8);
#pragma unroll
    for (int u = 0; u < 4; u++) {
      float v[8];
      unpack8(p[u], v);
#pragma unroll
      for (int k = 0; k < 8; k++) acc[k] += v[k];
    }
  }
  for (; r < r1; r += 32) {
    float v[8];
    unpack8(*(const Bf8 *)(a + (size_t)r * C + col0 + tx * 8), v);
#pragma unroll
    for (int k = 0; k < 8; k++) acc[k] += v[k];
  }
  // reduce over the 32 row lanes: lanes with equal tx live in different warps, go through shared memory
  __shared__ float red[32][64 + 1];
#pragma unroll
  for (int k = 0; k < 8; k++) red[ty][tx * 8 + k] = acc[k];
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll 8
    for (int j = 0; j < 32; j++) s += red[j][threadIdx.x];
    partial[(size_t)blockIdx.y * C + col0 + threadIdx.x] = s;
  }
}

__global__ void colSumReduceKernel(const float *__restrict__ partial, int nparts, int C, bf16 *__restrict__ out, int accumulate) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float s = 0.f;
  for (int p = 0; p < nparts; p++) s += partial[(size_t)p * C + c];
  if (accumulate) s += __bfloat162float(out[c]);
  out[c] = __float2bfloat16_rn(s);
}

// Both steps of the column sum in ONE launch: the CTA that finishes a 64-column block last (a ticket per block, taken
// after the partial sums are visible) folds the block's partial sums and writes the result.  The tickets live in the
// library image and return to zero by themselves; concurrent calls on one device would share them, so calls must be
// stream-ordered (they are: the backward pass runs on one stream).
__global__ void __launch_bounds__(256) colSumFusedKernel(const bf16 *__restrict__ a, float *__restrict__ partial, bf16 *__restrict__ out,
                                                         int M, int C, int accumulate) {
  const int col0 = blockIdx.x * 64;
  const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int rowsPer = (M + gridDim.y - 1) / gridDim.y;
  const int r0 = blockIdx.y * rowsPer, r1 = min(M, r0 + rowsPer);
  int r = r0 + ty;
  for (; r + 96 < r1; r += 128) {
    Bf8 p[4];
#pragma unroll
    for (int u = 0; u < 4; u++) p[u] = *(const Bf8 *)(a + (size_t)(r + 32 * u) * C + col0 + tx * 8);
#pragma unroll
    for (int u = 0; u < 4; u++) {
      float v[8];
      unpack8(p[u], v);
#pragma unroll
      for (int k = 0; k < 8; k++) acc[k] += v[k];
    }
  }
  for (; r < r1; r += 32) {
    float v[8];
    unpack8(*(const Bf8 *)(a + (size_t)r * C + col0 + tx * 8), v);
#pragma unroll
    for (int k = 0; k < 8; k++) acc[k] += v[k];
  }
  __shared__ float red[32][64 + 1];
  __shared__ unsigned int ticket;
#pragma unroll
  for (int k = 0; k < 8; k++) red[ty][tx * 8 + k] = acc[k];
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll 8
    for (int j = 0; j < 32; j++) s += red[j][threadIdx.x];
    partial[(size_t)blockIdx.y * C + col0 + threadIdx.x] = s;
    __threadfence();
  }
  __syncthreads();
  if (threadIdx.x == 0) ticket = atomicAdd(&gColTickets[blockIdx.x], 1u);
  __syncthreads();
  if (ticket != gridDim.y - 1) return;
  __threadfence();
  // last CTA of this column block: four groups of 64 threads fold a quarter of the partial sums each
  const int c = threadIdx.x & 63, grp = threadIdx.x >> 6;
  float s = 0.f;
  for (int p = grp; p < (int)gridDim.y; p += 4) s += __ldcg(partial + (size_t)p * C + col0 + c);
  __syncthreads();  // red is reused
  red[grp][c] = s;
  __syncthreads();
  if (threadIdx.x < 64) {
    s = red[0][c] + red[1][c] + red[2][c] + red[3][c];
    if (accumulate) s += __bfloat162float(out[col0 + c]);
    out[col0 + c] = __float2bfloat16_rn(s);
  }
  if (threadIdx.x == 0) gColTickets[blockIdx.x] = 0;
}

// ---------------------------------------------------------------- softmax cross-entropy
// One CTA per row of logits [M, Vpad] (V valid columns).  Writes the loss of
// the row and overwrites the logits with (softmax - onehot) * gradScale.
__global__ void __launch_bounds__(1024) ceFwdBwdKernel(bf16 *__restrict__ logits, const int64_t *__restrict__ targets,
                                                       float *__restrict__ losses, int V, int Vpad, float gradScale) {
  __shared__ float red[32];
  __shared__ float bcast;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5, nw = blockDim.x >> 5;
  bf16 *lr = logits + (size_t)row * Vpad;
  const int nvec = V / 8;
  const int tgt = (int)targets[row];
  // read before anything in the row is overwritten by the gradient pass
  const float tgtLogit = (tgt >= 0 && tgt < V) ? __bfloat162float(lr[tgt]) : 0.f;
  float mx = -INFINITY;
  for (int i = tid; i < nvec; i += blockDim.x) {
    float v[8];
    unpack8(((const Bf8 *)lr)[i], v);
#pragma unroll
    for (int k = 0; k < 8; k++) mx = fmaxf(mx, v[k]);
  }
  for (int i = nvec * 8 + tid; i < V; i += blockDim.x) mx = fmaxf(mx, __bfloat162float(lr[i]));
  mx = warpMax(mx);
  if (lane == 0) red[wid] = mx;
  __syncthreads();
  if (wid == 0) {
    float v = lane < nw ? red[lane] : -INFINITY;
    v = warpMax(v);
    if (lane == 0) bcast = v;
  }
  __syncthreads();
  mx = bcast;
  float sum = 0.f;
  for (int i = tid; i < nvec; i += blockDim.x) {
    float v[8];
    unpack8(((const Bf8 *)lr)[i], v);
#pragma unroll
    for (int k = 0; k < 8; k++) sum += __expf(v[k] - mx);
  }
  for (int i = nvec * 8 + tid; i < V; i += blockDim.x) sum += __expf(__bfloat162float(lr[i]) - mx);
  sum = warpSum(sum);
  __syncthreads();
  if (lane == 0) red[wid] = sum;
  __syncthreads();
  if (wid == 0) {
    float v = lane < nw ? red[lane] : 0.f;
    v = warpSum(v);
    if (lane == 0) bcast = v;
  }
  __syncthreads();
  sum = bcast;
  const float inv = 1.f / sum;
  if (tid == 0) losses[row] = tgt >= 0 ? (logf(sum) + mx - tgtLogit) : 0.f;
  const float gs = tgt >= 0 ? gradScale : 0.f;
  for (int i = tid; i < nvec; i += blockDim.x) {
    float v[8];
    unpack8(((const Bf8 *)lr)[i], v);
#pragma unroll
    for (int k = 0; k < 8; k++) {
      float p = __expf(v[k] - mx) * inv;
      v[k] = (p - ((i * 8 + k) == tgt ? 1.f : 0.f)) * gs;
    }
    ((Bf8 *)lr)[i] = pack8(v);
  }
  for (int i = nvec * 8 + tid; i < Vpad; i += blockDim.x) {
    float g = 0.f;
    if (i < V) g = (__expf(__bfloat162float(lr[i]) - mx) * inv - (i == tgt ? 1.f : 0.f)) * gs;
    lr[i] = __float2bfloat16_rn(g);
  }
}

// The same for rows that fit twice into shared memory (Vpad <= 56 K): persistent CTAs, one per SM, walk the rows; the
// row a CTA works on lies in shared memory, and the next row streams in with cp.async during the three passes over the
// current one, so the logits are read from DRAM exactly once and the reads never wait for the arithmetic.  A thread
// copies exactly the vectors it reads itself, so the only synchronisation of the ring is cp.async.wait_group.
__global__ void __launch_bounds__(1024, 1) ceFwdBwdStreamKernel(bf16 *__restrict__ logits, const int64_t *__restrict__ targets,
                                                                float *__restrict__ losses, int M, int V, int Vpad,
                                                                float gradScale) {
  extern __shared__ __align__(16) uint8_t ceSmem[];
  __shared__ float red[2][32];
  __shared__ float bcast[2];
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int nvecPad = Vpad / 8;
  const size_t rowBytes = (size_t)Vpad * 2;
  auto issue = [&](int row, int b) {
    if (row < M) {
      const uint8_t *src = (const uint8_t *)(logits + (size_t)row * Vpad);
      uint8_t *dst = ceSmem + (size_t)b * rowBytes;
      for (int i = tid; i < nvecPad; i += 1024) cpAsync16(dst + (size_t)i * 16, src + (size_t)i * 16);
    }
    cpAsyncCommit();
  };
  issue(blockIdx.x, 0);
  int k = 0;
  for (int row = blockIdx.x; row < M; row += gridDim.x, k++) {
    issue(row + gridDim.x, (k + 1) & 1);
    bf16 *lr = logits + (size_t)row * Vpad;
    const int tgt = (int)targets[row];
    const float tgtLogit = (tgt >= 0 && tgt < V) ? __bfloat162float(lr[tgt]) : 0.f;  // before the row is overwritten
    cpAsyncWait<1>();
    Bf8 *sr = (Bf8 *)(ceSmem + (size_t)(k & 1) * rowBytes);
    // pass 1: row maximum, on packed bf16 pairs
    __nv_bfloat162 mx2 = __floats2bfloat162_rn(-INFINITY, -INFINITY);
    float mx = -INFINITY;
    for (int i = tid; i < V / 8; i += 1024) {
      const Bf8 pv = sr[i];
      const __nv_bfloat162 *h = (const __nv_bfloat162 *)&pv;
#pragma unroll
      for (int j = 0; j < 4; j++) mx2 = __hmax2(mx2, h[j]);
    }
    for (int i = V / 8 + tid; i < nvecPad; i += 1024) {
      float v[8];
      unpack8(sr[i], v);
#pragma unroll
      for (int j = 0; j < 8; j++)
        if (i * 8 + j < V) mx = fmaxf(mx, v[j]);
    }
    mx = fmaxf(mx, fmaxf(__low2float(mx2), __high2float(mx2)));
    mx = warpMax(mx);
    if (lane == 0) red[0][wid] = mx;
    __syncthreads();
    if (wid == 0) {
      float v = warpMax(red[0][lane]);
      if (lane == 0) bcast[0] = v;
    }
    __syncthreads();
    mx = bcast[0];
    // pass 2: e = exp(v - max), summed in fp32 and left in the row buffer as bf16 (columns past V become 0), so that
    // the gradient pass needs no second exponential
    const float kLog2e = 1.4426950408889634f, mxl = mx * kLog2e;
    float sum = 0.f, sumB = 0.f;
    const int nvecFull = V / 8;
    for (int i = tid; i < nvecFull; i += 1024) {  // whole vectors: no masks, two independent partial sums
      float v[8];
      unpack8(sr[i], v);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        float e;
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(v[j], kLog2e, -mxl)));
        if (j & 1) sumB += e; else sum += e;
        v[j] = e;
      }
      sr[i] = pack8(v);
    }
    for (int i = nvecFull + tid; i < nvecPad; i += 1024) {  // the ragged vector and the padding behind it
      float v[8];
      unpack8(sr[i], v);
#pragma unroll
      for (int j = 0; j < 8; j++) {
        float e = 0.f;
        if (i * 8 + j < V) asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(fmaf(v[j], kLog2e, -mxl)));
        sum += e;
        v[j] = e;
      }
      sr[i] = pack8(v);
    }
    sum += sumB;
    sum = warpSum(sum);
    if (lane == 0) red[1][wid] = sum;
    __syncthreads();
    if (wid == 0) {
      float v = warpSum(red[1][lane]);
      if (lane == 0) bcast[1] = v;
    }
    __syncthreads();
    sum = bcast[1];
    if (tid == 0) losses[row] = tgt >= 0 ? (logf(sum) + mx - tgtLogit) : 0.f;
    // pass 3: gradient = (e / sum - onehot) * scale
    const float gs = tgt >= 0 ? gradScale : 0.f, scale = gs / sum;
    const int tgtVec = (tgt >= 0 && tgt < V) ? (tgt >> 3) : -1;
    for (int i = tid; i < nvecPad; i += 1024) {
      float v[8];
      unpack8(sr[i], v);
#pragma unroll
      for (int j = 0; j < 8; j++) v[j] *= scale;
      ((Bf8 *)lr)[i] = pack8(v);
    }
    // the target column, by the thread that stored the vector around it a moment ago
    if (tgtVec >= 0 && (tgtVec & 1023) == tid)
      lr[tgt] = __float2bfloat16_rn(__bfloat162float(((const bf16 *)sr)[tgt]) * scale - gs);
    // red / bcast are rewritten only after the next row's first barrier pair; nothing else is shared between rows
  }
  cpAsyncWait<0>();
}

// ---------------------------------------------------------------- AdamW on flat buffers
// master (fp32) is the truth; param (bf16) is refreshed from it.  The gradient
// is read once and cleared, so no separate zero_grad pass is needed.
__global__ void __launch_bounds__(256) adamwKernel(float *__restrict__ master, bf16 *__restrict__ param, bf16 *__restrict__ grad,
                                                   float *__restrict__ m, float *__restrict__ v, size_t n, float lr, float b1,
                                                   float b2, float eps, float wd, float bc1, float bc2, float gradScale,
                                                   int zeroGrad, const int *__restrict__ stepDev) {
  if (stepDev) {
    // step counter kept on the device so that a captured graph stays exact
    float st = (float)(*stepDev);
    bc1 = 1.f - powf(b1, st);
    bc2 = 1.f - powf(b2, st);
  }
  const size_t nvec = n / 8;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    float g[8];
    unpack8(((const Bf8 *)grad)[i], g);
    float4 w0 = ((float4 *)master)[2 * i], w1 = ((float4 *)master)[2 * i + 1];
    float4 m0 = ((float4 *)m)[2 * i], m1 = ((float4 *)m)[2 * i + 1];
    float4 v0 = ((float4 *)v)[2 * i], v1 = ((float4 *)v)[2 * i + 1];
    float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int k = 0; k < 8; k++) {
      float gk = g[k] * gradScale;
      mm[k] = b1 * mm[k] + (1.f - b1) * gk;
      vv[k] = b2 * vv[k] + (1.f - b2) * gk * gk;
      float upd = (mm[k] / bc1) / (sqrtf(vv[k] / bc2) + eps);
      w[k] = w[k] - lr * (upd + wd * w[k]);
    }
    ((float4 *)master)[2 * i] = make_float4(w[0], w[1], w[2], w[3]);
    ((float4 *)master)[2 * i + 1] = make_float4(w[4], w[5], w[6], w[7]);
    ((float4 *)m)[2 * i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    ((float4 *)m)[2 * i + 1] = make_float4(mm[4], mm[5], mm[6], mm[7]);
    ((float4 *)v)[2 * i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    ((float4 *)v)[2 * i + 1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
    ((Bf8 *)param)[i] = pack8(w);
    if (zeroGrad) {
      Bf8 z;
#pragma unroll
      for (int k = 0; k < 8; k++) z.v[k] = __float2bfloat16_rn(0.f);
      ((Bf8 *)grad)[i] = z;
    }
  }
  // tail (n not a multiple of 8)
  if (blockIdx.x == 0) {
    for (size_t i = nvec * 8 + threadIdx.x; i < n; i += blockDim.x) {
      float gk = __bfloat162float(grad[i]) * gradScale;
      float mk = b1 * m[i] + (1.f - b1) * gk, vk = b2 * v[i] + (1.f - b2) * gk * gk;
      float wk = master[i];
      wk = wk - lr * ((mk / bc1) / (sqrtf(vk / bc2) + eps) + wd * wk);
      m[i] = mk; v[i] = vk; master[i] = wk;
      param[i] = __float2bfloat16_rn(wk);
      if (zeroGrad) grad[i] = __float2bfloat16_rn(0.f);
    }
  }
}

int smCount() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace

// ---------------------------------------------------------------- launchers

extern "C" {

int fcxLnPartials(int M) { return max(1, min(32, M / 128)); }

cudaError_t fcxLayerNormFwd(const void *x, const void *delta, const void *gamma, const void *beta, void *resOut, void *y,
                            float *mean, float *rstd, int M, int C, float eps, cudaStream_t s) {
  if (C % 256 != 0 || C > 256 * 8) return cudaErrorInvalidValue;
  // rows up to 1024 wide: 16 warps per SM (the arithmetic needs the issue slots), wider rows: 8 warps; either way
  // warps x 3-deep ring x (x, delta) x row bytes <= 192 KB
  const int warps = C <= 1024 ? 16 : 8;
  const int grid = std::max(1, std::min(smCount(), (M + warps - 1) / warps));
  const size_t smem = (size_t)warps * 3 * 2 * C * 2;
  auto run = [&](auto kernel) {
    // both instantiations have the same pointer type, so this lambda exists once: remember the kernels by address
    static thread_local const void *configured[2] = {nullptr, nullptr};
    const void *id = (const void *)kernel;
    if (configured[0] != id && configured[1] != id) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return e;
      configured[configured[0] ? 1 : 0] = id;
    }
    kernel<<<grid, warps * 32, smem, s>>>((const bf16 *)x, (const bf16 *)delta, (const bf16 *)gamma, (const bf16 *)beta, (bf16 *)resOut,
                                          (bf16 *)y, mean, rstd, M, C, eps);
    return cudaGetLastError();
  };
  return C <= 1024 ? run(lnFwdKernel<4, 3, 16>) : run(lnFwdKernel<8, 3, 8>);
}

// `partial` must hold fcxLnPartials(M) * 2 * C floats.
cudaError_t fcxLayerNormBwd(const void *dy, const void *x, const void *gamma, const float *mean, const float *rstd,
                            const void *dres, void *dx, void *dgamma, void *dbeta, float *partial, int M, int C, int accumulate,
                            cudaStream_t s) {
  if (C % 256 != 0 || C > 256 * 8) return cudaErrorInvalidValue;
  const int warps = C <= 1024 ? 16 : 8;
  const int grid = std::max(1, std::min(smCount(), (M + warps - 1) / warps));
  const size_t smem = (size_t)warps * 3 * 2 * C * 2;  // warps x 3-deep ring x (dy, x) x row bytes <= 192 KB
  auto run = [&](auto kernel) {
    // both instantiations have the same pointer type, so this lambda exists once: remember the kernels by address
    static thread_local const void *configured[2] = {nullptr, nullptr};
    const void *id = (const void *)kernel;
    if (configured[0] != id && configured[1] != id) {
      cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
      if (e != cudaSuccess) return e;
      configured[configured[0] ? 1 : 0] = id;
    }
    kernel<<<grid, warps * 32, smem, s>>>((const bf16 *)dy, (const bf16 *)x, (const bf16 *)gamma, mean, rstd, (const bf16 *)dres, (bf16 *)dx,
                                          M, C);
    return cudaGetLastError();
  };
  cudaError_t e = C <= 1024 ? run(lnBwdDxKernel<4, 3, 16>) : run(lnBwdDxKernel<8, 3, 8>);
  if (e != cudaSuccess) return e;
  int parts = fcxLnPartials(M);
  // C <= 2048 here, so the 64-column blocks fit the ticket array: parameter partials and their reduction in one launch
  lnBwdParamKernel<<<dim3(C / 64, parts), 256, 0, s>>>((const bf16 *)dy, (const bf16 *)x, mean, rstd, partial, M, C, (bf16 *)dgamma,
                                                       (bf16 *)dbeta, accumulate);
  return cudaGetLastError();
}

cudaError_t fcxBiasGeluFwd(const void *x, const void *bias, void *y, size_t M, int C, cudaStream_t s) {
  if (C % 8 != 0) return cudaErrorInvalidValue;
  size_t nvec = M * C / 8;
  int grid = (int)std::min<size_t>((nvec + 255) / 256, (size_t)smCount() * 8);
  biasGeluFwdKernel<<<grid, 256, 0, s>>>((const bf16 *)x, (const bf16 *)bias, (bf16 *)y, nvec, C);
  return cudaGetLastError();
}

cudaError_t fcxBiasGeluBwd(const void *dy, const void *x, const void *bias, void *dx, size_t M, int C, cudaStream_t s) {
  if (C % 8 != 0) return cudaErrorInvalidValue;
  size_t nvec = M * C / 8;
  int grid = (int)std::min<size_t>((nvec + 255) / 256, (size_t)smCount() * 8);
  biasGeluBwdKernel<<<grid, 256, 0, s>>>((const bf16 *)dy, (const bf16 *)x, (const bf16 *)bias, (bf16 *)dx, nvec, C);
  return cudaGetLastError();
}

int fcxColSumPartials(int M) { return max(1, min(32, M / 256)); }

// `partial` must hold fcxColSumPartials(M) * C floats.
cudaError_t fcxColSum(const void *a, void *out, float *partial, int M, int C, int accumulate, cudaStream_t s) {
  if (C % 64 != 0) return cudaErrorInvalidValue;
  int parts = fcxColSumPartials(M);
  if (C / 64 <= 1024) {
    colSumFusedKernel<<<dim3(C / 64, parts), 256, 0, s>>>((const bf16 *)a, partial, (bf16 *)out, M, C, accumulate);
    return cudaGetLastError();
  }
  colSumKernel<<<dim3(C / 64, parts), 256, 0, s>>>((const bf16 *)a, partial, M, C);
  colSumReduceKernel<<<(C + 255) / 256, 256, 0, s>>>(partial, parts, C, (bf16 *)out, accumulate);
  return cudaGetLastError();
}

cudaError_t fcxCrossEntropyFwdBwd(void *logits, const int64_t *targets, float *losses, int M, int V, int Vpad, float gradScale,
                                  cudaStream_t s) {
  if (Vpad % 8 != 0 || V > Vpad) return cudaErrorInvalidValue;
  const size_t ring = (size_t)Vpad * 2 * 2;
  if (ring <= 224 * 1024 && ((uintptr_t)logits & 15) == 0) {
    static thread_local bool attr = false;
    if (!attr) {
      cudaError_t e = cudaFuncSetAttribute(ceFwdBwdStreamKernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
      if (e != cudaSuccess) return e;
      attr = true;
    }
    ceFwdBwdStreamKernel<<<std::min(M, smCount()), 1024, ring, s>>>((bf16 *)logits, targets, losses, M, V, Vpad, gradScale);
  } else {
    ceFwdBwdKernel<<<M, 1024, 0, s>>>((bf16 *)logits, targets, losses, V, Vpad, gradScale);
  }
  return cudaGetLastError();
}

cudaError_t fcxAdamW(float *master, void *param, void *grad, float *m, float *v, size_t n, float lr, float b1, float b2, float eps,
                     float wd, int step, float gradScale, int zeroGrad, const int *stepDev, cudaStream_t s) {
  float bc1 = 1.f - powf(b1, (float)step), bc2 = 1.f - powf(b2, (float)step);
  int grid = (int)std::min<size_t>((n / 8 + 255) / 256 + 1, (size_t)smCount() * 8);
  adamwKernel<<<grid, 256, 0, s>>>(master, (bf16 *)param, (bf16 *)grad, m, v, n, lr, b1, b2, eps, wd, bc1, bc2, gradScale, zeroGrad, stepDev);
  return cudaGetLastError();
}

}  // extern "C"

// ---------------------------------------------------------------- allocation-free column sum
// (contract in train_ops_noalloc.h)

// Scratch that belongs to the library image.  In host code this name is only
// a handle for the runtime; the address a kernel can use is obtained with
// cudaGetSymbolAddress below.
static __device__ __align__(256) float gNoAllocScratch[FCX_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float *gScratchAddr[kMaxDevices];
std::mutex gScratchMu;

// Device address of the scratch array on the current device, looked up once per device.
int scratchForCurrentDevice(float **out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return (int)cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(gScratchMu);
  if (!gScratchAddr[dev]) {
    float *p = nullptr;
    e = cudaGetSymbolAddress((void **)&p, gNoAllocScratch);
    if (e != cudaSuccess) return (int)e;
    gScratchAddr[dev] = p;
  }
  *out = gScratchAddr[dev];
  return 0;
}
}  // namespace

extern "C" int fcxColSumNoAlloc(const void *a, void *out, int M, int C, int accumulate, cudaStream_t stream) {
  if (!a || !out) return FCX_NOALLOC_NULL_POINTER;
  if (M <= 0 || C <= 0 || C % 64 != 0) return FCX_NOALLOC_BAD_SHAPE;
  // the kernels read `a` in 16-byte vectors; a raw-pointer caller with an odd offset gets a code, not a fault
  if (((uintptr_t)a & 15u) != 0 || ((uintptr_t)out & 15u) != 0) return FCX_NOALLOC_MISALIGNED;
  const int parts = fcxColSumPartials(M);
  if ((long long)parts * C > (long long)FCX_NOALLOC_MAX_FLOATS) return FCX_NOALLOC_TOO_LARGE;
  float *scratch = nullptr;
  int rc = scratchForCurrentDevice(&scratch);
  if (rc != 0) return rc;
  // Every partial[p][c] with p < parts, c < C is written by colSumKernel before
  // colSumReduceKernel reads it, so stale contents of earlier calls are harmless.
  colSumKernel<<<dim3(C / 64, parts), 256, 0, stream>>>((const bf16 *)a, scratch, M, C);
  colSumReduceKernel<<<(C + 255) / 256, 256, 0, stream>>>(scratch, parts, C, (bf16 *)out, accumulate);
  return (int)cudaGetLastError();
}

extern "C" const char *fcxNoAllocErrorString(int code) {
  switch (code) {
    case 0: return "success";
    case FCX_NOALLOC_TOO_LARGE: return "shape needs more than the built-in scratch (partials x C > 262144 floats); use fcxColSum with your own scratch";
    case FCX_NOALLOC_BAD_SHAPE: return "M and C must be positive and C a multiple of 64";
    case FCX_NOALLOC_NULL_POINTER: return "input and output pointers must not be null";
    case FCX_NOALLOC_MISALIGNED: return "input and output pointers must be 16-byte aligned";
    default: return code > 0 ? cudaGetErrorString((cudaError_t)code) : "unknown code";
  }
}
