// Block-scaled fp8 (e4m3) GEMM on tcgen05: C[M,N] (bf16) = (A_q * sa) x (B_q * sb)^T.
//
// Scaling granularity is the one used for fp8 training of large transformer
// layers: activations carry one fp32 scale per row and 128 columns of K
// (sa[K/128][M]), weights one per 128x128 block (sb[ceil(N/128)][K/128]).
// The tensor cores cannot apply such scales themselves, so every 128-deep
// slice of K is multiplied into its own TMEM accumulator (tcgen05.mma
// kind::f8f6f4, fp32 accumulate) and the epilogue warps fold it into
// registers as acc += sa[row,kb] * sb[nb,kb] * partial while the next slices
// are already being multiplied: four TMEM accumulators of 128 columns rotate
// between the MMA issuer and the epilogue.
//
// The reference has no GEMM; its users would pair flagcx collectives with a
// vendor scaled matmul.
//
// One CTA per SM, 384 threads, persistent over 128x128 tiles:
//   warp 0     TMA producer (A and B slices of 128x128 bytes, 128-byte swizzle, 6 stages, no multicast)
//   warp 1     MMA issuer (4 x K32 instructions per slice)
//   warp 2     TMEM allocation
//   warps 4-11 promotion + epilogue: warp w reads TMEM lanes 32*(w%4).. (one output row per thread) and the
//              column half (w-4)/4 of the tile, 64 fp32 accumulators per thread, two TMEM loads in flight
// Every wait is bounded; a wait that gives up sets the error flag and the kernel drains and returns.
#include <algorithm>
#include <cstdlib>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_fp8_sm100.h"
#include "tcgen05.cuh"

namespace {

using namespace fcxmma;

constexpr int BM = 128, BN = 128, BK = 128, STAGES = 6, ACC_BUFS = 4;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_WARPS = 8;
constexpr int EPI_BYTES = EPI_WARPS * 32 * 128;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
constexpr int THREADS = 384;

struct Params {
  int M, N, K;
  const float *sa;  // [K/128][M]
  const float *sb;  // [ceil(N/128)][K/128]
  __nv_bfloat16 *c;
  int ldc, group;
  int *errFlag;
};

// D fp32, A and B e4m3 (format 0), both K-major, M = 128, N = 128
__device__ __forceinline__ constexpr uint32_t instrDescF8() { return (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24); }

__device__ __forceinline__ void tileCoord(const Params &p, int nM, int nN, int t, int *mb, int *nb) {
  const int perBand = p.group * nN, band = t / perBand, first = band * p.group;
  const int rowsHere = min(p.group, nM - first), within = t - band * perBand;
  *mb = first + within % rowsHere;
  *nb = within / rowsHere;
}

__global__ void __launch_bounds__(THREADS, 1) gemmFp8Kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                            const Params p) {
  extern __shared__ uint8_t smemRaw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *err = p.errFlag;
  uint8_t *tiles = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  uint8_t *epiStage = tiles + STAGES * STAGE_BYTES;
  uint64_t *bars = (uint64_t *)(epiStage + EPI_BYTES);
  uint64_t *fullBar = bars, *emptyBar = bars + STAGES, *tmemFull = bars + 2 * STAGES, *tmemEmpty = bars + 2 * STAGES + ACC_BUFS;
  uint32_t *tmemBaseSlot = (uint32_t *)(bars + 2 * STAGES + 2 * ACC_BUFS);

  const int nN = (p.N + BN - 1) / BN, nM = (p.M + BM - 1) / BM, nTiles = nN * nM, nK = p.K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbarInit(&fullBar[s], 1); mbarInit(&emptyBar[s], 1); }
    for (int b = 0; b < ACC_BUFS; b++) { mbarInit(&tmemFull[b], 1); mbarInit(&tmemEmpty[b], EPI_WARPS); }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmemBaseSlot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fenceBefore();
  __syncthreads();
  fenceAfter();
  const uint32_t tmemBase = *tmemBaseSlot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < nTiles && ok; t += gridDim.x) {
        int mb, nb;
        tileCoord(p, nM, nN, t, &mb, &nb);
        for (int kb = 0; kb < nK; kb++) {
          if (!mbarWait(&emptyBar[stage], phase ^ 1, err)) { ok = false; break; }
          mbarExpectTx(&fullBar[stage], STAGE_BYTES);
          uint8_t *sa = tiles + stage * STAGE_BYTES, *sb = sa + A_BYTES;
          tmaLoad2d(sa, &tmA, kb * BK, mb * BM, &fullBar[stage]);
          tmaLoad2d(sb, &tmB, kb * BK, nb * BN, &fullBar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, buf = 0;
      uint32_t phase = 0, accPhase = 0;
      bool ok = true;
      const uint32_t idesc = instrDescF8();
      for (int t = blockIdx.x; t < nTiles && ok; t += gridDim.x) {
        for (int kb = 0; kb < nK; kb++) {
          if (!mbarWait(&tmemEmpty[buf], accPhase ^ 1, err)) { ok = false; break; }
          if (!mbarWait(&fullBar[stage], phase, err)) { ok = false; break; }
          fenceAfter();
          const uint32_t dTmem = tmemBase + (uint32_t)buf * BN;
          const uint32_t sa = smemAddr(tiles + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 32; k++)  // 32 fp8 = 32 bytes further along K inside the 128-byte swizzle row
            mmaF8(dTmem, smemDesc(sa + k * 32), smemDesc(sb + k * 32), idesc, k > 0 ? 1u : 0u);
          mmaCommit(&emptyBar[stage]);
          mmaCommit(&tmemFull[buf]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
          if (++buf == ACC_BUFS) { buf = 0; accPhase ^= 1; }
        }
      }
    }
  } else if (warp >= 4) {
    const int q = warp & 3, half = (warp - 4) >> 2;  // TMEM lane quarter (fixed by warp index % 4) and column half
    constexpr int COLS = BN / 2;
    int buf = 0;
    uint32_t accPhase = 0;
    bool live = true;
    for (int t = blockIdx.x; t < nTiles; t += gridDim.x) {
      int mb, nb;
      tileCoord(p, nM, nN, t, &mb, &nb);
      const int row = mb * BM + q * 32 + lane;
      const float *saRow = p.sa + min(row, p.M - 1);
      const float *sbRow = p.sb + (size_t)nb * nK;
      float acc[COLS];
#pragma unroll
      for (int j = 0; j < COLS; j++) acc[j] = 0.f;
      // The scales of the next eight slices are always in flight (a global load takes several slice times).
      constexpr int AHEAD = 8;
      float ringA[AHEAD], ringB[AHEAD];
#pragma unroll
      for (int j = 0; j < AHEAD; j++) {
        ringA[j] = j < nK ? saRow[(size_t)j * p.M] : 0.f;
        ringB[j] = j < nK ? sbRow[j] : 0.f;
      }
      for (int kb0 = 0; kb0 < nK; kb0 += AHEAD) {
#pragma unroll
        for (int j = 0; j < AHEAD; j++) {
          const int kb = kb0 + j;
          if (kb < nK) {
            const float scale = ringA[j] * ringB[j];
            if (kb + AHEAD < nK) {
              ringA[j] = saRow[(size_t)(kb + AHEAD) * p.M];
              ringB[j] = sbRow[kb + AHEAD];
            }
            if (live) live = __all_sync(0xffffffffu, mbarWait(&tmemFull[buf], accPhase, err));
            if (live) {
              fenceAfter();
              uint32_t r0[32], r1[32];
              const uint32_t taddr = tmemBase + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * COLS);
              tmemLd32(taddr, r0);
              tmemLd32(taddr + 32, r1);
              tmemLdWait();
              fenceBefore();
              __syncwarp();
              if (lane == 0) mbarArrive(&tmemEmpty[buf]);  // the values are in registers: the accumulator may be overwritten
#pragma unroll
              for (int i = 0; i < 32; i++) acc[i] = fmaf(scale, __uint_as_float(r0[i]), acc[i]);
#pragma unroll
              for (int i = 0; i < 32; i++) acc[32 + i] = fmaf(scale, __uint_as_float(r1[i]), acc[32 + i]);
            }
            if (++buf == ACC_BUFS) { buf = 0; accPhase ^= 1; }
          }
        }
      }
      if (!live) continue;
      // one row per lane -> transposed through shared memory so that 8 lanes store one 128-byte line of a row
      const int row0 = mb * BM + q * 32;
      uint4 *stg = (uint4 *)(epiStage + (size_t)(warp - 4) * 32 * 128);
#pragma unroll
      for (int v = 0; v < 8; v++) {
        uint4 o;
        o.x = pack2(acc[8 * v + 0], acc[8 * v + 1]);
        o.y = pack2(acc[8 * v + 2], acc[8 * v + 3]);
        o.z = pack2(acc[8 * v + 4], acc[8 * v + 5]);
        o.w = pack2(acc[8 * v + 6], acc[8 * v + 7]);
        stg[lane * 8 + (v ^ (lane & 7))] = o;
      }
      __syncwarp();
      const int col = nb * BN + half * COLS + (lane & 7) * 8;
#pragma unroll
      for (int i = 0; i < 8; i++) {
        const int rr = i * 4 + (lane >> 3);
        uint4 o = stg[rr * 8 + ((lane & 7) ^ (rr & 7))];
        if (row0 + rr < p.M) {
          __nv_bfloat16 *d = p.c + (size_t)(row0 + rr) * p.ldc + col;
          if (col + 8 <= p.N) *(uint4 *)d = o;
          else {
            const __nv_bfloat16 *e = (const __nv_bfloat16 *)&o;
            for (int j = 0; j < 8 && col + j < p.N; j++) d[j] = e[j];
          }
        }
      }
      __syncwarp();
    }
  }

  fenceBefore();
  __syncthreads();
  fenceAfter();
  if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(512) : "memory");
}

// ------------------------------------------------------------------ quantisation

// One warp per (row, 128-column block): scale = amax / 448, q = x / scale.
__global__ void __launch_bounds__(256) quantActKernel(const __nv_bfloat16 *__restrict__ x, __nv_fp8_storage_t *__restrict__ q,
                                                      float *__restrict__ sa, int M, int K, int ldx) {
  const int nKb = K / 128;
  const size_t warpId = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5), total = (size_t)M * nKb;
  if (warpId >= total) return;
  const int lane = threadIdx.x & 31;
  const int row = (int)(warpId / nKb), kb = (int)(warpId % nKb);
  const uint2 raw = *(const uint2 *)(x + (size_t)row * ldx + kb * 128 + lane * 4);
  const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
  float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = amax > 0.f ? amax / 448.f : 1.f, inv = 1.f / scale;
  uint32_t out = (uint32_t)__nv_cvt_float_to_fp8(a.x * inv, __NV_SATFINITE, __NV_E4M3) |
                 (uint32_t)__nv_cvt_float_to_fp8(a.y * inv, __NV_SATFINITE, __NV_E4M3) << 8 |
                 (uint32_t)__nv_cvt_float_to_fp8(b.x * inv, __NV_SATFINITE, __NV_E4M3) << 16 |
                 (uint32_t)__nv_cvt_float_to_fp8(b.y * inv, __NV_SATFINITE, __NV_E4M3) << 24;
  *(uint32_t *)(q + (size_t)row * K + kb * 128 + lane * 4) = out;
  if (lane == 0) sa[(size_t)kb * M + row] = scale;
}

// One CTA per 128x128 block of the weight.
__global__ void __launch_bounds__(256) quantWeightKernel(const __nv_bfloat16 *__restrict__ w, __nv_fp8_storage_t *__restrict__ q,
                                                         float *__restrict__ sb, int N, int K, int ldw) {
  const int nKb = K / 128, nb = blockIdx.x / nKb, kb = blockIdx.x % nKb;
  __shared__ float red[8];
  __shared__ float scaleS;
  // thread -> (row offset, 4 columns): 32 lanes cover 128 columns, 8 warps step through the rows
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float amax = 0.f;
  for (int r = warp; r < 128; r += 8) {
    const int row = nb * 128 + r;
    if (row < N) {
      const uint2 raw = *(const uint2 *)(w + (size_t)row * ldw + kb * 128 + lane * 4);
      const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
      float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
      amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) red[warp] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < 8; i++) m = fmaxf(m, red[i]);
    scaleS = m > 0.f ? m / 448.f : 1.f;
    sb[(size_t)nb * nKb + kb] = scaleS;
  }
  __syncthreads();
  const float inv = 1.f / scaleS;
  for (int r = warp; r < 128; r += 8) {
    const int row = nb * 128 + r;
    if (row < N) {
      const uint2 raw = *(const uint2 *)(w + (size_t)row * ldw + kb * 128 + lane * 4);
      const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
      float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
      uint32_t out = (uint32_t)__nv_cvt_float_to_fp8(a.x * inv, __NV_SATFINITE, __NV_E4M3) |
                     (uint32_t)__nv_cvt_float_to_fp8(a.y * inv, __NV_SATFINITE, __NV_E4M3) << 8 |
                     (uint32_t)__nv_cvt_float_to_fp8(b.x * inv, __NV_SATFINITE, __NV_E4M3) << 16 |
                     (uint32_t)__nv_cvt_float_to_fp8(b.y * inv, __NV_SATFINITE, __NV_E4M3) << 24;
      *(uint32_t *)(q + (size_t)row * K + kb * 128 + lane * 4) = out;
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

extern "C" cudaError_t fcxGemmFp8Blockwise(const void *aq, const float *sa, const void *bq, const float *sb, void *c, int M, int N, int K,
                                           int ldc, int *errFlag, cudaStream_t s) {
  if (K % 128 || ldc % 8 || M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  if (((uintptr_t)aq | (uintptr_t)bq | (uintptr_t)c) & 15) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!makeTileMap(&ma, aq, M, K, K, BM, 1) || !makeTileMap(&mb, bq, N, K, K, BN, 1)) return cudaErrorNotSupported;
  Params p{};
  p.M = M; p.N = N; p.K = K; p.sa = sa; p.sb = sb; p.c = (__nv_bfloat16 *)c; p.ldc = ldc; p.errFlag = errFlag;
  const int nN = (N + BN - 1) / BN;
  p.group = nN >= 48 ? 16 : 8;
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(gemmFp8Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  const int tiles = ((M + BM - 1) / BM) * nN;
  gemmFp8Kernel<<<std::min(tiles, smCount()), THREADS, SMEM_BYTES, s>>>(ma, mb, p);
  return cudaGetLastError();
}

extern "C" cudaError_t fcxQuantFp8Act(const void *x, void *q, float *sa, int M, int K, int ldx, cudaStream_t s) {
  if (K % 128 || ldx % 4) return cudaErrorInvalidValue;
  const size_t warps = (size_t)M * (K / 128);
  quantActKernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>((const __nv_bfloat16 *)x, (__nv_fp8_storage_t *)q, sa, M, K, ldx);
  return cudaGetLastError();
}

extern "C" cudaError_t fcxQuantFp8Weight(const void *w, void *q, float *sb, int N, int K, int ldw, cudaStream_t s) {
  if (K % 128 || ldw % 4) return cudaErrorInvalidValue;
  quantWeightKernel<<<((N + 127) / 128) * (K / 128), 256, 0, s>>>((const __nv_bfloat16 *)w, (__nv_fp8_storage_t *)q, sb, N, K, ldw);
  return cudaGetLastError();
}
