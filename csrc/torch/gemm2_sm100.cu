// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2 (M 256, N 256, K 16 per instruction).
//
//   C[M,N] = A[M,K] * B[N,K]^T (+ bias), operands K-major or MN-major as in the one-CTA kernel.
//
// Two CTAs of a cluster, resident on the two SMs of one pair, work on one 256 x 256 output tile.  Each CTA
// loads ITS 128 rows of A and ITS 128 of the 256 columns of B into its own shared memory (plain TMA loads, never
// multicast); the instruction, issued by one thread of the pair's leader CTA, reads the A half of each CTA for that
// CTA's 128 accumulator rows and the two B halves for the 256 columns, and writes each CTA's accumulator into that
// CTA's own TMEM.  Against the one-CTA kernel (128 x 256 tile, 48 KB per K block of 64 through one SM's shared
// memory) a CTA now feeds 32 KB per K block for the same math, which lifts the shared-memory bound on the MMA rate
// and halves the L2 reads of B; the smaller stage also buys a 5-deep pipeline.
//
// Roles per CTA (384 threads): warp 0 TMA producer, warp 1 MMA issuer (leader CTA only), warp 2 TMEM allocation,
// warps 4-11 epilogue (TMEM -> registers -> bf16 blocks in shared memory -> TMA store, or TMA add for split K and
// accumulated gradients).
// Barriers: the leader's full[stage] collects the bytes of both CTAs' loads; tcgen05.commit arrives on empty[stage]
// and accFull[buf] of BOTH CTAs (barrier multicast inside the cluster; that is a signal, not a load); the epilogue
// warps of both CTAs arrive on the leader's accEmpty[buf].  Every wait is bounded: after the limit the kernel
// records an error, leaves its loops, meets its peer at the closing cluster barrier, frees its TMEM and returns.
//
// The reference has no GEMM; this kernel serves the model's projections (forward, input gradient, weight gradient).
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_sm100.h"
#include "tcgen05.cuh"

namespace {

using namespace fcxmma;

constexpr int BM = 128;    // accumulator rows per CTA (256 per pair)
constexpr int BN = 256;    // columns per tile
constexpr int BNH = 128;   // B columns that one CTA holds
#ifndef FCX_PAIR_STAGES
#define FCX_PAIR_STAGES 5
#endif
constexpr int BK = 64, STAGES = FCX_PAIR_STAGES;
constexpr int STG_DEPTH = STAGES >= 6 ? 1 : 2;  // staging blocks per epilogue warp: the sixth stage takes the room of the second block
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BNH * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STG_BYTES = 32 * 64;                 // staging block: 32 rows x 32 bf16 columns
constexpr int EPI_BYTES = 8 * STG_DEPTH * STG_BYTES;  // 8 epilogue warps
constexpr int BIAS_BYTES = 8 * 128 * 4;  // per epilogue warp: its 128 bias values as fp32
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BIAS_BYTES + 1024 + 256;
constexpr int THREADS = 384;
constexpr int MN_BLOCK_BYTES = 64 * BK * 2;

__device__ __forceinline__ uint32_t ctaRankInCluster() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t mapToCta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void clusterSync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// TMA tile load into this CTA's shared memory whose bytes are counted on a barrier of the pair's leader CTA.
__device__ __forceinline__ void tmaLoad2dPair(void *smemDst, const CUtensorMap *map, int x, int y, uint32_t barClusterAddr) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smemAddr(smemDst)), "l"(map), "r"(x), "r"(y), "r"(barClusterAddr) : "memory");
}
__device__ __forceinline__ void mmaF16Pair(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrive on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done.
__device__ __forceinline__ void mmaCommitPair(uint64_t *bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smemAddr(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void mbarArriveRemote(uint32_t barClusterAddr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(barClusterAddr) : "memory");
}

// D fp32, A/B bf16, M = 256 over the pair, N = 256.
__device__ __forceinline__ uint32_t instrDescPair(int aMN, int bMN) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(aMN ? 1 : 0) << 15) | ((uint32_t)(bMN ? 1 : 0) << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
}

// Tile t -> (256-row block, 256-column block); bands of `group` row blocks as in the one-CTA kernel.
__device__ __forceinline__ void tileCoord2(int group, int nM, int nN, int t, int *mb, int *nb) {
  if (group > 0) {
    const int perBand = group * nN, band = t / perBand, first = band * group;
    const int rowsHere = min(group, nM - first), within = t - band * perBand;
    *mb = first + within % rowsHere;
    *nb = within / rowsHere;
  } else {
    *mb = t / nN;
    *nb = t % nN;
  }
}

// tanh-form GELU, the same arithmetic as the stand-alone bias+GELU kernel of the training ops
__device__ __forceinline__ float geluTanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(k0 * (x + k1 * x * x * x)));
  return 0.5f * x * (1.f + t);
}

// GELU = true: two outputs per tile: C = A B^T (kept for the backward pass) and C2 = gelu(A B^T + bias).
template <bool GELU>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
    fcxGemmPairKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const __grid_constant__ CUtensorMap tmC,
                      const __grid_constant__ CUtensorMap tmC2, const FcxGemmParams p) {
  extern __shared__ uint8_t smemRaw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *err = p.errFlag;
  const uint32_t cr = ctaRankInCluster();  // 0 = leader
  const int pair = blockIdx.x >> 1, nPairs = gridDim.x >> 1;

  uint8_t *tiles = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  uint8_t *epiStage = tiles + STAGES * STAGE_BYTES;
  float *biasStage = (float *)(epiStage + EPI_BYTES);
  uint64_t *bars = (uint64_t *)(epiStage + EPI_BYTES + BIAS_BYTES);
  uint64_t *fullBar = bars, *emptyBar = bars + STAGES, *accFull = bars + 2 * STAGES, *accEmpty = bars + 2 * STAGES + 2;
  uint32_t *tmemBaseSlot = (uint32_t *)(bars + 2 * STAGES + 4);

  const int nN = (p.N + BN - 1) / BN, nM = (p.M + 2 * BM - 1) / (2 * BM);
  const int nK = (p.K + BK - 1) / BK;
  const int splitK = p.splitK > 1 ? p.splitK : 1;
  const int kPer = (nK + splitK - 1) / splitK;
  const int nTiles = nN * nM * splitK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbarInit(&fullBar[s], 1); mbarInit(&emptyBar[s], 1); }
    for (int b = 0; b < 2; b++) { mbarInit(&accFull[b], 1); mbarInit(&accEmpty[b], 16); }  // 8 epilogue warps in each CTA
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smemAddr(tmemBaseSlot)), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  fenceBefore();
  __syncthreads();
  clusterSync();  // the peer's barriers exist before anything arrives on them
  fenceAfter();
  const uint32_t tmemBase = *tmemBaseSlot;

  if (warp == 0) {
    // ---- TMA producer (both CTAs): own half of A and of B; bytes counted on the leader's barrier
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < nTiles && ok; t += nPairs) {
        int mb, nb;
        tileCoord2(p.group, nM, nN, t / splitK, &mb, &nb);
        const int kLo = (t % splitK) * kPer, kHi = min(nK, kLo + kPer);
        const int rowA = mb * 2 * BM + (int)cr * BM, colB = nb * BN + (int)cr * BNH;
        for (int kb = kLo; kb < kHi; kb++) {
          if (!mbarWait(&emptyBar[stage], phase ^ 1, err)) { ok = false; break; }
          if (cr == 0) mbarExpectTx(&fullBar[stage], 2 * STAGE_BYTES);
          const uint32_t bar = mapToCta(smemAddr(&fullBar[stage]), 0);
          uint8_t *sa = tiles + stage * STAGE_BYTES, *sb = sa + A_BYTES;
          if (p.aMN) {
            for (int j = 0; j < BM / 64; j++) tmaLoad2dPair(sa + j * MN_BLOCK_BYTES, &tmA, rowA + j * 64, kb * BK, bar);
          } else {
            tmaLoad2dPair(sa, &tmA, kb * BK, rowA, bar);
          }
          if (p.bMN) {
            for (int j = 0; j < BNH / 64; j++) tmaLoad2dPair(sb + j * MN_BLOCK_BYTES, &tmB, colB + j * 64, kb * BK, bar);
          } else {
            tmaLoad2dPair(sb, &tmB, kb * BK, colB, bar);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one thread of the leader CTA drives the tensor cores of both SMs
    if (lane == 0 && cr == 0) {
      int stage = 0, buf = 0;
      uint32_t phase = 0, accPhase = 0;
      bool ok = true;
      const uint32_t idesc = instrDescPair(p.aMN, p.bMN);
      for (int t = pair; t < nTiles && ok; t += nPairs) {
        if (!mbarWait(&accEmpty[buf], accPhase ^ 1, err)) break;
        fenceAfter();
        const uint32_t dTmem = tmemBase + (uint32_t)buf * BN;
        const int kLo = (t % splitK) * kPer, kHi = min(nK, kLo + kPer);
        for (int kb = kLo; kb < kHi; kb++) {
          if (!mbarWait(&fullBar[stage], phase, err)) { ok = false; break; }
          fenceAfter();
          const uint32_t sa = smemAddr(tiles + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            const uint64_t da = p.aMN ? smemDescMN(sa + k * 2048, MN_BLOCK_BYTES) : smemDesc(sa + k * 32);
            const uint64_t db = p.bMN ? smemDescMN(sb + k * 2048, MN_BLOCK_BYTES) : smemDesc(sb + k * 32);
            mmaF16Pair(dTmem, da, db, idesc, (kb > kLo || k > 0) ? 1u : 0u);
          }
          mmaCommitPair(&emptyBar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mmaCommitPair(&accFull[buf]);
        if (++buf == 2) { buf = 0; accPhase ^= 1; }
      }
    }
  } else if (warp >= 4) {
    // ---- epilogue (both CTAs, 8 warps): warp w owns TMEM lanes [32*(w%4), +32) = 32 of this CTA's 128 rows, and the
    // left (warps 4-7) or right (warps 8-11) 128 of the tile's 256 columns.  32 columns at a time: tcgen05.ld (one row
    // per lane), bias, fp32 -> bf16, 16-byte stores into a staging block laid out as the TMA's 64-byte swizzle wants it
    // (conflict-free), then ONE thread hands the 32 x 32 block to the TMA unit, as a store or, for a piece of a split K
    // or an accumulated gradient, as a reduction (add) into C.  The TMA clips what lies beyond M and N.  Two staging
    // blocks per warp: the next block is filled while the unit still reads the previous one.
    const int ew = warp - 4, q = ew & 3, half = ew >> 2;
    int buf = 0;
    uint32_t accPhase = 0, chunkNo = 0;
    bool live = true;
    uint8_t *stgBase = epiStage + (size_t)ew * STG_DEPTH * STG_BYTES;
    float *biasW = biasStage + ew * 128;
    const bool reduce = splitK > 1 || p.accumulate;
    for (int t = pair; t < nTiles; t += nPairs) {
      int mb, nb;
      tileCoord2(p.group, nM, nN, t / splitK, &mb, &nb);
      const bool firstSplit = (t % splitK) == 0;
      if (live) live = __all_sync(0xffffffffu, mbarWait(&accFull[buf], accPhase, err));
      if (live) {
        fenceAfter();
        const int row0 = mb * 2 * BM + (int)cr * BM + q * 32, colBase = nb * BN + half * 128;
        const bool addBias = p.bias != nullptr && firstSplit;
        if (addBias) {  // this warp's 128 bias values, once per tile, as fp32 in shared memory (columns past N read as 0)
          const __nv_bfloat16 *bias = (const __nv_bfloat16 *)p.bias;
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int cidx = colBase + j * 32 + lane;
            biasW[j * 32 + lane] = cidx < p.N ? __bfloat162float(bias[cidx]) : 0.f;
          }
          __syncwarp();
        }
#pragma unroll 1
        for (int c0 = 0; c0 < 128; c0 += 32) {
          if (colBase + c0 >= p.N || row0 >= p.M) break;
          uint32_t r[32];
          tmemLd32(tmemBase + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * 128 + c0), r);
          if (GELU) {
            // both staging blocks of this warp are used per step: the product goes into the first, the activation
            // into the second, and one thread hands both to the TMA unit
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
            tmemLdWait();
            uint4 *stgPre = (uint4 *)stgBase, *stgAct = (uint4 *)(stgBase + STG_BYTES);
#pragma unroll
            for (int v = 0; v < 4; v++) {
              uint4 o;
              o.x = pack2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              stgPre[lane * 4 + (v ^ ((lane >> 1) & 3))] = o;
            }
            const float4 *bv = (const float4 *)(biasW + c0);
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const float4 f = addBias ? bv[j] : make_float4(0.f, 0.f, 0.f, 0.f);
              r[4 * j + 0] = __float_as_uint(geluTanh(__uint_as_float(r[4 * j + 0]) + f.x));
              r[4 * j + 1] = __float_as_uint(geluTanh(__uint_as_float(r[4 * j + 1]) + f.y));
              r[4 * j + 2] = __float_as_uint(geluTanh(__uint_as_float(r[4 * j + 2]) + f.z));
              r[4 * j + 3] = __float_as_uint(geluTanh(__uint_as_float(r[4 * j + 3]) + f.w));
            }
#pragma unroll
            for (int v = 0; v < 4; v++) {
              uint4 o;
              o.x = pack2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              stgAct[lane * 4 + (v ^ ((lane >> 1) & 3))] = o;
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&tmC), "r"(colBase + c0), "r"(row0), "r"(smemAddr(stgPre)) : "memory");
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&tmC2), "r"(colBase + c0), "r"(row0), "r"(smemAddr(stgAct)) : "memory");
              asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            chunkNo++;
            continue;
          }
          // the staging block about to be refilled must have been read out by the TMA unit
          if (lane == 0) {
            if (STG_DEPTH == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          __syncwarp();
          tmemLdWait();
          if (addBias) {
            const float4 *bv = (const float4 *)(biasW + c0);  // same address in every lane: broadcast reads
#pragma unroll
            for (int j = 0; j < 8; j++) {
              const float4 f = bv[j];
              r[4 * j + 0] = __float_as_uint(__uint_as_float(r[4 * j + 0]) + f.x);
              r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + f.y);
              r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + f.z);
              r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + f.w);
            }
          }
          uint4 *stg = (uint4 *)(stgBase + (chunkNo % STG_DEPTH) * STG_BYTES);
#pragma unroll
          for (int v = 0; v < 4; v++) {
            uint4 o;
            o.x = pack2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
            o.y = pack2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
            o.z = pack2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
            o.w = pack2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
            stg[lane * 4 + (v ^ ((lane >> 1) & 3))] = o;  // row = lane (64 bytes), 16-byte chunk XOR bits 1-2 of the row
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> the TMA unit's reads
          __syncwarp();
          if (lane == 0) {
            if (reduce)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&tmC), "r"(colBase + c0), "r"(row0), "r"(smemAddr(stg)) : "memory");
            else
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&tmC), "r"(colBase + c0), "r"(row0), "r"(smemAddr(stg)) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          chunkNo++;
        }
        fenceBefore();
        __syncwarp();
        if (lane == 0) mbarArriveRemote(mapToCta(smemAddr(&accEmpty[buf]), 0));
      }
      if (++buf == 2) { buf = 0; accPhase ^= 1; }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every block has reached C
  }

  // ---- tear-down: nobody leaves, and no TMEM is freed, while the peer may still read this CTA's shared memory,
  // write its TMEM or arrive on its barriers
  fenceBefore();
  __syncthreads();
  clusterSync();
  fenceAfter();
  if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(512) : "memory");
}

int smCount2() {
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

// 0 = never, 1 = when the shape suits (default), 2 = whenever the kernel can take the shape.
extern "C" int fcxGemmPairMode() {
  static int mode = -1;
  if (mode < 0) {
    const char *e = getenv("FLAGCX_GEMM_2SM");
    mode = e ? std::max(0, std::min(2, atoi(e))) : 1;
  }
  return mode;
}

// Whether the pair kernel is the better choice for this shape: whole 256-row blocks (or so many rows that the
// half-empty last block does not matter) and at least most of one 256-column block.
extern "C" int fcxGemmPairSuits(int M, int N, int K) {
  const int mode = fcxGemmPairMode();
  if (mode == 0 || M < 129 || K < 8) return 0;
  if (mode == 2) return 1;
  const int padded = (M + 255) / 256 * 256;
  return (double)padded <= 1.07 * M && N >= 192;
}

extern "C" cudaError_t fcxGemmPairBf16(const void *a, const void *b, void *c, int M, int N, int K, int lda, int ldb, int ldc, int aMN, int bMN,
                                       const void *bias, int splitK, int accumulate, void *geluOut, int group, int *errFlag, cudaStream_t s,
                                       char *detail, size_t detailLen) {
  CUtensorMap ma, mb;
  const bool okA = aMN ? makeTileMap(&ma, a, K, M, lda, BK, 2) : makeTileMap(&ma, a, M, K, lda, BM, 2);
  const bool okB = bMN ? makeTileMap(&mb, b, K, N, ldb, BK, 2) : makeTileMap(&mb, b, N, K, ldb, BNH, 2);
  CUtensorMap mc, mc2;
  bool okC = makeStoreMap(&mc, c, M, N, ldc);
  if (geluOut) {
    if (accumulate || ((uintptr_t)geluOut & 15)) return cudaErrorInvalidValue;
    okC = okC && makeStoreMap(&mc2, geluOut, M, N, ldc);
    splitK = 1;  // the activation needs the whole sum
  } else {
    mc2 = mc;
  }
  if (!okA || !okB || !okC) {
    if (detail)
      snprintf(detail, detailLen, "tensor map of %s refused (pair kernel, M %d N %d K %d)", !okA ? "operand A" : !okB ? "operand B" : "C", M, N, K);
    return cudaErrorNotSupported;
  }
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fcxGemmPairKernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(fcxGemmPairKernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  FcxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.errFlag = errFlag; p.bn = BN; p.group = group;
  p.aMN = aMN; p.bMN = bMN; p.bias = bias;
  const int units = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN), nK = (K + BK - 1) / BK, pairs = smCount2() / 2;
  p.splitK = fcxGemmPickSplitK(splitK, units, pairs, nK, N);
  p.accumulate = accumulate;
  if (p.splitK > 1 && !accumulate) {
    cudaError_t e = cudaMemsetAsync(c, 0, ((size_t)(M - 1) * ldc + N) * 2, s);
    if (e != cudaSuccess) return e;
  }
  const int grid = 2 * std::min(units * p.splitK, pairs);
  if (geluOut) fcxGemmPairKernel<true><<<grid, THREADS, SMEM_BYTES, s>>>(ma, mb, mc, mc2, p);
  else fcxGemmPairKernel<false><<<grid, THREADS, SMEM_BYTES, s>>>(ma, mb, mc, mc2, p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess && detail)
    snprintf(detail, detailLen, "pair kernel launch: %s (M %d N %d K %d splitK %d grid %d)", cudaGetErrorString(e), M, N, K, p.splitK, grid);
  return e;
}
