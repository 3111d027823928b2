// bf16 GEMM family on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// written for sm_100a, with communication fused into the same kernel:
//
//   mode PLAIN   C[M,N] = A[M,K] * B[N,K]^T
//   mode AG      all-gather -> GEMM: A is the concatenation of every rank's
//                [M/n, K] block.  Dedicated "comm" CTAs push this rank's block
//                into every peer's gathered buffer over NVLink (plain stores)
//                and raise one flag per 128-row block; the GEMM CTAs start
//                with the local block, read in place through its own tensor
//                map, and consume remote blocks as their flags arrive, so
//                the transfer hides behind the math.
//   mode RS      GEMM -> reduce-scatter: every finished 128x256 tile is
//                written straight from TMEM (through registers) into the
//                staging area of the rank that owns those rows, tiles owned by
//                other ranks first, then an arrival counter is raised; after
//                its last tile each CTA turns to the reduction of the tiles
//                this rank owns (sum of the n partial tiles, fp32) as their
//                counters fill.
//
// The reference has no GEMM and no fused path: its users run a vendor
// all-gather / reduce-scatter and a vendor GEMM back to back.
//
// Structure (one CTA per SM, 256 threads, persistent over tiles):
//   warp 0    TMA producer: cp.async.bulk.tensor loads of A (128x64) and B
//             (256x64) tiles, 128-byte swizzle, 4-stage mbarrier pipeline.
//             All loads read this GPU's own memory and none is multicast.
//   warp 1    MMA issuer: one elected lane issues tcgen05.mma (M128 N256 K16,
//             bf16 x bf16 -> fp32) into one of two TMEM accumulators,
//             tcgen05.commit releases smem stages / publishes the accumulator.
//   warp 2    allocates and frees the 512 TMEM columns.
//   warps 4-7 epilogue: tcgen05.ld (32 lanes x 32 columns per warp and step),
//             fp32 -> bf16, transposed through shared memory so that global
//             stores (possibly into a peer) cover whole 128-byte lines.
// Every wait (mbarrier, flag, counter) is bounded: after the limit the kernel
// records an error, drains, frees its TMEM and returns.
#include "../kernels/prims.cuh"

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

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BYTES = 4 * 32 * 128;  // per epilogue warp: 32 rows x 64 bf16
constexpr int BIAS_BYTES = 4 * 256 * 4;  // per epilogue warp: the tile's bias values as fp32
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + BIAS_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int THREADS = 256;

// Instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = 256.
__device__ __forceinline__ uint32_t instrDesc(int bn, int aMN = 0, int bMN = 0) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(aMN ? 1 : 0) << 15) | ((uint32_t)(bMN ? 1 : 0) << 16) |
         ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}
constexpr int MN_BLOCK_BYTES = 64 * BK * 2;  // one 64-column block of an MN-major tile: BK lines of 128 bytes

// Tile t of this CTA's sequence -> (row block, column block).  Row blocks are
// visited in rotated order so that (AG) the local block comes first and (RS)
// the blocks this rank owns come last.
__device__ __forceinline__ void tileCoord(const FcxGemmParams &p, int nM, int t, int *mb, int *nb) {
  const int nN = (p.N + p.bn - 1) / p.bn;
  int g;
  if (p.group > 0) {
    // Row blocks in bands of `group`; inside a band the row block changes fastest, so the CTAs of one wave
    // share a few A row blocks and a few B column blocks and both stay in L2.
    const int perBand = p.group * nN, band = t / perBand, first = band * p.group;
    const int rowsHere = min(p.group, nM - first), within = t - band * perBand;
    g = first + within % rowsHere;
    *nb = within / rowsHere;
  } else {
    g = t / nN;
    *nb = t % nN;
  }
  *mb = (g + p.rotate) % nM;  // AG: the local rows first; RS: the rows this rank owns last
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1) fcxGemmKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                            const __grid_constant__ CUtensorMap tmALocal, const FcxGemmParams p,
                                                            const FcxDevComm dc) {
  extern __shared__ uint8_t smemRaw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int *err = p.errFlag;

  // ------------------------------------------------------------ communication CTAs (AG mode only)
  if (MODE == FCX_GEMM_AG && (int)blockIdx.x >= p.gemmCtas) {
    // This rank's [rowsPerRank, K] block goes, 128 rows at a time, to every rank's gathered buffer
    // (this rank's own copy included); one flag per destination and 128-row block.
    const int commCta = blockIdx.x - p.gemmCtas, nComm = gridDim.x - p.gemmCtas;
    const int n = dc.nranks, me = dc.rank;
    const int blocksPerRank = p.rowsPerRank / BM;
    const size_t blockBytes = (size_t)BM * p.K * 2;
    const int work = blocksPerRank * (n - 1);  // (remote destination, block) pairs; the local block is read where it lies
    for (int w = commCta; w < work; w += nComm) {
      // destinations rotate so that the ranks do not all write to the same GPU at once:
      // step k goes to rank me-k, so every rank receives from rank+1, rank+2, ... which is the
      // order in which its GEMM CTAs consume the remote blocks
      const int k = 1 + w / blocksPerRank, b = w % blocksPerRank;
      const int dst = (me - k + n) % n;
      const char *src = (const char *)p.aLocal + (size_t)b * blockBytes;
      char *d = dc.heap[dst] + p.gatherOff + ((size_t)me * blocksPerRank + b) * blockBytes;
      const uint4 *s4 = (const uint4 *)src;
      uint4 *d4 = (uint4 *)d;
      const size_t nvec = blockBytes / 16;
      size_t i = threadIdx.x;
      for (; i + 3 * THREADS < nvec; i += 4 * THREADS) {
        uint4 a = s4[i], bb = s4[i + THREADS], c = s4[i + 2 * THREADS], e = s4[i + 3 * THREADS];
        d4[i] = a; d4[i + THREADS] = bb; d4[i + 2 * THREADS] = c; d4[i + 3 * THREADS] = e;
      }
      for (; i < nvec; i += THREADS) d4[i] = s4[i];
      __syncthreads();
      if (threadIdx.x == 0) {
        uint64_t *flag = (uint64_t *)(dc.heap[dst] + p.flagOff) + (size_t)me * blocksPerRank + b;
        fcxdev::stRelease(flag, p.epoch);
      }
    }
    return;
  }

  // ------------------------------------------------------------ GEMM CTAs
  uint8_t *tiles = (uint8_t *)(((uintptr_t)smemRaw + 1023) & ~(uintptr_t)1023);
  uint8_t *epiStage = tiles + STAGES * STAGE_BYTES;
  float *biasStage = (float *)(epiStage + EPI_BYTES);
  uint64_t *bars = (uint64_t *)(epiStage + EPI_BYTES + BIAS_BYTES);
  uint64_t *fullBar = bars, *emptyBar = bars + STAGES, *tmemFull = bars + 2 * STAGES, *tmemEmpty = bars + 2 * STAGES + 2;
  uint32_t *tmemBaseSlot = (uint32_t *)(bars + 2 * STAGES + 4);

  const int Mrows = p.mPtr ? min(*p.mPtr, p.M) : p.M;  // the row count may live on the device
  const int bn = p.bn;  // columns per tile: 256, or 128 when that fills the SMs better
  const int nN = (p.N + bn - 1) / bn, nM = (Mrows + BM - 1) / BM;
  const int nK = (p.K + BK - 1) / BK;
  const int splitK = (MODE == FCX_GEMM_PLAIN && p.splitK > 1) ? p.splitK : 1;
  const int kPer = (nK + splitK - 1) / splitK;  // K blocks per split
  const int nTiles = nN * nM * splitK;
  const int gemmCtas = (MODE == FCX_GEMM_AG) ? p.gemmCtas : gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; s++) { mbarInit(&fullBar[s], 1); mbarInit(&emptyBar[s], 1); }
    for (int b = 0; b < 2; b++) { mbarInit(&tmemFull[b], 1); mbarInit(&tmemEmpty[b], 4); }
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
    // ---- TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < nTiles && ok; t += gemmCtas) {
        int mb, nb;
        tileCoord(p, nM, t / splitK, &mb, &nb);
        const int kLo = (t % splitK) * kPer, kHi = min(nK, kLo + kPer);
        const CUtensorMap *mapA = &tmA;
        int rowA = mb * BM;
        if (MODE == FCX_GEMM_AG) {
          const int blocksPerRank = p.rowsPerRank / BM, owner = mb / blocksPerRank;
          if (owner == dc.rank) {
            // this rank's own rows are read straight from the caller's tensor
            mapA = &tmALocal;
            rowA = (mb - owner * blocksPerRank) * BM;
          } else {
            // rows of block mb must have arrived in the gathered buffer
            const uint64_t *flag = (const uint64_t *)(dc.heap[dc.rank] + p.flagOff) + mb;
            ok = fcxdev::waitGe(dc, flag, p.epoch, owner, FCX_WAIT_DEVAPI, blockIdx.x, p.epoch);
            if (!ok) { *err = 1; break; }
            asm volatile("fence.proxy.async;" ::: "memory");  // remote generic-proxy writes -> this CTA's TMA reads
          }
        }
        for (int kb = kLo; kb < kHi; kb++) {
          if (!mbarWait(&emptyBar[stage], phase ^ 1, err)) { ok = false; break; }
          mbarExpectTx(&fullBar[stage], A_BYTES + bn * BK * 2);
          uint8_t *sa = tiles + stage * STAGE_BYTES, *sb = sa + A_BYTES;
          if (MODE == FCX_GEMM_PLAIN && p.aMN) {
            // stored [K, M]: two blocks of 64 columns (M) x BK lines (K)
            for (int j = 0; j < BM / 64; j++) tmaLoad2d(sa + j * MN_BLOCK_BYTES, mapA, rowA + j * 64, kb * BK, &fullBar[stage]);
          } else {
            tmaLoad2d(sa, mapA, kb * BK, rowA, &fullBar[stage]);
          }
          if (MODE == FCX_GEMM_PLAIN && p.bMN) {
            for (int j = 0; j < bn / 64; j++) tmaLoad2d(sb + j * MN_BLOCK_BYTES, &tmB, nb * bn + j * 64, kb * BK, &fullBar[stage]);
          } else {
            tmaLoad2d(sb, &tmB, kb * BK, nb * bn, &fullBar[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer
    if (lane == 0) {
      int stage = 0, buf = 0;
      uint32_t phase = 0, accPhase = 0;
      bool ok = true;
      const bool aMN = MODE == FCX_GEMM_PLAIN && p.aMN, bMN = MODE == FCX_GEMM_PLAIN && p.bMN;
      const uint32_t idesc = instrDesc(bn, aMN, bMN);
      for (int t = blockIdx.x; t < nTiles && ok; t += gemmCtas) {
        if (!mbarWait(&tmemEmpty[buf], accPhase ^ 1, err)) break;
        fenceAfter();
        const uint32_t dTmem = tmemBase + (uint32_t)buf * bn;
        const int kLo = (t % splitK) * kPer, kHi = min(nK, kLo + kPer);
        for (int kb = kLo; kb < kHi; kb++) {
          if (!mbarWait(&fullBar[stage], phase, err)) { ok = false; break; }
          fenceAfter();
          const uint32_t sa = smemAddr(tiles + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            // K-major: 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row;
            // MN-major: 16 K indices = two eight-line groups = 2048 bytes further
            const uint64_t da = aMN ? smemDescMN(sa + k * 2048, MN_BLOCK_BYTES) : smemDesc(sa + k * 32);
            const uint64_t db = bMN ? smemDescMN(sb + k * 2048, MN_BLOCK_BYTES) : smemDesc(sb + k * 32);
            mmaF16(dTmem, da, db, idesc, (kb > kLo || k > 0) ? 1u : 0u);
          }
          mmaCommit(&emptyBar[stage]);  // the stage may be refilled once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        mmaCommit(&tmemFull[buf]);  // accumulator complete
        if (++buf == 2) { buf = 0; accPhase ^= 1; }
      }
    }
  } else if (warp >= 4) {
    // ---- epilogue: warp w owns TMEM lanes [32*(w%4), +32) = rows of the tile.
    // A wait that gives up turns the warp "dead": it keeps walking the tile list (so that the
    // barriers it shares with the other epilogue warps stay matched) but touches nothing.
    const int q = warp & 3;
    int buf = 0;
    uint32_t accPhase = 0;
    bool live = true;
    for (int t = blockIdx.x; t < nTiles; t += gemmCtas) {
      int mb, nb;
      tileCoord(p, nM, t / splitK, &mb, &nb);
      const bool firstSplit = (t % splitK) == 0;
      if (live) live = __all_sync(0xffffffffu, mbarWait(&tmemFull[buf], accPhase, err));
      if (live) {
        fenceAfter();
        // first row of this warp's 32-row band and where it goes
        const int row0 = mb * BM + q * 32;
        __nv_bfloat16 *dst0;
        size_t ldd;
        if (MODE == FCX_GEMM_RS) {
          const int owner = min(row0 / p.rowsPerRank, dc.nranks - 1), lrow0 = row0 - owner * p.rowsPerRank;
          dst0 = (__nv_bfloat16 *)(dc.heap[owner] + p.stageOff) + ((size_t)dc.rank * p.rowsPerRank + lrow0) * p.N;
          ldd = p.N;
        } else {
          dst0 = (__nv_bfloat16 *)p.c + (size_t)row0 * p.ldc;
          ldd = p.ldc;
        }
        // The accumulator comes out of TMEM one row per lane; a transposition through
        // shared memory (32 rows x 128 bytes per warp, 16-byte chunks XOR-swizzled by row)
        // turns that into stores where 8 lanes write one full 128-byte line of a row.
        uint4 *stg = (uint4 *)(epiStage + (size_t)q * 32 * 128);
        // the tile's bias values, once per tile and warp, as fp32 in shared memory (columns past N read as 0)
        const bool addBias = MODE == FCX_GEMM_PLAIN && p.bias != nullptr && firstSplit;
        float *biasW = biasStage + q * 256;
        if (addBias) {
          const __nv_bfloat16 *bias = (const __nv_bfloat16 *)p.bias;
#pragma unroll
          for (int j = 0; j < 8; j++) {
            const int cidx = nb * bn + j * 32 + lane;
            biasW[j * 32 + lane] = (j * 32 < bn && cidx < p.N) ? __bfloat162float(bias[cidx]) : 0.f;
          }
          __syncwarp();
        }
#pragma unroll 1
        for (int c0 = 0; c0 < bn; c0 += 64) {
          uint32_t r[32];
#pragma unroll
          for (int h = 0; h < 2; h++) {
            tmemLd32(tmemBase + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * bn + c0 + 32 * h), r);
            tmemLdWait();
            if (addBias) {
              // every lane holds one row and the same 32 columns: broadcast reads of the staged bias values
              const float4 *bv = (const float4 *)(biasW + c0 + 32 * h);
#pragma unroll
              for (int j = 0; j < 8; j++) {
                const float4 f = bv[j];
                r[4 * j + 0] = __float_as_uint(__uint_as_float(r[4 * j + 0]) + f.x);
                r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + f.y);
                r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + f.z);
                r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + f.w);
              }
            }
#pragma unroll
            for (int v = 0; v < 4; v++) {
              uint4 o;
              o.x = pack2(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              o.y = pack2(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              o.z = pack2(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              o.w = pack2(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              stg[lane * 8 + ((4 * h + v) ^ (lane & 7))] = o;
            }
          }
          __syncwarp();
          const int col = nb * bn + c0 + (lane & 7) * 8;
#pragma unroll
          for (int i = 0; i < 8; i++) {
            const int rr = i * 4 + (lane >> 3);
            uint4 o = stg[rr * 8 + ((lane & 7) ^ (rr & 7))];
            if (row0 + rr < Mrows) {
              __nv_bfloat16 *d = dst0 + (size_t)rr * ldd + col;
              if (MODE == FCX_GEMM_ROWMAP) {
                const int4 info = p.rowInfo[row0 + rr];
                d = (__nv_bfloat16 *)(dc.heap[info.x] + p.combineOff) + ((size_t)info.y * p.topk + info.z) * p.N + col;
              }
              if (MODE == FCX_GEMM_PLAIN && (splitK > 1 || p.accumulate)) {
                // one K piece of several, or a contribution to a gradient that is being accumulated: added into C
                const uint32_t *w = (const uint32_t *)&o;
                for (int j = 0; j < 4; j++)
                  if (col + 2 * j + 1 < p.N || (col + 2 * j < p.N && (p.N & 1) == 0))
                    asm volatile("red.global.add.noftz.bf16x2 [%0], %1;" ::"l"(d + 2 * j), "r"(w[j]) : "memory");
              } else if (col + 8 <= p.N) *(uint4 *)d = o;
              else {
                const __nv_bfloat16 *e = (const __nv_bfloat16 *)&o;
                for (int j = 0; j < 8 && col + j < p.N; j++) d[j] = e[j];
              }
            }
          }
          __syncwarp();
        }
        fenceBefore();
        __syncwarp();
        if (lane == 0) mbarArrive(&tmemEmpty[buf]);
      }
      if (MODE == FCX_GEMM_RS) {
        // publish the tile to its owner: every epilogue warp fences its stores, then one thread counts the tile
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (live && warp == 4 && lane == 0) {
          const int owner = (mb * BM) / p.rowsPerRank, lmb = (mb * BM % p.rowsPerRank) / BM;
          uint64_t *cnt = (uint64_t *)(dc.heap[owner] + p.flagOff) + (size_t)lmb * nN + nb;
          asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(cnt), "l"((uint64_t)1) : "memory");
        }
      }
      if (++buf == 2) { buf = 0; accPhase ^= 1; }
    }
  }

  // ------------------------------------------------------------ tear-down
  fenceBefore();
  __syncthreads();
  fenceAfter();
  if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmemBase), "r"(512) : "memory");

  if (MODE == FCX_GEMM_ROWMAP) {
    // every row this CTA produced has been stored (possibly on peers): tell every rank that this CTA is done
    __threadfence_system();
    __syncthreads();
    if ((int)threadIdx.x < dc.nranks) {
      uint64_t *cnt = (uint64_t *)(dc.heap[threadIdx.x] + p.doneOff);
      asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(cnt), "l"((uint64_t)1) : "memory");
    }
  }

  // ------------------------------------------------------------ RS: reduce the tiles this rank owns
  if (MODE == FCX_GEMM_RS) {
    const int n = dc.nranks, lBlocks = p.rowsPerRank / BM;
    const int items = lBlocks * nN;
    const uint64_t want = p.epoch * (uint64_t)n;
    for (int it = blockIdx.x; it < items; it += gridDim.x) {
      const int lmb = it / nN, nb = it % nN;
      bool ok = true;
      if (threadIdx.x == 0) {
        const uint64_t *cnt = (const uint64_t *)(dc.heap[dc.rank] + p.flagOff) + (size_t)lmb * nN + nb;
        ok = fcxdev::waitGe(dc, cnt, want, -1, FCX_WAIT_DEVAPI, blockIdx.x, p.epoch);
        if (!ok) *err = 1;
      }
      if (!__syncthreads_and(ok)) break;
      // 128 x 256 outputs, 8 per thread step: thread handles 16-byte vectors
      const int colsHere = min(BN, p.N - nb * BN);
      const int vecPerRow = colsHere / 8;
      const __nv_bfloat16 *stage = (const __nv_bfloat16 *)(dc.heap[dc.rank] + p.stageOff);
      for (int v = threadIdx.x; v < BM * vecPerRow; v += THREADS) {
        const int r = v / vecPerRow, cv = v % vecPerRow;
        const int lrow = lmb * BM + r;
        if (lrow >= p.rowsPerRank) break;
        const size_t off = (size_t)lrow * p.N + nb * BN + cv * 8;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int s = 0; s < n; s++) {
          uint4 x = *(const uint4 *)(stage + (size_t)s * p.rowsPerRank * p.N + off);
          const __nv_bfloat162 *h = (const __nv_bfloat162 *)&x;
#pragma unroll
          for (int j = 0; j < 4; j++) {
            float2 f = __bfloat1622float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
        uint4 o;
        o.x = pack2(acc[0], acc[1]); o.y = pack2(acc[2], acc[3]); o.z = pack2(acc[4], acc[5]); o.w = pack2(acc[6], acc[7]);
        *(uint4 *)((__nv_bfloat16 *)p.c + (size_t)lrow * p.ldc + nb * BN + cv * 8) = o;
      }
    }
  }
}

// ------------------------------------------------------------------ host side

// Row-major [rows, cols] bf16 matrix with `ld` elements between rows; box = [boxRows, 64 columns], 128-byte swizzle.
bool makeMap(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t boxRows) {
  return makeTileMap(m, base, rows, cols, ld, boxRows, 2);
}

template <int MODE>
cudaError_t launch(const CUtensorMap &a, const CUtensorMap &b, const FcxGemmParams &p, const FcxDevComm &dc, int grid, cudaStream_t s,
                   const CUtensorMap *aLocal = nullptr) {
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fcxGemmKernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  fcxGemmKernel<MODE><<<grid, THREADS, SMEM_BYTES, s>>>(a, b, aLocal ? *aLocal : a, p, dc);
  return cudaGetLastError();
}

// Row blocks per band of the tile order (FLAGCX_GEMM_TILE_GROUP; 0 = plain row-major order).
int tileGroup(int nN) {
  static int g = -2;
  if (g == -2) {
    const char *e = getenv("FLAGCX_GEMM_TILE_GROUP");
    g = e ? std::max(0, atoi(e)) : -1;
  }
  return g >= 0 ? g : (nN >= 24 ? 16 : 8);  // wide outputs: taller bands keep more of B in L2 per wave
}

// Columns per tile.  128-column tiles cost almost as much as 256-column ones (the A tile is re-read for half the
// math, and shared-memory bandwidth is what bounds the MMA), so they do not pay even when they fill the last
// wave better; FLAGCX_GEMM_BN=128 selects them for experiments.
int pickBn(int, int, int) {
  static int bn = 0;
  if (!bn) {
    const char *e = getenv("FLAGCX_GEMM_BN");
    bn = e && atoi(e) == 128 ? 128 : 256;
  }
  return bn;
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

extern "C" cudaError_t fcxGemmBf16(const void *a, const void *b, void *c, int M, int N, int K, int lda, int ldb, int ldc, int *errFlag,
                                   cudaStream_t s) {
  if (K % 8 || lda % 8 || ldb % 8 || ldc % 8 || M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  const int bn = pickBn(M, N, smCount());
  if (!makeMap(&ma, a, M, K, lda, BM) || !makeMap(&mb, b, N, K, ldb, bn)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.errFlag = errFlag; p.rotate = 0; p.bn = bn; p.group = tileGroup((N + bn - 1) / bn);
  FcxDevComm dc{};
  int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn);
  return launch<FCX_GEMM_PLAIN>(ma, mb, p, dc, std::min(tiles, smCount()), s);
}

// Pieces to cut K into.  requested > 0: that many (at most one per K block, and no piece may be empty).  Otherwise: few
// tiles and a long K (the weight-gradient GEMMs: K = tokens) are cut so that the pieces fill whole waves; a split into
// s pieces takes ceil(units * s / slots) waves of 1/s the length, and every extra piece costs some reduction traffic,
// counted as 3 % of a tile (1 % when K is very long).
extern "C" int fcxGemmPickSplitK(int requested, int units, int slots, int nK, int N) {
  int splitK = requested;
  if (splitK <= 0) {
    splitK = 1;
    const bool few = units < slots && nK >= 32;
    // more tiles than slots but a poor last wave and a very long K (the LM head's input gradient: 128 tiles on 74
    // pairs, K = 50304): zeroing C is noise against such a K, and the pieces stay long
    const bool longK = units >= slots && nK >= 256;
    if (few || longK) {
      const double base = (double)((units + slots - 1) / slots), piece = few ? 0.03 : 0.01;
      double best = 1.0;
      for (int sk = 2; sk <= 8 && nK / sk >= 8; sk++) {
        const double waves = (double)((units * sk + slots - 1) / slots);
        const double cost = waves / (sk * base) + piece * (sk - 1);
        if (cost < best - (splitK == 1 ? 0.05 : 0.0)) { best = cost; splitK = sk; }  // a first cut must pay clearly
      }
    }
  }
  if (N % 2) return 1;  // the partial results are added two columns at a time
  splitK = std::max(1, std::min(splitK, nK));
  const int kPer = (nK + splitK - 1) / splitK;
  return (nK + kPer - 1) / kPer;
}

// What went wrong in the last fcxGemmBf16Ex call of this thread that did not return cudaSuccess.
static thread_local char gGemmDetail[256];
extern "C" const char *fcxGemmLastDetail() { return gGemmDetail; }

extern "C" cudaError_t fcxGemmBf16Opts(const void *a, const void *b, void *c, int M, int N, int K, int lda, int ldb, int ldc,
                                       const FcxGemmOpts *o, int *errFlag, cudaStream_t s) {
  const int aMN = o->aMN, bMN = o->bMN, accumulate = o->accumulate;
  const void *bias = o->bias;
  int splitK = o->splitK;
  if (K % 8 || lda % 8 || ldb % 8 || ldc % 8 || M <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  if (((uintptr_t)a | (uintptr_t)b | (uintptr_t)c) & 15) return cudaErrorInvalidValue;
  if ((aMN && M % 8) || (bMN && N % 8) || (bias && ((uintptr_t)bias & 1)) || (accumulate && N % 2)) return cudaErrorInvalidValue;
  gGemmDetail[0] = 0;
  cudaGetLastError();  // an error left behind by an earlier, unrelated call of this thread is not this launch's
  if (o->geluOut || (o->pair >= 0 ? o->pair > 0 : fcxGemmPairSuits(M, N, K) != 0))  // CTA pairs on 256 x 256 tiles (gemm2_sm100.cu)
    return fcxGemmPairBf16(a, b, c, M, N, K, lda, ldb, ldc, aMN, bMN, bias, splitK, accumulate, o->geluOut, tileGroup((N + 255) / 256) / 2,
                           errFlag, s, gGemmDetail, sizeof gGemmDetail);
  CUtensorMap ma, mb;
  const int bn = pickBn(M, N, smCount());
  // K-major operand: rows = M (or N), box of 128 (bn) rows x 64 K; MN-major operand: rows = K, box of 64 lines x 64 columns
  const bool okA = aMN ? makeMap(&ma, a, K, M, lda, BK) : makeMap(&ma, a, M, K, lda, BM);
  const bool okB = bMN ? makeMap(&mb, b, K, N, ldb, BK) : makeMap(&mb, b, N, K, ldb, bn);
  if (!okA || !okB) {
    snprintf(gGemmDetail, sizeof gGemmDetail, "tensor map of operand %s refused (M %d N %d K %d lda %d ldb %d aMN %d bMN %d a %p b %p)",
             !okA ? "A" : "B", M, N, K, lda, ldb, aMN, bMN, a, b);
    return cudaErrorNotSupported;
  }
  FcxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.errFlag = errFlag; p.rotate = 0; p.bn = bn; p.group = tileGroup((N + bn - 1) / bn);
  p.aMN = aMN; p.bMN = bMN; p.bias = bias; p.accumulate = accumulate;
  const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn), nK = (K + BK - 1) / BK;
  p.splitK = fcxGemmPickSplitK(splitK, tiles, smCount(), nK, N);
  if (p.splitK > 1 && !accumulate) {
    cudaError_t e = cudaMemsetAsync(c, 0, ((size_t)(M - 1) * ldc + N) * 2, s);
    if (e != cudaSuccess) return e;
  }
  FcxDevComm dc{};
  cudaError_t e = launch<FCX_GEMM_PLAIN>(ma, mb, p, dc, std::min(tiles * p.splitK, smCount()), s);
  if (e != cudaSuccess)
    snprintf(gGemmDetail, sizeof gGemmDetail, "kernel launch: %s (M %d N %d K %d aMN %d bMN %d splitK %d grid %d)", cudaGetErrorString(e), M, N,
             K, aMN, bMN, p.splitK, std::min(tiles * p.splitK, smCount()));
  return e;
}

extern "C" cudaError_t fcxGemmBf16Ex(const void *a, const void *b, void *c, int M, int N, int K, int lda, int ldb, int ldc, int aMN, int bMN,
                                     const void *bias, int splitK, int *errFlag, cudaStream_t s) {
  FcxGemmOpts o{};
  o.aMN = aMN; o.bMN = bMN; o.bias = bias; o.splitK = splitK; o.accumulate = 0; o.pair = -1;
  return fcxGemmBf16Opts(a, b, c, M, N, K, lda, ldb, ldc, &o, errFlag, s);
}

extern "C" cudaError_t fcxGemmBf16DynM(const void *a, const void *b, void *c, int Mmax, const int *mPtr, int N, int K, int lda, int ldb, int ldc,
                                       int *errFlag, cudaStream_t s) {
  if (K % 8 || lda % 8 || ldb % 8 || ldc % 8 || Mmax <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  const int bn = pickBn(Mmax, N, smCount());
  if (!makeMap(&ma, a, Mmax, K, lda, BM) || !makeMap(&mb, b, N, K, ldb, bn)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = Mmax; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.errFlag = errFlag; p.mPtr = mPtr; p.bn = bn; p.group = tileGroup((N + bn - 1) / bn);
  FcxDevComm dc{};
  int tiles = ((Mmax + BM - 1) / BM) * ((N + bn - 1) / bn);
  return launch<FCX_GEMM_PLAIN>(ma, mb, p, dc, std::min(tiles, smCount()), s);
}

extern "C" cudaError_t fcxGemmRowMapBf16(const FcxDevComm *dc, const void *a, const void *b, int Mmax, const int *mPtr, int N, int K, int lda,
                                         int ldb, const void *rowInfo, size_t combineOff, size_t doneOff, int topk, int *errFlag,
                                         int *gridOut, cudaStream_t s) {
  if (K % 8 || lda % 8 || ldb % 8 || N % 8 || Mmax <= 0) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  const int bn = pickBn(Mmax, N, smCount());
  if (!makeMap(&ma, a, Mmax, K, lda, BM) || !makeMap(&mb, b, N, K, ldb, bn)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = Mmax; p.N = N; p.K = K; p.c = nullptr; p.ldc = N; p.errFlag = errFlag; p.mPtr = mPtr;
  p.bn = bn; p.group = tileGroup((N + bn - 1) / bn);
  p.rowInfo = (const int4 *)rowInfo; p.combineOff = combineOff; p.doneOff = doneOff; p.topk = topk;
  // a fixed grid: the receivers count one arrival per CTA of every rank
  int grid = smCount();
  if (gridOut) *gridOut = grid;
  return launch<FCX_GEMM_ROWMAP>(ma, mb, p, *dc, grid, s);
}

extern "C" cudaError_t fcxAgGemmBf16(const FcxDevComm *dc, const void *aLocal, const void *gathered, size_t gatherOff, size_t flagOff,
                                     const void *b, void *c, int M, int N, int K, int ldb, int ldc, uint64_t epoch, int commCtas,
                                     int *errFlag, cudaStream_t s) {
  const int n = dc->nranks;
  if (K % 8 || ldb % 8 || ldc % 8 || M % (n * BM) || commCtas < 1) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  const int bn = pickBn(M, N, std::max(1, smCount() - commCtas));
  CUtensorMap mal;
  if (!makeMap(&ma, gathered, M, K, K, BM) || !makeMap(&mb, b, N, K, ldb, bn) || !makeMap(&mal, aLocal, M / n, K, K, BM))
    return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.errFlag = errFlag; p.bn = bn; p.group = tileGroup((N + bn - 1) / bn);
  p.rowsPerRank = M / n;
  p.rotate = dc->rank * (p.rowsPerRank / BM);
  p.group = std::max(1, std::min(p.group, p.rowsPerRank / BM));  // a band never mixes rows of two ranks: they arrive at different times
  p.aLocal = aLocal; p.gatherOff = gatherOff; p.flagOff = flagOff; p.epoch = epoch;
  int tiles = (M / BM) * ((N + bn - 1) / bn);
  p.gemmCtas = std::max(1, std::min(tiles, smCount() - commCtas));
  return launch<FCX_GEMM_AG>(ma, mb, p, *dc, p.gemmCtas + commCtas, s, &mal);
}

extern "C" cudaError_t fcxGemmRsBf16(const FcxDevComm *dc, const void *a, const void *b, void *out, size_t stageOff, size_t flagOff, int M,
                                     int N, int K, int lda, int ldb, int ldc, uint64_t epoch, int *errFlag, cudaStream_t s) {
  const int n = dc->nranks;
  if (K % 8 || lda % 8 || ldb % 8 || ldc % 8 || N % 8 || M % (n * BM)) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!makeMap(&ma, a, M, K, lda, BM) || !makeMap(&mb, b, N, K, ldb, BN)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.c = out; p.ldc = ldc; p.errFlag = errFlag; p.bn = BN;  // counters are laid out per 256 columns
  p.group = tileGroup((N + BN - 1) / BN);
  p.rowsPerRank = M / n;
  p.rotate = ((dc->rank + 1) % n) * (p.rowsPerRank / BM);
  p.stageOff = stageOff; p.flagOff = flagOff; p.epoch = epoch;
  int tiles = (M / BM) * ((N + BN - 1) / BN);
  return launch<FCX_GEMM_RS>(ma, mb, p, *dc, std::min(tiles, smCount()), s);
}
