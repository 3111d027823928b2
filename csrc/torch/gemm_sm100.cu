// bf16 GEMM family on the 5th-generation tensor cores (tcgen05 + TMEM + TMA),
// written for sm_100a, with communication fused into the same kernel:
//
//   mode PLAIN   C[M,N] = A[M,K] * B[N,K]^T
//   mode AG      all-gather -> GEMM: A is the concatenation of every rank's
//                [M/n, K] block.  Dedicated "comm" CTAs push this rank's block
//                into every peer's gathered buffer over NVLink (plain stores)
//                and raise one flag per 128-row block; the GEMM CTAs start
//                with the local block and consume remote blocks as their
//                flags arrive, so the transfer hides behind the math.
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
#include <cstdlib>
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_sm100.h"

namespace {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int EPI_BYTES = 4 * 32 * 128;  // per epilogue warp: 32 rows x 64 bf16
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int THREADS = 256;
constexpr uint32_t SPIN_LIMIT = 1u << 28;  // mbarrier polls before giving up (seconds of wall time)

__device__ __forceinline__ uint32_t smemAddr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbarInit(uint64_t *bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smemAddr(bar)), "r"(count));
}
__device__ __forceinline__ void mbarExpectTx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smemAddr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbarArrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smemAddr(bar)) : "memory");
}
// Bounded wait for the phase with the given parity.  false = gave up.
__device__ __forceinline__ bool mbarWait(uint64_t *bar, uint32_t parity, volatile int *errFlag) {
  uint32_t addr = smemAddr(bar), done = 0;
  for (uint32_t spin = 0; spin < SPIN_LIMIT; spin++) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
    if ((spin & 0xffff) == 0xffff && *errFlag) return false;
  }
  *errFlag = 1;
  return false;
}

__device__ __forceinline__ void tmaLoad2d(void *smemDst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(smemAddr(smemDst)), "l"(map), "r"(x), "r"(y), "r"(smemAddr(bar)) : "memory");
}

// Shared-memory matrix descriptor: K-major tile, 128-byte swizzle, rows 128 bytes apart,
// 8-row groups 1024 bytes apart (descriptor version 1 = Blackwell).
__device__ __forceinline__ uint64_t smemDesc(uint32_t addr) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffff) >> 4);        // start address, 16-byte units
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // version
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}

// Instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = 256.
__device__ __forceinline__ constexpr uint32_t instrDesc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void mmaF16(uint32_t dTmem, uint64_t aDesc, uint64_t bDesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(dTmem), "l"(aDesc), "l"(bDesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mmaCommit(uint64_t *bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smemAddr(bar)) : "memory");
}
__device__ __forceinline__ void tmemLd32(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tmemLdWait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void fenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *(uint32_t *)&v;
}

// Tile t of this CTA's sequence -> (row block, column block).  Row blocks are
// visited in rotated order so that (AG) the local block comes first and (RS)
// the blocks this rank owns come last.
__device__ __forceinline__ void tileCoord(const FcxGemmParams &p, int nM, int t, int *mb, int *nb) {
  const int nN = (p.N + BN - 1) / BN;
  if (p.group > 0) {
    // Row blocks in bands of `group`; inside a band the row block changes fastest, so the CTAs of one wave
    // share a few A row blocks and a few B column blocks and both stay in L2.
    const int perBand = p.group * nN, band = t / perBand, first = band * p.group;
    const int rowsHere = min(p.group, nM - first), within = t - band * perBand;
    *mb = first + within % rowsHere;
    *nb = within / rowsHere;
    return;
  }
  int g = t / nN;
  *nb = t % nN;
  *mb = (g + p.rotate) % nM;
}

template <int MODE>
__global__ void __launch_bounds__(THREADS, 1) fcxGemmKernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                                                            const FcxGemmParams p, const FcxDevComm dc) {
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
    const int work = blocksPerRank * n;  // (destination, block) pairs
    for (int w = commCta; w < work; w += nComm) {
      // destinations rotate so that the ranks do not all write to the same GPU at once;
      // the local copy (k == 0) is made first because the GEMM CTAs start on it;
      // step k goes to rank me-k, so every rank receives from itself, then rank+1, rank+2, ...
      // which is the order in which its GEMM CTAs consume the blocks
      const int k = w / blocksPerRank, b = w % blocksPerRank;
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
  uint64_t *bars = (uint64_t *)(epiStage + EPI_BYTES);
  uint64_t *fullBar = bars, *emptyBar = bars + STAGES, *tmemFull = bars + 2 * STAGES, *tmemEmpty = bars + 2 * STAGES + 2;
  uint32_t *tmemBaseSlot = (uint32_t *)(bars + 2 * STAGES + 4);

  const int Mrows = p.mPtr ? min(*p.mPtr, p.M) : p.M;  // the row count may live on the device
  const int nN = (p.N + BN - 1) / BN, nM = (Mrows + BM - 1) / BM;
  const int nTiles = nN * nM, nK = (p.K + BK - 1) / BK;
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
        tileCoord(p, nM, t, &mb, &nb);
        if (MODE == FCX_GEMM_AG) {
          // rows of block mb must have arrived in the gathered buffer
          const uint64_t *flag = (const uint64_t *)(dc.heap[dc.rank] + p.flagOff) + mb;
          ok = fcxdev::waitGe(dc, flag, p.epoch, mb / (p.rowsPerRank / BM), FCX_WAIT_DEVAPI, blockIdx.x, p.epoch);
          if (!ok) { *err = 1; break; }
          asm volatile("fence.proxy.async;" ::: "memory");  // remote generic-proxy writes -> this CTA's TMA reads
        }
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
    // ---- MMA issuer
    if (lane == 0) {
      int stage = 0, buf = 0;
      uint32_t phase = 0, accPhase = 0;
      bool ok = true;
      const uint32_t idesc = instrDesc();
      for (int t = blockIdx.x; t < nTiles && ok; t += gemmCtas) {
        if (!mbarWait(&tmemEmpty[buf], accPhase ^ 1, err)) break;
        fenceAfter();
        const uint32_t dTmem = tmemBase + (uint32_t)buf * BN;
        for (int kb = 0; kb < nK; kb++) {
          if (!mbarWait(&fullBar[stage], phase, err)) { ok = false; break; }
          fenceAfter();
          const uint32_t sa = smemAddr(tiles + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / 16; k++) {
            // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row
            mmaF16(dTmem, smemDesc(sa + k * 32), smemDesc(sb + k * 32), idesc, (kb > 0 || k > 0) ? 1u : 0u);
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
      tileCoord(p, nM, t, &mb, &nb);
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
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          uint32_t r[32];
#pragma unroll
          for (int h = 0; h < 2; h++) {
            tmemLd32(tmemBase + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + c0 + 32 * h), r);
            tmemLdWait();
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
          const int col = nb * BN + c0 + (lane & 7) * 8;
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
              if (col + 8 <= p.N) *(uint4 *)d = o;
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

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encodeFn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult st;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &p, 12000, cudaEnableDefault, &st) == cudaSuccess &&
        st == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// Row-major [rows, cols] bf16 matrix with `ld` elements between rows; box = [boxRows, 64 columns], 128-byte swizzle.
bool makeMap(CUtensorMap *m, const void *base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t boxRows) {
  EncodeTiledFn fn = encodeFn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)BK, boxRows};
  cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE>
cudaError_t launch(const CUtensorMap &a, const CUtensorMap &b, const FcxGemmParams &p, const FcxDevComm &dc, int grid, cudaStream_t s) {
  static bool attr = false;
  if (!attr) {
    cudaError_t e = cudaFuncSetAttribute(fcxGemmKernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return e;
    attr = true;
  }
  fcxGemmKernel<MODE><<<grid, THREADS, SMEM_BYTES, s>>>(a, b, p, dc);
  return cudaGetLastError();
}

// Row blocks per band of the tile order (FLAGCX_GEMM_TILE_GROUP; 0 = plain row-major order).
int tileGroup() {
  static int g = -1;
  if (g < 0) {
    const char *e = getenv("FLAGCX_GEMM_TILE_GROUP");
    g = e ? std::max(0, atoi(e)) : 8;
  }
  return g;
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
  if (!makeMap(&ma, a, M, K, lda, BM) || !makeMap(&mb, b, N, K, ldb, BN)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.errFlag = errFlag; p.rotate = 0; p.group = tileGroup();
  FcxDevComm dc{};
  int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  return launch<FCX_GEMM_PLAIN>(ma, mb, p, dc, std::min(tiles, smCount()), s);
}

extern "C" cudaError_t fcxGemmBf16DynM(const void *a, const void *b, void *c, int Mmax, const int *mPtr, int N, int K, int lda, int ldb, int ldc,
                                       int *errFlag, cudaStream_t s) {
  if (K % 8 || lda % 8 || ldb % 8 || ldc % 8 || Mmax <= 0 || N <= 0 || K <= 0) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!makeMap(&ma, a, Mmax, K, lda, BM) || !makeMap(&mb, b, N, K, ldb, BN)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = Mmax; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.errFlag = errFlag; p.mPtr = mPtr; p.group = tileGroup();
  FcxDevComm dc{};
  int tiles = ((Mmax + BM - 1) / BM) * ((N + BN - 1) / BN);
  return launch<FCX_GEMM_PLAIN>(ma, mb, p, dc, std::min(tiles, smCount()), s);
}

extern "C" cudaError_t fcxGemmRowMapBf16(const FcxDevComm *dc, const void *a, const void *b, int Mmax, const int *mPtr, int N, int K, int lda,
                                         int ldb, const void *rowInfo, size_t combineOff, size_t doneOff, int topk, int *errFlag,
                                         int *gridOut, cudaStream_t s) {
  if (K % 8 || lda % 8 || ldb % 8 || N % 8 || Mmax <= 0) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!makeMap(&ma, a, Mmax, K, lda, BM) || !makeMap(&mb, b, N, K, ldb, BN)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = Mmax; p.N = N; p.K = K; p.c = nullptr; p.ldc = N; p.errFlag = errFlag; p.mPtr = mPtr;
  p.group = tileGroup();
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
  if (!makeMap(&ma, gathered, M, K, K, BM) || !makeMap(&mb, b, N, K, ldb, BN)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.c = c; p.ldc = ldc; p.errFlag = errFlag;
  p.rowsPerRank = M / n;
  p.rotate = dc->rank * (p.rowsPerRank / BM);
  p.aLocal = aLocal; p.gatherOff = gatherOff; p.flagOff = flagOff; p.epoch = epoch;
  int tiles = (M / BM) * ((N + BN - 1) / BN);
  p.gemmCtas = std::max(1, std::min(tiles, smCount() - commCtas));
  return launch<FCX_GEMM_AG>(ma, mb, p, *dc, p.gemmCtas + commCtas, s);
}

extern "C" cudaError_t fcxGemmRsBf16(const FcxDevComm *dc, const void *a, const void *b, void *out, size_t stageOff, size_t flagOff, int M,
                                     int N, int K, int lda, int ldb, int ldc, uint64_t epoch, int *errFlag, cudaStream_t s) {
  const int n = dc->nranks;
  if (K % 8 || lda % 8 || ldb % 8 || ldc % 8 || N % 8 || M % (n * BM)) return cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  if (!makeMap(&ma, a, M, K, lda, BM) || !makeMap(&mb, b, N, K, ldb, BN)) return cudaErrorNotSupported;
  FcxGemmParams p{};
  p.M = M; p.N = N; p.K = K; p.c = out; p.ldc = ldc; p.errFlag = errFlag;
  p.rowsPerRank = M / n;
  p.rotate = ((dc->rank + 1) % n) * (p.rowsPerRank / BM);
  p.stageOff = stageOff; p.flagOff = flagOff; p.epoch = epoch;
  int tiles = (M / BM) * ((N + BN - 1) / BN);
  return launch<FCX_GEMM_RS>(ma, mb, p, *dc, std::min(tiles, smCount()), s);
}
