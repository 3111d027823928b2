// Parameters and launchers of the tcgen05 GEMM family (gemm_sm100.cu).
#pragma once
#include "../kernels/devcomm.h"
#include <cuda_runtime_api.h>
#include <stdint.h>

#define FCX_GEMM_PLAIN 0
#define FCX_GEMM_AG 1
#define FCX_GEMM_RS 2
#define FCX_GEMM_ROWMAP 3

struct FcxGemmParams {
  int M, N, K;          // C[M,N] = A[M,K] * B[N,K]^T, bf16 in, fp32 accumulate, bf16 out
  void *c;              // PLAIN/AG: C; RS: this rank's [M/n, N] result
  int ldc;
  int rotate;           // first row block (of 128 rows) this rank works on
  int bn;               // columns per tile: 256 or 128 (RS: 256)
  int group;            // PLAIN/ROWMAP: row blocks per band of the tile order (0: row-major)
  int rowsPerRank;      // M / nranks (AG, RS)
  int gemmCtas;         // AG: CTAs [0, gemmCtas) compute, the rest move data
  const void *aLocal;   // AG: this rank's [rowsPerRank, K] block
  size_t gatherOff;     // AG: heap offset of the gathered [M, K] buffer (same on every rank)
  size_t stageOff;      // RS: heap offset of the partial-tile staging [n][rowsPerRank][N]
  size_t flagOff;       // AG: heap offset of u64 flags [M/128]; RS: of u64 counters [rowsPerRank/128][ceil(N/256)]
  uint64_t epoch;       // 1-based use count of the flag/counter array that flagOff points to
  int *errFlag;         // device int, set to 1 when a bounded wait gave up
  const int *mPtr;      // optional device-resident row count (<= M); rows beyond it are neither computed nor stored
  // ROWMAP (mixture-of-experts combine): output row r goes to rank rowInfo[r].x, token rowInfo[r].y, choice rowInfo[r].z:
  // heap[rank] + combineOff + ((token * topk + choice) * N) bf16 elements; afterwards every CTA adds 1 to the u64 counter
  // at doneOff on every rank.
  const int4 *rowInfo;
  size_t combineOff, doneOff;
  int topk;
  // PLAIN only.  Operand storage: 0 = K-major (A is [M,K], B is [N,K], rows contiguous along K, the default);
  // 1 = MN-major (A is stored [K,M], B is stored [K,N]: the transposed operands of the backward GEMMs, read
  // where they lie instead of being transposed first).
  int aMN, bMN;
  const void *bias;     // optional bf16 [N], added to every row of C
  int accumulate;       // the result is added to what C holds (red.global.add) instead of replacing it
  int splitK;           // > 1: the K range is cut into that many pieces worked on by different CTAs, which add their
                        // bf16 partial results into C (zeroed by the launcher) with red.global.add
};

#ifdef __cplusplus
extern "C" {
#endif
cudaError_t fcxGemmBf16(const void *a, const void *b, void *c, int M, int N, int K, int lda, int ldb, int ldc, int *errFlag, cudaStream_t s);
cudaError_t fcxAgGemmBf16(const FcxDevComm *dc, const void *aLocal, const void *gathered, size_t gatherOff, size_t flagOff, const void *b,
                          void *c, int M, int N, int K, int ldb, int ldc, uint64_t epoch, int commCtas, int *errFlag, cudaStream_t s);
cudaError_t fcxGemmRsBf16(const FcxDevComm *dc, const void *a, const void *b, void *out, size_t stageOff, size_t flagOff, int M, int N, int K,
                          int lda, int ldb, int ldc, uint64_t epoch, int *errFlag, cudaStream_t s);
// General form: operand storage per FcxGemmParams::aMN / bMN (lda / ldb = elements between the stored rows),
// optional bias row, splitK = 0 lets the launcher pick (it splits K when the tiles would fill under half of the SMs).
cudaError_t fcxGemmBf16Ex(const void *a, const void *b, void *c, int M, int N, int K, int lda, int ldb, int ldc, int aMN, int bMN,
                          const void *bias, int splitK, int *errFlag, cudaStream_t s);
// The same with every option in a struct.  pair: -1 kernel chosen by shape (FLAGCX_GEMM_2SM: 0 never the pair kernel, 1 by
// shape, 2 whenever possible), 0 one-CTA kernel (128 x 256 tiles), 1 CTA-pair kernel (tcgen05.mma.cta_group::2, 256 x 256
// tiles; gemm2_sm100.cu).  accumulate: C += A B^T (a gradient that collects several contributions; C is not zeroed).
typedef struct FcxGemmOpts {
  int aMN, bMN;
  const void *bias;
  int splitK, accumulate, pair;
  void *geluOut;  // when set: C receives A B^T and geluOut (same shape and row stride) gelu_tanh(A B^T + bias); CTA-pair kernel only
} FcxGemmOpts;
cudaError_t fcxGemmBf16Opts(const void *a, const void *b, void *c, int M, int N, int K, int lda, int ldb, int ldc, const FcxGemmOpts *o,
                            int *errFlag, cudaStream_t s);
int fcxGemmPickSplitK(int requested, int units, int slots, int nK, int N);
int fcxGemmPairMode();
int fcxGemmPairSuits(int M, int N, int K);
cudaError_t fcxGemmPairBf16(const void *a, const void *b, void *c, int M, int N, int K, int lda, int ldb, int ldc, int aMN, int bMN,
                            const void *bias, int splitK, int accumulate, void *geluOut, int group, int *errFlag, cudaStream_t s,
                            char *detail, size_t detailLen);
const char *fcxGemmLastDetail();  // what the calling thread's last failed fcxGemmBf16Ex call tripped over
// c[Mmax,N] = a[*mPtr rows, K] @ b^T with the row count read on the device.
cudaError_t fcxGemmBf16DynM(const void *a, const void *b, void *c, int Mmax, const int *mPtr, int N, int K, int lda, int ldb, int ldc,
                            int *errFlag, cudaStream_t s);
// Expert output GEMM with the combine all-to-all fused into its epilogue (see FcxGemmParams::rowInfo).
cudaError_t fcxGemmRowMapBf16(const FcxDevComm *dc, const void *a, const void *b, int Mmax, const int *mPtr, int N, int K, int lda, int ldb,
                              const void *rowInfo, size_t combineOff, size_t doneOff, int topk, int *errFlag, int *gridOut, cudaStream_t s);
#ifdef __cplusplus
}
#endif
