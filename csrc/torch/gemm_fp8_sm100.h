// Launchers of the block-scaled fp8 GEMM and its quantisation kernels (gemm_fp8_sm100.cu).
#pragma once
#include <cuda_runtime_api.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
// c[M,N] (bf16) = (aq[M,K] e4m3, scales sa[K/128][M]) x (bq[N,K] e4m3, scales sb[ceil(N/128)][K/128])^T; K % 128 == 0.
cudaError_t fcxGemmFp8Blockwise(const void *aq, const float *sa, const void *bq, const float *sb, void *c, int M, int N, int K, int ldc,
                                int *errFlag, cudaStream_t s);
// bf16 x[M,K] -> e4m3 q[M,K] (contiguous) with one scale per row and 128 columns, stored as sa[K/128][M]
cudaError_t fcxQuantFp8Act(const void *x, void *q, float *sa, int M, int K, int ldx, cudaStream_t s);
// bf16 w[N,K] -> e4m3 q[N,K] (contiguous) with one scale per 128x128 block, stored as sb[ceil(N/128)][K/128]
cudaError_t fcxQuantFp8Weight(const void *w, void *q, float *sb, int N, int K, int ldw, cudaStream_t s);
#ifdef __cplusplus
}
#endif
