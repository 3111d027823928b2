// Launchers of the fused training kernels (train_ops.cu).  All tensors are
// bf16 unless a float pointer says otherwise; sizes in elements.
#pragma once
#include <cuda_runtime_api.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
int fcxLnPartials(int M);
cudaError_t fcxLayerNormFwd(const void *x, const void *delta, const void *gamma, const void *beta, void *resOut, void *y,
                            float *mean, float *rstd, int M, int C, float eps, cudaStream_t s);
cudaError_t fcxLayerNormBwd(const void *dy, const void *x, const void *gamma, const float *mean, const float *rstd,
                            const void *dres, void *dx, void *dgamma, void *dbeta, float *partial, int M, int C, int accumulate,
                            cudaStream_t s);
cudaError_t fcxBiasGeluFwd(const void *x, const void *bias, void *y, size_t M, int C, cudaStream_t s);
cudaError_t fcxBiasGeluBwd(const void *dy, const void *x, const void *bias, void *dx, size_t M, int C, cudaStream_t s);
int fcxColSumPartials(int M);
cudaError_t fcxColSum(const void *a, void *out, float *partial, int M, int C, int accumulate, cudaStream_t s);
cudaError_t fcxCrossEntropyFwdBwd(void *logits, const int64_t *targets, float *losses, int M, int V, int Vpad, float gradScale,
                                  cudaStream_t s);
cudaError_t fcxAdamW(float *master, void *param, void *grad, float *m, float *v, size_t n, float lr, float b1, float b2, float eps,
                     float wd, int step, float gradScale, int zeroGrad, const int *stepDev, cudaStream_t s);
#ifdef __cplusplus
}
#endif
