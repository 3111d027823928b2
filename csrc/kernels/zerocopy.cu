// Entry points and launchers of the zero-copy collective kernels (bodies in zerocopy.cuh).
#include "zerocopy.cuh"
#include "launch.h"
#include "dispatch.h"

#include <cuda_runtime.h>

namespace fcxdev {

template <typename TIn, typename TOut>
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxZcReduceKernel(FcxDevComm dc, FcxCollArgs a) {
  fcxZcReduceBody<TIn, TOut>(dc, a, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxZcMoveKernel(FcxDevComm dc, FcxCollArgs a) {
  fcxZcMoveBody(dc, a, blockIdx.x, gridDim.x);
}
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxZcReduceEmuKernel(const FcxDevComm *dcs, const FcxCollArgs *as, int ctasPerRank) {
  int r = blockIdx.x / ctasPerRank;
  fcxZcReduceBody<TIn, TOut>(dcs[r], as[r], blockIdx.x % ctasPerRank, ctasPerRank);
}
__global__ void __launch_bounds__(FCX_THREADS, 1) fcxZcMoveEmuKernel(const FcxDevComm *dcs, const FcxCollArgs *as, int ctasPerRank) {
  int r = blockIdx.x / ctasPerRank;
  fcxZcMoveBody(dcs[r], as[r], blockIdx.x % ctasPerRank, ctasPerRank);
}

}  // namespace fcxdev

using namespace fcxdev;

namespace {

template <typename TIn, typename TOut>
cudaError_t launchZc(const FcxDevComm &dc, const FcxCollArgs &a, int nctas, cudaStream_t s) {
  fcxZcReduceKernel<TIn, TOut><<<nctas, FCX_THREADS, 0, s>>>(dc, a);
  return cudaGetLastError();
}
template <typename TIn, typename TOut>
cudaError_t launchZcEmu(const FcxDevComm *dcs, const FcxCollArgs *as, int nranks, int nctas, cudaStream_t s) {
  void *params[] = {(void *)&dcs, (void *)&as, (void *)&nctas};
  return cudaLaunchCooperativeKernel((const void *)fcxZcReduceEmuKernel<TIn, TOut>, dim3(nranks * nctas), dim3(FCX_THREADS),
                                     params, 0, s);
}

}  // namespace

extern "C" cudaError_t fcxLaunchZc(const FcxDevComm *dc, const FcxCollArgs *a, int nctas, cudaStream_t s) {
  if (a->kind == FCX_K_MOVE_ZC) {
    fcxZcMoveKernel<<<nctas, FCX_THREADS, 0, s>>>(*dc, *a);
    return cudaGetLastError();
  }
#define CALL(TI, TO) launchZc<TI, TO>(*dc, *a, nctas, s)
  FCX_DISPATCH_ALL(a, CALL);
#undef CALL
}

extern "C" cudaError_t fcxLaunchZcEmu(const FcxDevComm *dcs, const FcxCollArgs *as, const FcxCollArgs *a, int nranks, int nctas,
                                      cudaStream_t s) {
  if (a->kind == FCX_K_MOVE_ZC) {
    void *params[] = {(void *)&dcs, (void *)&as, (void *)&nctas};
    return cudaLaunchCooperativeKernel((const void *)fcxZcMoveEmuKernel, dim3(nranks * nctas), dim3(FCX_THREADS), params, 0, s);
  }
#define CALL(TI, TO) launchZcEmu<TI, TO>(dcs, as, nranks, nctas, s)
  FCX_DISPATCH_ALL(a, CALL);
#undef CALL
}
