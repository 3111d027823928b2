// fcxColSumNoAlloc - column sums of a bf16 matrix without any allocation.
//
// This entry point has no counterpart in the reference library.
//
// Who needs it: programs that may not (or cannot) ask the CUDA allocator for
// memory at the moment they need a bias gradient.  Examples are a serving
// process that handed the whole device to its own memory pool at start-up (a
// later cudaMalloc simply fails), a control loop that cannot afford the
// device-wide synchronisation hidden in cudaMalloc/cudaFree, and callers
// outside PyTorch that have no caching allocator to lean on.  The regular
// entry point, fcxColSum (train_ops.h), wants a scratch buffer from its
// caller; this one brings its own.
//
// How: the per-row-slice partial sums go to a fixed array that is part of the
// library image (`static __device__`, 1 MiB).  Every GPU that loads the
// library holds that megabyte until the process exits.
//
// Contract
//   * a: [M, C] bf16 row-major, out: [C] bf16, both device memory supplied by
//     the caller, both 16-byte aligned (the kernels use 16-byte accesses; a
//     pointer that is not is refused with FCX_NOALLOC_MISALIGNED); C must be a
//     multiple of 64.
//   * Limit: fcxColSumPartials(M) * C <= FCX_NOALLOC_MAX_FLOATS (262144), which
//     always holds for C <= 8192; larger shapes are refused with
//     FCX_NOALLOC_TOO_LARGE and nothing is launched.
//   * The first call on a device looks up the device address of the array
//     (cudaGetSymbolAddress, with that device current) and remembers it.  Make
//     that first call during set-up, before any stream capture begins.
//   * All calls on one device share the one array.  Its contents after a call
//     are the last call's partial sums; nothing in it has to start at zero
//     (each call overwrites every element it later reads).  Two calls that can
//     run at the same time on the GPU (different streams) race on it: keep
//     calls stream-ordered.
//   * No cudaMalloc, cudaFree or other allocating routine is called.
//
// Returns 0 on success, one of the negative codes below, or a positive
// cudaError_t from the runtime.  fcxNoAllocErrorString() explains any of them.
#pragma once
#include <cuda_runtime_api.h>

#define FCX_NOALLOC_MAX_FLOATS (256 * 1024)
#define FCX_NOALLOC_TOO_LARGE (-1)
#define FCX_NOALLOC_BAD_SHAPE (-2)
#define FCX_NOALLOC_NULL_POINTER (-3)
#define FCX_NOALLOC_MISALIGNED (-4)

#ifdef __cplusplus
extern "C" {
#endif
int fcxColSumNoAlloc(const void *a, void *out, int M, int C, int accumulate, cudaStream_t stream);
const char *fcxNoAllocErrorString(int code);
#ifdef __cplusplus
}
#endif
