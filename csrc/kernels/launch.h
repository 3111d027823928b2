// Host-callable launchers of the collective kernels (implemented in
// collectives.cu) and launch-shape constants shared with the runtime.
#pragma once
#include "devcomm.h"
#include <cuda_runtime_api.h>

#define FCX_THREADS 512

#ifdef __cplusplus
extern "C" {
#endif
cudaError_t fcxLaunchColl(const FcxDevComm *dc, const FcxCollArgs *a, int nctas, cudaStream_t s);
// zero-copy kinds (zerocopy.cu); fcxLaunchColl forwards to these
cudaError_t fcxLaunchZc(const FcxDevComm *dc, const FcxCollArgs *a, int nctas, cudaStream_t s);
cudaError_t fcxLaunchZcEmu(const FcxDevComm *dcs, const FcxCollArgs *as, const FcxCollArgs *hostArgs0, int nranks, int nctas,
                           cudaStream_t s);
cudaError_t fcxLaunchP2p(const FcxDevComm *dc, const FcxP2pArgs *g, cudaStream_t s);
cudaError_t fcxLaunchWaitTest(const FcxDevComm *dc, uint64_t want, cudaStream_t s);
// Single-GPU emulation of `nranks` ranks in one cooperative launch.  dcs, as
// and gs are device arrays with one entry per emulated rank; hostArgs0 is a
// host copy of the first entry (used to pick the template instance).
cudaError_t fcxLaunchCollEmu(const FcxDevComm *dcs, const FcxCollArgs *as, const FcxCollArgs *hostArgs0, int nranks,
                             int nctas, cudaStream_t s);
cudaError_t fcxLaunchP2pEmu(const FcxDevComm *dcs, const FcxP2pArgs *gs, int nranks, int ctasPerRank, cudaStream_t s);
#ifdef __cplusplus
}
#endif
