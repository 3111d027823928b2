// Parameters and launchers of the expert-parallel MoE kernels (moe_sm100.cu).
#pragma once
#include "../kernels/devcomm.h"
#include <cuda_runtime_api.h>
#include <stdint.h>

struct FcxMoeParams {
  const void *x;        // bf16 [T, H] tokens of this rank
  const int *topkIdx;   // int32 [T, K] expert of every choice (expert e lives on rank e / L as its local expert e % L);
                        // values outside [0, nranks * L) are skipped
  int T, H, K;
  int L;                // experts per rank (>= 1; nranks * L <= 64)
  int cap;              // rows of the expert input buffer on every rank: L segments of cap / L rows, one per local expert
  // Offsets into the symmetric heap, equal on every rank.  The caller alternates between two sets of buffers from
  // call to call (a rank may start the next dispatch while a peer still reads what the previous one left).
  size_t countMatOff;   // int32 [nranks][nranks * L]: tokens from source s for expert e
  size_t countFlagOff;  // u64 [nranks]: source s has written its row of the matrix (value = epoch)
  size_t recvOff;       // bf16 [cap][H]: expert input rows; inside a local expert's segment grouped by source rank
  size_t infoOff;       // int4 [cap]: (source rank, token, choice, 0) of every row
  size_t doneOff;       // u64 [nranks]: source s has finished pushing (value = epoch)
  uint64_t epoch;       // 1-based use count of this buffer set
  int *slot;            // local scratch int32 [T*K]
  int *localCounts;     // local scratch int32 [nranks * L]
  int *recvTotal;       // out, device int32 [L]: rows received by each of this rank's experts
  int *errFlag;         // device int32: 1 = a bounded wait gave up, 2 = an expert's buffer overflowed (extra tokens dropped)
};

#ifdef __cplusplus
extern "C" {
#endif
cudaError_t fcxMoeDispatch(const FcxDevComm *dc, const FcxMoeParams *p, int ctas, cudaStream_t s);
// h[r, :F] = silu(gu[r, :F]) * gu[r, F:2F] for the first min(*rows, maxRows) rows (rows may be null)
cudaError_t fcxSiluMul(const void *gu, void *h, const int *rows, int maxRows, int F, cudaStream_t s);
// out[t] = sum_k w[t,k] * ret[t,k,:] once the u64 counter at doneOff on this rank has reached `want`
cudaError_t fcxMoeCombine(const FcxDevComm *dc, const void *ret, const float *w, void *out, int T, int H, int K, size_t doneOff,
                          uint64_t want, int *errFlag, cudaStream_t s);
#ifdef __cplusplus
}
#endif
