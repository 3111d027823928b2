/*
 * flagcx_ext.h - additions of the B200-native library that have no
 * counterpart in the reference's flagcx.h.  Everything here is optional: a
 * program written against flagcx.h alone never needs it.
 */
#ifndef FLAGCX_EXT_H_
#define FLAGCX_EXT_H_

#include "flagcx.h"

#ifdef __cplusplus
extern "C" {
#endif

/* All-reduce with the output cast and a scale fused into the reduction pass:
 * recv[i] = cast_out( scale * reduce_r(send_r[i]) ).  Accumulation is fp32.
 * Supported (in -> out): fp32 -> bf16/fp16/fp8e4m3, bf16 -> fp8e4m3/fp8e5m2/fp32,
 * fp8e4m3 -> bf16, and in == out for every type. */
flagcxResult_t flagcxAllReduceCast(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t inType,
                                   flagcxDataType_t outType, float scale, flagcxRedOp_t op, flagcxComm_t comm,
                                   flagcxStream_t stream);

/* flagcxCommInitRank with options.  FLAGCX_INIT_HOST_ONLY makes a communicator
 * whose buffers are host memory (TCP host path) even on a machine with GPUs. */
#define FLAGCX_INIT_HOST_ONLY 1u
flagcxResult_t flagcxCommInitRankEx(flagcxComm_t *comm, int nranks, flagcxUniqueId_t commId, int rank, unsigned flags);

/* Split a communicator MPI-style: ranks passing the same color form a new
 * communicator, ordered by key (ties by old rank).  color < 0 yields NULL.
 * Collective over the parent. */
flagcxResult_t flagcxCommSplit(flagcxComm_t comm, int color, int key, flagcxComm_t *newcomm);

/* The same, with the size of the new communicator's symmetric heap given: bytes of one staging half (two are
 * kept) and bytes of the flagcxMemAlloc area; 0 keeps the default of a split (a quarter of FLAGCX_STAGE_BYTES /
 * FLAGCX_HEAP_USER_BYTES).  A trainer that keeps its gradients in the heap sizes its communicator with this. */
flagcxResult_t flagcxCommSplitSized(flagcxComm_t comm, int color, int key, size_t stageBytes, size_t userBytes,
                                    flagcxComm_t *newcomm);

/* Heap memory whose owner may outlive the communicator (a framework tensor built on flagcxMemAlloc memory):
 * Retain before handing the memory out, Release(ptr) instead of flagcxMemFree when the owner dies.  A
 * communicator destroyed while such memory is outstanding stops serving calls at once but keeps its heap
 * mapped until the last Release, so the memory never dangles. */
flagcxResult_t flagcxCommHeapRetain(flagcxComm_t comm);
flagcxResult_t flagcxCommHeapRelease(flagcxComm_t comm, void *ptr);

/* Per-communicator statistics. */
typedef struct {
  uint64_t calls[flagcxNumCommOps];
  uint64_t bytes[flagcxNumCommOps];
  uint64_t launches;      /* kernels launched by the library on behalf of this communicator */
  uint64_t timeouts;      /* device waits that ended by deadline */
  uint64_t kindLaunches[24];
} flagcxCommCounters;
flagcxResult_t flagcxCommGetCounters(flagcxComm_t comm, flagcxCommCounters *out);

/* Cluster view of a communicator (FLAGCX_CLUSTER_SPLIT_LIST emulates several
 * clusters on one box). */
flagcxResult_t flagcxCommGetClusterInfo(flagcxComm_t comm, int *nclusters, int *myCluster, int *clusterOfRank /* nranks ints, may be NULL */);

/* Topology queries.  NVLink links that are up on the GPU with this PCI bus id and their generation, read
 * through the management library (flagcxNotSupported when it cannot be loaded); the network port that
 * FLAGCX_TOPO_FILE attaches to a rank's GPU (empty string without one). */
flagcxResult_t flagcxTopoNvlinkCount(const char *busId, int *activeLinks, int *version);
flagcxResult_t flagcxCommGetNetOfRank(flagcxComm_t comm, int rank, char *out, size_t outBytes);

/* Symmetric heap access for fused kernels written by the user: device
 * pointers through which this rank reaches every rank's heap, the multicast
 * alias (NULL when the box has none), and translation of a pointer returned by
 * flagcxMemAlloc(comm) into its heap offset. */
flagcxResult_t flagcxCommHeapInfo(flagcxComm_t comm, void **peerBases /* nranks */, void **mcBase, size_t *heapBytes);
flagcxResult_t flagcxHeapOffset(flagcxComm_t comm, const void *ptr, size_t *offset);
/* A copy of the device-side communicator descriptor (struct FcxDevComm, see
 * flagcx_device.cuh) to pass to user kernels by value. */
flagcxResult_t flagcxCommDeviceDescriptor(flagcxComm_t comm, void *out, size_t outBytes);
/* Reserve `n` consecutive user signal slots (at most 48 per communicator). */
flagcxResult_t flagcxCommAllocSignals(flagcxComm_t comm, int n, int *first);

/* Tuner control. */
flagcxResult_t flagcxTunerRecord(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, const char *kind, int nctas, double us);
flagcxResult_t flagcxTunerSave(flagcxComm_t comm, const char *path);
flagcxResult_t flagcxTunerLoad(flagcxComm_t comm, const char *path);
/* Force the variant of subsequent calls ("ar_twoshot", 32); kind NULL clears. */
flagcxResult_t flagcxTunerPin(flagcxComm_t comm, const char *kind, int nctas);
/* For tuning tools: every kernel variant (kind, CTA count) that can legally serve a call, the cost model's
 * favourite first; the name of a kind; pin / record with an explicit pipeline sub-chunk size for the staged
 * kinds (0 = the communicator's FLAGCX_PIPE_BYTES). */
flagcxResult_t flagcxTunerCandidates(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red,
                                     int zeroCopy, int maxOut, int *kinds, int *nctas, int *count);
const char *flagcxKindName(int kind);
flagcxResult_t flagcxTunerPinEx(flagcxComm_t comm, const char *kind, int nctas, unsigned int pipeBytes);
flagcxResult_t flagcxTunerRecordEx(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, const char *kind, int nctas,
                                   unsigned int pipeBytes, double us);

/* Upper bound on the CTAs any collective of this communicator launches (0 lifts it).  For callers that run
 * collectives beside compute kernels (gradient buckets during the backward pass): a collective that takes
 * every SM stalls the kernels it was meant to overlap.  Every rank must set the same value. */
flagcxResult_t flagcxCommSetCtaBudget(flagcxComm_t comm, int maxCtas);
/* Whether the zero-copy kinds of this communicator go through the switch (multimem): 0 never, 1 from three
 * ranks on (the default; FLAGCX_ZC_MC), 2 whenever the box has a multicast alias.  With two ranks the switch
 * moves more bytes than a plain exchange, but it does the reduction, which suits a caller that runs its
 * collectives under a small CTA budget.  Every rank must set the same value. */
flagcxResult_t flagcxCommSetZeroCopyMulticast(flagcxComm_t comm, int mode);
/* Writes a NUL-terminated description of the plan that would run. */
flagcxResult_t flagcxTunerQuery(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red,
                                char *kindOut, size_t kindOutBytes, int *nctas, double *estimateUs);

/* The same for a call whose buffers are peer-visible on every rank (zeroCopy != 0: symmetric heap or registered). */
flagcxResult_t flagcxTunerQueryEx(flagcxComm_t comm, flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, flagcxRedOp_t red,
                                  int zeroCopy, char *kindOut, size_t kindOutBytes, int *nctas, double *estimateUs);

/* The plan the cost-model prior picks for a machine of `nranks` GPUs; needs neither a communicator nor a GPU. */
flagcxResult_t flagcxTunerPriorPlan(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, int nranks, int multicast, char *kindOut,
                                    size_t kindOutBytes, int *nctas, double *estimateUs);
// The same with the caller's buffers taken as peer-visible (zeroCopy != 0: the zero-copy kinds may be chosen) and
// under a CTA budget (0 = none).
flagcxResult_t flagcxTunerPriorPlanEx(flagcxCommOp_t op, size_t bytes, flagcxDataType_t dt, int nranks, int multicast, int zeroCopy,
                                      int ctaBudget, char *kindOut, size_t kindOutBytes, int *nctas, double *estimate);

/* Failure handling.  Device waits are bounded by this many milliseconds
 * (default FLAGCX_KERNEL_TIMEOUT_MS or 30000). */
flagcxResult_t flagcxCommSetTimeoutMs(flagcxComm_t comm, int ms);
/* Launch a kernel that waits for a signal nobody raises; after the time-out
 * it returns and flagcxCommGetAsyncError reports flagcxRemoteError.  Used to
 * test the bounded-wait path without disturbing the GPU. */
flagcxResult_t flagcxCommWaitTest(flagcxComm_t comm, flagcxStream_t stream);
/* Details of the last device-side give-up: code 0 none / 1 time-out / 2 abort. */
flagcxResult_t flagcxCommGetDeviceError(flagcxComm_t comm, int *code, int *peer, int *where, unsigned long long *expected,
                                        unsigned long long *seen);
/* Clear a recorded device error.  Local, not collective: enough when the wait that gave up belonged to no
 * collective (a device-API wait, flagcxCommWaitTest).  After a COLLECTIVE gave up on any rank the ranks may
 * disagree on how many collectives completed; use flagcxCommRecover then, or destroy the communicator. */
flagcxResult_t flagcxCommClearError(flagcxComm_t comm);
/* Collective over all ranks of the communicator (host side, over the bootstrap network): drain the device,
 * agree on a sequence number above anything used so far, reset flags, counters, mailboxes and point-to-point
 * state, clear the error.  Afterwards the communicator serves collectives again.  Every rank must call it,
 * with nothing of this communicator in flight. */
flagcxResult_t flagcxCommRecover(flagcxComm_t comm);

/* Single-GPU emulation of an n-rank collective (protocol tests without
 * NVLink): runs `nranks` emulated ranks inside one cooperative launch.
 * send[r]/recv[r] are device pointers on the current device. */
typedef struct flagcxEmu *flagcxEmu_t;
flagcxResult_t flagcxEmuCreate(flagcxEmu_t *emu, int nranks, size_t stageBytes);
flagcxResult_t flagcxEmuDestroy(flagcxEmu_t emu);
flagcxResult_t flagcxEmuCollective(flagcxEmu_t emu, flagcxCommOp_t op, const char *kind, int nctas, void *const *send,
                                   void *const *recv, size_t count, flagcxDataType_t dt, flagcxDataType_t outDt, float scale,
                                   flagcxRedOp_t red, int root, const size_t *a2avTables /* [nranks][4][nranks] or NULL */,
                                   void *cudaStream);
flagcxResult_t flagcxEmuSendRecv(flagcxEmu_t emu, int nops, const int *srcRank, const int *dstRank, void *const *sendbuf,
                                 void *const *recvbuf, const size_t *bytes, int ctasPerOp, void *cudaStream);
flagcxResult_t flagcxEmuGetError(flagcxEmu_t emu, int *code);

#ifdef __cplusplus
}
#endif
#endif
