/*
 * flagcx.h - public C interface of the B200-native FlagCX library.
 *
 * The function names, enumerator values and struct layouts below form the
 * same binary interface that FlagCX applications are written against
 * (reference: flagcx/include/flagcx.h), so an existing program relinks
 * unchanged.  Everything behind the interface is different: collectives are
 * sm_100a kernels that read and write peer GPUs' memory over NVLink, launched
 * directly on the caller's stream.  Additions that the reference does not
 * have (fp8 data types, fused cast/scale all-reduce, tuner and counter
 * queries, the symmetric-heap helpers) live in flagcx_ext.h.
 */
#ifndef FLAGCX_H_
#define FLAGCX_H_

#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>

#ifdef __cplusplus
#define FLAGCX_DEFAULT(x) = x
extern "C" {
#else
#define FLAGCX_DEFAULT(x)
#endif

/* ---- result codes ------------------------------------------------------ */
typedef enum {
  flagcxSuccess = 0,
  flagcxUnhandledDeviceError = 1,
  flagcxSystemError = 2,
  flagcxInternalError = 3,
  flagcxInvalidArgument = 4,
  flagcxInvalidUsage = 5,
  flagcxRemoteError = 6,
  flagcxInProgress = 7,
  flagcxUnhandledCCLError = 8,
  flagcxNotSupported = 9,
  flagcxNumResults = 10
} flagcxResult_t;

/* ---- element types -----------------------------------------------------
 * Values 0..9 match the reference.  10 and 11 are new: the two 8-bit float
 * formats of Blackwell tensor cores.  Reductions on them accumulate in fp32
 * and round once on the way out. */
typedef enum {
  flagcxInt8 = 0,
  flagcxChar = 0,
  flagcxUint8 = 1,
  flagcxInt32 = 2,
  flagcxInt = 2,
  flagcxUint32 = 3,
  flagcxInt64 = 4,
  flagcxUint64 = 5,
  flagcxFloat16 = 6,
  flagcxHalf = 6,
  flagcxFloat32 = 7,
  flagcxFloat = 7,
  flagcxFloat64 = 8,
  flagcxDouble = 8,
  flagcxBfloat16 = 9,
  flagcxFloat8e4m3 = 10,
  flagcxFloat8e5m2 = 11,
  flagcxNumTypes = 12
} flagcxDataType_t;

/* Bytes per element; 0 for an unknown type. */
size_t getFlagcxDataTypeSize(flagcxDataType_t dtype);

/* ---- reduction operators ---------------------------------------------- */
typedef enum { flagcxNumRedOps_dummy = 5 } flagcxRedOp_dummy_t;
typedef enum {
  flagcxSum = 0,
  flagcxProd = 1,
  flagcxMax = 2,
  flagcxMin = 3,
  flagcxAvg = 4,
  flagcxRedNoOp = 5,
  flagcxNumRedOps = 5,
  flagcxMaxRedOp = 0x7fffffff >> (32 - 8 * sizeof(flagcxRedOp_dummy_t))
} flagcxRedOp_t;

/* ---- operation identifiers (tuner keys, plan files, logs) ------------- */
typedef enum {
  flagcxCommOpSend = 0,
  flagcxCommOpRecv = 1,
  flagcxCommOpBroadcast = 2,
  flagcxCommOpGather = 3,
  flagcxCommOpScatter = 4,
  flagcxCommOpReduce = 5,
  flagcxCommOpAllReduce = 6,
  flagcxCommOpAllGather = 7,
  flagcxCommOpReduceScatter = 8,
  flagcxCommOpAlltoAll = 9,
  flagcxCommOpAlltoAllv = 10,
  flagcxCommNoOp = 11,
  flagcxNumCommOps = 12
} flagcxCommOp_t;

typedef enum {
  flagcxMemcpyHostToDevice = 0,
  flagcxMemcpyDeviceToHost = 1,
  flagcxMemcpyDeviceToDevice = 2
} flagcxMemcpyType_t;

typedef enum {
  flagcxMemHost = 0, /* page-locked and device-mapped */
  flagcxMemDevice = 1,
  flagcxMemManaged = 2
} flagcxMemType_t;

typedef enum {
  flagcxEventDefault = 0,
  flagcxEventDisableTiming = 1
} flagcxEventType_t;

typedef enum {
  FLAGCX_VENDOR_NVIDIA = 0,
  FLAGCX_VENDOR_ILUVATAR_COREX = 1,
  FLAGCX_VENDOR_MLU = 2,
  FLAGCX_VENDOR_METAX = 3
} flagcxVendorType;

/* ---- opaque handles ---------------------------------------------------- */
#define FLAGCX_UNIQUE_ID_BYTES 256
typedef struct {
  char internal[FLAGCX_UNIQUE_ID_BYTES];
} flagcxUniqueId;
typedef flagcxUniqueId *flagcxUniqueId_t;

typedef struct flagcxComm *flagcxComm_t;
typedef struct flagcxStream *flagcxStream_t; /* wraps one cudaStream_t */
typedef struct flagcxEvent *flagcxEvent_t;   /* wraps one cudaEvent_t */
typedef struct flagcxIpcMemHandle *flagcxIpcMemHandle_t;

typedef struct {
  flagcxStream_t stream;
  flagcxEvent_t event;
  void **argList;
} flagcxFuncArgs;

/* ---- device handle: a table of runtime helpers ------------------------
 * Applications written against FlagCX never call the CUDA runtime directly;
 * they go through this table so the same source runs on other vendors.  Here
 * every slot is a thin wrapper over the CUDA runtime.  Slot order is part of
 * the binary interface. */
struct flagcxDeviceHandle {
  flagcxResult_t (*deviceSynchronize)();
  flagcxResult_t (*deviceMemcpy)(void *dst, void *src, size_t size,
                                 flagcxMemcpyType_t type,
                                 flagcxStream_t stream);
  flagcxResult_t (*deviceMemset)(void *ptr, int value, size_t size,
                                 flagcxMemType_t type, flagcxStream_t stream);
  flagcxResult_t (*deviceMalloc)(void **ptr, size_t size, flagcxMemType_t type,
                                 flagcxStream_t stream);
  flagcxResult_t (*deviceFree)(void *ptr, flagcxMemType_t type,
                               flagcxStream_t stream);
  flagcxResult_t (*setDevice)(int dev);
  flagcxResult_t (*getDevice)(int *dev);
  flagcxResult_t (*getDeviceCount)(int *count);
  flagcxResult_t (*getVendor)(char *vendor);
  flagcxResult_t (*hostGetDevicePointer)(void **pDevice, void *pHost);
  flagcxResult_t (*streamCreate)(flagcxStream_t *stream);
  flagcxResult_t (*streamDestroy)(flagcxStream_t stream);
  /* Wrap an existing cudaStream_t: pass the handle itself cast to void*
   * (reference: flagcx/adaptor/device/cuda_adaptor.cc:190-196); release the
   * wrapper with streamFree, which leaves the CUDA stream alone. */
  flagcxResult_t (*streamCopy)(flagcxStream_t *newStream, void *oldStream);
  flagcxResult_t (*streamFree)(flagcxStream_t stream);
  flagcxResult_t (*streamSynchronize)(flagcxStream_t stream);
  flagcxResult_t (*streamQuery)(flagcxStream_t stream);
  flagcxResult_t (*streamWaitEvent)(flagcxStream_t stream, flagcxEvent_t event);
  flagcxResult_t (*eventCreate)(flagcxEvent_t *event,
                                flagcxEventType_t eventType);
  flagcxResult_t (*eventDestroy)(flagcxEvent_t event);
  flagcxResult_t (*eventRecord)(flagcxEvent_t event, flagcxStream_t stream);
  flagcxResult_t (*eventSynchronize)(flagcxEvent_t event);
  flagcxResult_t (*eventQuery)(flagcxEvent_t event);
  flagcxResult_t (*ipcMemHandleCreate)(flagcxIpcMemHandle_t *handle,
                                       size_t *size);
  flagcxResult_t (*ipcMemHandleGet)(flagcxIpcMemHandle_t handle, void *devPtr);
  flagcxResult_t (*ipcMemHandleOpen)(flagcxIpcMemHandle_t handle,
                                     void **devPtr);
  flagcxResult_t (*ipcMemHandleClose)(void *devPtr);
  flagcxResult_t (*ipcMemHandleFree)(flagcxIpcMemHandle_t handle);
};
typedef struct flagcxDeviceHandle *flagcxDeviceHandle_t;

struct flagcxHandlerGroup {
  flagcxUniqueId_t uniqueId;
  flagcxComm_t comm;
  flagcxDeviceHandle_t devHandle;
};
typedef struct flagcxHandlerGroup *flagcxHandlerGroup_t;

/* Allocate / release the {uniqueId, comm, devHandle} bundle. */
flagcxResult_t flagcxHandleInit(flagcxHandlerGroup_t *handler);
flagcxResult_t flagcxHandleFree(flagcxHandlerGroup_t handler);

/* ---- memory ------------------------------------------------------------
 * flagcxMemAlloc with a communicator carves the buffer out of that
 * communicator's symmetric heap: every peer already maps it, so collectives
 * on it run zero-copy (and through the NVSwitch multicast address where the
 * box has one).  Without a communicator it is a plain device allocation.
 * flagcxCommRegister makes an arbitrary device buffer peer-visible; all
 * ranks must register their buffers in the same order (the call exchanges
 * export handles over the bootstrap network). */
flagcxResult_t flagcxMemAlloc(void **ptr, size_t size, flagcxComm_t comm FLAGCX_DEFAULT(NULL));
flagcxResult_t flagcxMemFree(void *ptr, flagcxComm_t comm FLAGCX_DEFAULT(NULL));
flagcxResult_t flagcxCommRegister(const flagcxComm_t comm, void *buff, size_t size, void **handle);
flagcxResult_t flagcxCommDeregister(const flagcxComm_t comm, void *handle);

/* ---- communicator life cycle ------------------------------------------ */
flagcxResult_t flagcxIsHomoComm(flagcxComm_t comm, int *isHomo);
flagcxResult_t flagcxGetVersion(int *version);
/* Rank 0 calls this once and ships the 256 bytes to the other ranks by any
 * out-of-band means.  *uniqueId may be NULL, in which case it is allocated. */
flagcxResult_t flagcxGetUniqueId(flagcxUniqueId_t *uniqueId);
flagcxResult_t flagcxCommInitRank(flagcxComm_t *comm, int nranks, flagcxUniqueId_t commId, int rank);
flagcxResult_t flagcxCommFinalize(flagcxComm_t comm);
flagcxResult_t flagcxCommDestroy(flagcxComm_t comm);
flagcxResult_t flagcxCommAbort(flagcxComm_t comm);
flagcxResult_t flagcxCommResume(flagcxComm_t comm);
flagcxResult_t flagcxCommSuspend(flagcxComm_t comm);
const char *flagcxGetErrorString(flagcxResult_t result);
const char *flagcxGetLastError(flagcxComm_t comm);
flagcxResult_t flagcxCommGetAsyncError(flagcxComm_t comm, flagcxResult_t *asyncError);
flagcxResult_t flagcxCommCount(const flagcxComm_t comm, int *count);
flagcxResult_t flagcxCommGetDeviceNumber(const flagcxComm_t comm, int *device);
flagcxResult_t flagcxCommUserRank(const flagcxComm_t comm, int *rank);
/* Device address of the device->host request queue used by the
 * flagcxDeviceSend/Recv/Term/Wait compatibility calls (flagcx_kernel.h). */
flagcxResult_t flagcxCommFifoBuffer(const flagcxComm_t comm, void **buffer);

/* ---- collectives --------------------------------------------------------
 * All calls enqueue work on `stream` and return; counts are in elements.
 * In-place use follows the usual rules: all-reduce/reduce/broadcast with
 * sendbuff == recvbuff; all-gather with sendbuff == recvbuff + rank*count;
 * reduce-scatter with recvbuff == sendbuff + rank*recvcount. */
flagcxResult_t flagcxBarrier(flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxReduce(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, flagcxRedOp_t op, int root,
                            flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxGather(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root, flagcxComm_t comm,
                            flagcxStream_t stream);
flagcxResult_t flagcxScatter(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root, flagcxComm_t comm,
                             flagcxStream_t stream);
flagcxResult_t flagcxBroadcast(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, int root, flagcxComm_t comm,
                               flagcxStream_t stream);
flagcxResult_t flagcxAllReduce(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, flagcxRedOp_t op,
                               flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxReduceScatter(const void *sendbuff, void *recvbuff, size_t recvcount, flagcxDataType_t datatype, flagcxRedOp_t op,
                                   flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxAllGather(const void *sendbuff, void *recvbuff, size_t sendcount, flagcxDataType_t datatype, flagcxComm_t comm,
                               flagcxStream_t stream);
flagcxResult_t flagcxAlltoAll(const void *sendbuff, void *recvbuff, size_t count, flagcxDataType_t datatype, flagcxComm_t comm,
                              flagcxStream_t stream);
/* counts and displacements are host arrays of nranks elements, in elements */
flagcxResult_t flagcxAlltoAllv(const void *sendbuff, size_t *sendcounts, size_t *sdispls, void *recvbuff, size_t *recvcounts,
                               size_t *rdispls, flagcxDataType_t datatype, flagcxComm_t comm, flagcxStream_t stream);
flagcxResult_t flagcxSend(const void *sendbuff, size_t count, flagcxDataType_t datatype, int peer, flagcxComm_t comm,
                          flagcxStream_t stream);
flagcxResult_t flagcxRecv(void *recvbuff, size_t count, flagcxDataType_t datatype, int peer, flagcxComm_t comm, flagcxStream_t stream);
/* Calls between GroupStart and GroupEnd are collected and issued as one
 * fused launch at the outermost GroupEnd. */
flagcxResult_t flagcxGroupStart(flagcxComm_t comm);
flagcxResult_t flagcxGroupEnd(flagcxComm_t comm);

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* FLAGCX_H_ */
