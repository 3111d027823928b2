"""ctypes binding of the C API (``libflagcx.so``).

Serving stacks that cannot take a dependency on ``torch.distributed`` drive
the library through a thin ctypes layer; the reference ships one as
``plugin/interservice/flagcx_wrapper.py:190-424``.  ``FLAGCXLibrary`` keeps
that surface (same method names) and adds the remaining collectives, the
memory API and the extensions of ``flagcx_ext.h``.

Buffers are passed as raw addresses (``tensor.data_ptr()`` or a numpy
``ctypes.data``); streams as ``flagcxStream_t`` obtained from
``adaptor_stream_copy(torch_stream)`` or ``adaptor_stream_create()``.
With a communicator created on a machine without a GPU the buffers are host
memory and the stream argument is ignored.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path
from typing import Optional, Sequence

flagcxResult_t = ctypes.c_int
flagcxDataType_t = ctypes.c_int
flagcxRedOp_t = ctypes.c_int
flagcxComm_t = ctypes.c_void_p
flagcxStream_t = ctypes.c_void_p
flagcxEvent_t = ctypes.c_void_p
buffer_type = ctypes.c_void_p


class flagcxUniqueId(ctypes.Structure):
    _fields_ = [("internal", ctypes.c_byte * 256)]


flagcxUniqueId_t = ctypes.POINTER(flagcxUniqueId)

_F = ctypes.CFUNCTYPE
_R = flagcxResult_t
_vp = ctypes.c_void_p


class flagcxDeviceHandle(ctypes.Structure):
    _fields_ = [
        ("deviceSynchronize", _F(_R)),
        ("deviceMemcpy", _F(_R, _vp, _vp, ctypes.c_size_t, ctypes.c_int, flagcxStream_t)),
        ("deviceMemset", _F(_R, _vp, ctypes.c_int, ctypes.c_size_t, ctypes.c_int, flagcxStream_t)),
        ("deviceMalloc", _F(_R, ctypes.POINTER(_vp), ctypes.c_size_t, ctypes.c_int, flagcxStream_t)),
        ("deviceFree", _F(_R, _vp, ctypes.c_int, flagcxStream_t)),
        ("setDevice", _F(_R, ctypes.c_int)),
        ("getDevice", _F(_R, ctypes.POINTER(ctypes.c_int))),
        ("getDeviceCount", _F(_R, ctypes.POINTER(ctypes.c_int))),
        ("getVendor", _F(_R, ctypes.c_char_p)),
        ("hostGetDevicePointer", _F(_R, ctypes.POINTER(_vp), _vp)),
        ("streamCreate", _F(_R, ctypes.POINTER(flagcxStream_t))),
        ("streamDestroy", _F(_R, flagcxStream_t)),
        ("streamCopy", _F(_R, ctypes.POINTER(flagcxStream_t), _vp)),
        ("streamFree", _F(_R, flagcxStream_t)),
        ("streamSynchronize", _F(_R, flagcxStream_t)),
        ("streamQuery", _F(_R, flagcxStream_t)),
        ("streamWaitEvent", _F(_R, flagcxStream_t, flagcxEvent_t)),
        ("eventCreate", _F(_R, ctypes.POINTER(flagcxEvent_t), ctypes.c_int)),
        ("eventDestroy", _F(_R, flagcxEvent_t)),
        ("eventRecord", _F(_R, flagcxEvent_t, flagcxStream_t)),
        ("eventSynchronize", _F(_R, flagcxEvent_t)),
        ("eventQuery", _F(_R, flagcxEvent_t)),
        ("ipcMemHandleCreate", _F(_R, ctypes.POINTER(_vp), ctypes.POINTER(ctypes.c_size_t))),
        ("ipcMemHandleGet", _F(_R, _vp, _vp)),
        ("ipcMemHandleOpen", _F(_R, _vp, ctypes.POINTER(_vp))),
        ("ipcMemHandleClose", _F(_R, _vp)),
        ("ipcMemHandleFree", _F(_R, _vp)),
    ]


flagcxDeviceHandle_t = ctypes.POINTER(flagcxDeviceHandle)


class flagcxHandlerGroup(ctypes.Structure):
    _fields_ = [("uniqueId", flagcxUniqueId_t), ("comm", flagcxComm_t), ("devHandle", flagcxDeviceHandle_t)]


flagcxHandlerGroup_t = ctypes.POINTER(flagcxHandlerGroup)


class flagcxCommCounters(ctypes.Structure):
    _fields_ = [("calls", ctypes.c_uint64 * 12), ("bytes", ctypes.c_uint64 * 12), ("launches", ctypes.c_uint64),
                ("timeouts", ctypes.c_uint64), ("kindLaunches", ctypes.c_uint64 * 24)]


class flagcxDataTypeEnum:
    flagcxInt8 = 0
    flagcxChar = 0
    flagcxUint8 = 1
    flagcxInt32 = 2
    flagcxInt = 2
    flagcxUint32 = 3
    flagcxInt64 = 4
    flagcxUint64 = 5
    flagcxFloat16 = 6
    flagcxHalf = 6
    flagcxFloat32 = 7
    flagcxFloat = 7
    flagcxFloat64 = 8
    flagcxDouble = 8
    flagcxBfloat16 = 9
    flagcxFloat8e4m3 = 10
    flagcxFloat8e5m2 = 11
    flagcxNumTypes = 12

    @classmethod
    def from_torch(cls, dtype) -> int:
        import torch
        table = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
                 torch.float64: 8, torch.bfloat16: 9, torch.bool: 1}
        if hasattr(torch, "float8_e4m3fn"):
            table[torch.float8_e4m3fn] = 10
            table[torch.float8_e5m2] = 11
        if hasattr(torch, "uint32"):
            table[torch.uint32] = 3
            table[torch.uint64] = 5
        if dtype not in table:
            raise ValueError(f"Unsupported dtype: {dtype}")
        return table[dtype]

    @classmethod
    def from_numpy(cls, dtype) -> int:
        import numpy as np
        table = {np.dtype(np.int8): 0, np.dtype(np.uint8): 1, np.dtype(np.int32): 2, np.dtype(np.uint32): 3,
                 np.dtype(np.int64): 4, np.dtype(np.uint64): 5, np.dtype(np.float16): 6, np.dtype(np.float32): 7,
                 np.dtype(np.float64): 8}
        return table[np.dtype(dtype)]


class flagcxRedOpTypeEnum:
    flagcxSum = 0
    flagcxProd = 1
    flagcxMax = 2
    flagcxMin = 3
    flagcxAvg = 4
    flagcxNumRedOps = 5

    @classmethod
    def from_torch(cls, op) -> int:
        from torch.distributed import ReduceOp
        table = {ReduceOp.SUM: 0, ReduceOp.PRODUCT: 1, ReduceOp.MAX: 2, ReduceOp.MIN: 3, ReduceOp.AVG: 4}
        if op not in table:
            raise ValueError(f"Unsupported op: {op}")
        return table[op]


def default_library_path() -> str:
    env = os.environ.get("FLAGCX_LIBRARY_PATH")
    if env:
        return env
    return str(Path(__file__).resolve().parent / "lib" / "libflagcx.so")


_sz = ctypes.c_size_t
_szp = ctypes.POINTER(ctypes.c_size_t)

_SIGNATURES = {
    "flagcxHandleInit": (_R, [ctypes.POINTER(flagcxHandlerGroup_t)]),
    "flagcxHandleFree": (_R, [flagcxHandlerGroup_t]),
    "flagcxGetErrorString": (ctypes.c_char_p, [_R]),
    "flagcxGetLastError": (ctypes.c_char_p, [flagcxComm_t]),
    "flagcxGetVersion": (_R, [ctypes.POINTER(ctypes.c_int)]),
    "flagcxGetUniqueId": (_R, [ctypes.POINTER(flagcxUniqueId_t)]),
    "flagcxCommInitRank": (_R, [ctypes.POINTER(flagcxComm_t), ctypes.c_int, flagcxUniqueId_t, ctypes.c_int]),
    "flagcxCommFinalize": (_R, [flagcxComm_t]),
    "flagcxCommDestroy": (_R, [flagcxComm_t]),
    "flagcxCommAbort": (_R, [flagcxComm_t]),
    "flagcxCommSuspend": (_R, [flagcxComm_t]),
    "flagcxCommResume": (_R, [flagcxComm_t]),
    "flagcxCommCount": (_R, [flagcxComm_t, ctypes.POINTER(ctypes.c_int)]),
    "flagcxCommUserRank": (_R, [flagcxComm_t, ctypes.POINTER(ctypes.c_int)]),
    "flagcxCommGetDeviceNumber": (_R, [flagcxComm_t, ctypes.POINTER(ctypes.c_int)]),
    "flagcxCommGetAsyncError": (_R, [flagcxComm_t, ctypes.POINTER(_R)]),
    "flagcxCommFifoBuffer": (_R, [flagcxComm_t, ctypes.POINTER(_vp)]),
    "flagcxIsHomoComm": (_R, [flagcxComm_t, ctypes.POINTER(ctypes.c_int)]),
    "flagcxMemAlloc": (_R, [ctypes.POINTER(_vp), _sz, flagcxComm_t]),
    "flagcxMemFree": (_R, [_vp, flagcxComm_t]),
    "flagcxCommRegister": (_R, [flagcxComm_t, _vp, _sz, ctypes.POINTER(_vp)]),
    "flagcxCommDeregister": (_R, [flagcxComm_t, _vp]),
    "flagcxBarrier": (_R, [flagcxComm_t, flagcxStream_t]),
    "flagcxAllReduce": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, flagcxRedOp_t, flagcxComm_t, flagcxStream_t]),
    "flagcxReduce": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, flagcxRedOp_t, ctypes.c_int, flagcxComm_t, flagcxStream_t]),
    "flagcxAllGather": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, flagcxComm_t, flagcxStream_t]),
    "flagcxReduceScatter": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, flagcxRedOp_t, flagcxComm_t, flagcxStream_t]),
    "flagcxBroadcast": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, ctypes.c_int, flagcxComm_t, flagcxStream_t]),
    "flagcxGather": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, ctypes.c_int, flagcxComm_t, flagcxStream_t]),
    "flagcxScatter": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, ctypes.c_int, flagcxComm_t, flagcxStream_t]),
    "flagcxAlltoAll": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, flagcxComm_t, flagcxStream_t]),
    "flagcxAlltoAllv": (_R, [buffer_type, _szp, _szp, buffer_type, _szp, _szp, flagcxDataType_t, flagcxComm_t, flagcxStream_t]),
    "flagcxSend": (_R, [buffer_type, _sz, flagcxDataType_t, ctypes.c_int, flagcxComm_t, flagcxStream_t]),
    "flagcxRecv": (_R, [buffer_type, _sz, flagcxDataType_t, ctypes.c_int, flagcxComm_t, flagcxStream_t]),
    "flagcxGroupStart": (_R, [flagcxComm_t]),
    "flagcxGroupEnd": (_R, [flagcxComm_t]),
    # extensions
    "flagcxAllReduceCast": (_R, [buffer_type, buffer_type, _sz, flagcxDataType_t, flagcxDataType_t, ctypes.c_float, flagcxRedOp_t,
                                 flagcxComm_t, flagcxStream_t]),
    "flagcxCommSplit": (_R, [flagcxComm_t, ctypes.c_int, ctypes.c_int, ctypes.POINTER(flagcxComm_t)]),
    "flagcxCommSplitSized": (_R, [flagcxComm_t, ctypes.c_int, ctypes.c_int, _sz, _sz, ctypes.POINTER(flagcxComm_t)]),
    "flagcxCommSetCtaBudget": (_R, [flagcxComm_t, ctypes.c_int]),
    "flagcxCommSetZeroCopyMulticast": (_R, [flagcxComm_t, ctypes.c_int]),
    "flagcxCommHeapRetain": (_R, [flagcxComm_t]),
    "flagcxCommHeapRelease": (_R, [flagcxComm_t, _vp]),
    "flagcxTunerQueryEx": (_R, [flagcxComm_t, ctypes.c_int, _sz, flagcxDataType_t, flagcxRedOp_t, ctypes.c_int, ctypes.c_char_p, _sz,
                                ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_double)]),
    "flagcxCommGetCounters": (_R, [flagcxComm_t, ctypes.POINTER(flagcxCommCounters)]),
    "flagcxCommGetClusterInfo": (_R, [flagcxComm_t, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                      ctypes.POINTER(ctypes.c_int)]),
    "flagcxCommHeapInfo": (_R, [flagcxComm_t, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _szp]),
    "flagcxHeapOffset": (_R, [flagcxComm_t, _vp, _szp]),
    "flagcxCommSetTimeoutMs": (_R, [flagcxComm_t, ctypes.c_int]),
    "flagcxCommWaitTest": (_R, [flagcxComm_t, flagcxStream_t]),
    "flagcxCommGetDeviceError": (_R, [flagcxComm_t, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                      ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_ulonglong),
                                      ctypes.POINTER(ctypes.c_ulonglong)]),
    "flagcxCommClearError": (_R, [flagcxComm_t]),
    "flagcxCommGetNetOfRank": (_R, [flagcxComm_t, ctypes.c_int, ctypes.c_char_p, _sz]),
    "flagcxTopoNvlinkCount": (_R, [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]),
    "flagcxCommRecover": (_R, [flagcxComm_t]),
    "flagcxTunerRecord": (_R, [flagcxComm_t, ctypes.c_int, _sz, ctypes.c_char_p, ctypes.c_int, ctypes.c_double]),
    "flagcxTunerSave": (_R, [flagcxComm_t, ctypes.c_char_p]),
    "flagcxTunerLoad": (_R, [flagcxComm_t, ctypes.c_char_p]),
    "flagcxTunerPin": (_R, [flagcxComm_t, ctypes.c_char_p, ctypes.c_int]),
    "flagcxTunerPriorPlan": (_R, [ctypes.c_int, _sz, flagcxDataType_t, ctypes.c_int, ctypes.c_int, ctypes.c_char_p, _sz,
                                  ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_double)]),
    "flagcxTunerPriorPlanEx": (_R, [ctypes.c_int, _sz, flagcxDataType_t, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                    ctypes.c_char_p, _sz, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_double)]),
    "flagcxTunerQuery": (_R, [flagcxComm_t, ctypes.c_int, _sz, flagcxDataType_t, flagcxRedOp_t, ctypes.c_char_p, _sz,
                              ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_double)]),
    "flagcxEmuCreate": (_R, [ctypes.POINTER(_vp), ctypes.c_int, _sz]),
    "flagcxEmuDestroy": (_R, [_vp]),
    "flagcxEmuCollective": (_R, [_vp, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(_vp), ctypes.POINTER(_vp), _sz,
                                 flagcxDataType_t, flagcxDataType_t, ctypes.c_float, flagcxRedOp_t, ctypes.c_int, _szp, _vp]),
    "flagcxEmuSendRecv": (_R, [_vp, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(_vp),
                               ctypes.POINTER(_vp), _szp, ctypes.c_int, _vp]),
    "flagcxEmuGetError": (_R, [_vp, ctypes.POINTER(ctypes.c_int)]),
}


class FLAGCXError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"FLAGCX error {code}: {text}")
        self.code = code


class FLAGCXLibrary:
    """Loaded ``libflagcx.so`` with typed entry points."""

    _cache = {}

    def __init__(self, so_file: Optional[str] = None):
        so_file = so_file or default_library_path()
        if so_file not in FLAGCXLibrary._cache:
            lib = ctypes.CDLL(so_file)
            funcs = {}
            for name, (res, args) in _SIGNATURES.items():
                f = getattr(lib, name, None)
                if f is None:
                    continue  # e.g. the reference's libflagcx.so has none of the extensions
                f.restype = res
                f.argtypes = args
                funcs[name] = f
            FLAGCXLibrary._cache[so_file] = (lib, funcs)
        self.lib, self._funcs = FLAGCXLibrary._cache[so_file]
        self.handler = flagcxHandlerGroup_t()
        self.FLAGCX_CHECK(self._funcs["flagcxHandleInit"](ctypes.byref(self.handler)))

    def __del__(self):
        try:
            if getattr(self, "handler", None):
                self._funcs["flagcxHandleFree"](self.handler)
        except Exception:
            pass

    # ---- helpers
    def flagcxGetErrorString(self, result: int) -> str:
        return self._funcs["flagcxGetErrorString"](result).decode()

    def FLAGCX_CHECK(self, result: int) -> None:
        if result != 0:
            raise FLAGCXError(result, self.flagcxGetErrorString(result))

    def call(self, name: str, *args):
        self.FLAGCX_CHECK(self._funcs[name](*args))

    # ---- reference surface
    def flagcxGetVersion(self) -> str:
        v = ctypes.c_int()
        self.call("flagcxGetVersion", ctypes.byref(v))
        s = str(v.value)
        return f"{int(s[0])}.{int(s[1:3])}.{int(s[3:])}"

    def flagcxGetUniqueId(self) -> flagcxUniqueId:
        p = flagcxUniqueId_t()
        self.call("flagcxGetUniqueId", ctypes.byref(p))
        uid = flagcxUniqueId()
        ctypes.memmove(ctypes.byref(uid), p, 256)
        return uid

    def unique_id_from_bytes(self, data: bytes) -> flagcxUniqueId:
        if len(data) != 256:
            raise ValueError(f"expected 256 bytes, got {len(data)}")
        uid = flagcxUniqueId()
        ctypes.memmove(ctypes.addressof(uid.internal), data, 256)
        return uid

    @staticmethod
    def unique_id_to_bytes(uid: flagcxUniqueId) -> bytes:
        return bytes(bytearray(uid.internal))

    def flagcxCommInitRank(self, world_size: int, unique_id: flagcxUniqueId, rank: int):
        comm = flagcxComm_t()
        self.call("flagcxCommInitRank", ctypes.byref(comm), world_size, ctypes.byref(unique_id), rank)
        return comm

    def flagcxAllReduce(self, sendbuff, recvbuff, count, datatype, op, comm, stream=None):
        self.call("flagcxAllReduce", sendbuff, recvbuff, count, datatype, op, comm, stream)

    def flagcxReduce(self, sendbuff, recvbuff, count, datatype, op, root, comm, stream=None):
        self.call("flagcxReduce", sendbuff, recvbuff, count, datatype, op, root, comm, stream)

    def flagcxReduceScatter(self, sendbuff, recvbuff, count, datatype, op, comm, stream=None):
        self.call("flagcxReduceScatter", sendbuff, recvbuff, count, datatype, op, comm, stream)

    def flagcxAllGather(self, sendbuff, recvbuff, count, datatype, comm, stream=None):
        self.call("flagcxAllGather", sendbuff, recvbuff, count, datatype, comm, stream)

    def flagcxBroadcast(self, sendbuff, recvbuff, count, datatype, root, comm, stream=None):
        self.call("flagcxBroadcast", sendbuff, recvbuff, count, datatype, root, comm, stream)

    def flagcxGather(self, sendbuff, recvbuff, count, datatype, root, comm, stream=None):
        self.call("flagcxGather", sendbuff, recvbuff, count, datatype, root, comm, stream)

    def flagcxScatter(self, sendbuff, recvbuff, count, datatype, root, comm, stream=None):
        self.call("flagcxScatter", sendbuff, recvbuff, count, datatype, root, comm, stream)

    def flagcxAlltoAll(self, sendbuff, recvbuff, count, datatype, comm, stream=None):
        self.call("flagcxAlltoAll", sendbuff, recvbuff, count, datatype, comm, stream)

    def flagcxAlltoAllv(self, sendbuff, sendcounts: Sequence[int], sdispls: Sequence[int], recvbuff,
                        recvcounts: Sequence[int], rdispls: Sequence[int], datatype, comm, stream=None):
        n = len(sendcounts)
        arr = ctypes.c_size_t * n
        self.call("flagcxAlltoAllv", sendbuff, arr(*sendcounts), arr(*sdispls), recvbuff, arr(*recvcounts), arr(*rdispls),
                  datatype, comm, stream)

    def flagcxSend(self, sendbuff, count, datatype, dest, comm, stream=None):
        self.call("flagcxSend", sendbuff, count, datatype, dest, comm, stream)

    def flagcxRecv(self, recvbuff, count, datatype, src, comm, stream=None):
        self.call("flagcxRecv", recvbuff, count, datatype, src, comm, stream)

    def flagcxBarrier(self, comm, stream=None):
        self.call("flagcxBarrier", comm, stream)

    def flagcxGroupStart(self, comm=None):
        self.call("flagcxGroupStart", comm)

    def flagcxGroupEnd(self, comm=None):
        self.call("flagcxGroupEnd", comm)

    def flagcxCommDestroy(self, comm):
        self.call("flagcxCommDestroy", comm)

    def flagcxCommCount(self, comm) -> int:
        v = ctypes.c_int()
        self.call("flagcxCommCount", comm, ctypes.byref(v))
        return v.value

    def flagcxCommUserRank(self, comm) -> int:
        v = ctypes.c_int()
        self.call("flagcxCommUserRank", comm, ctypes.byref(v))
        return v.value

    def flagcxCommGetAsyncError(self, comm) -> int:
        v = ctypes.c_int()
        self.call("flagcxCommGetAsyncError", comm, ctypes.byref(v))
        return v.value

    # ---- memory
    def flagcxMemAlloc(self, size: int, comm=None) -> int:
        p = ctypes.c_void_p()
        self.call("flagcxMemAlloc", ctypes.byref(p), size, comm)
        return p.value

    def flagcxMemFree(self, ptr: int, comm=None):
        self.call("flagcxMemFree", ptr, comm)

    def flagcxCommRegister(self, comm, buff: int, size: int):
        h = ctypes.c_void_p()
        self.call("flagcxCommRegister", comm, buff, size, ctypes.byref(h))
        return h

    def flagcxCommDeregister(self, comm, handle):
        self.call("flagcxCommDeregister", comm, handle)

    # ---- streams through the device handle table
    def adaptor_stream_create(self):
        s = flagcxStream_t()
        self.FLAGCX_CHECK(self.handler.contents.devHandle.contents.streamCreate(ctypes.byref(s)))
        return s

    def adaptor_stream_copy(self, old_stream):
        """Wrap a ``torch.cuda.Stream`` (or a raw cudaStream_t integer)."""
        s = flagcxStream_t()
        raw = ctypes.c_void_p(getattr(old_stream, "cuda_stream", old_stream))
        self.FLAGCX_CHECK(self.handler.contents.devHandle.contents.streamCopy(ctypes.byref(s), raw))
        return s

    def adaptor_stream_free(self, stream):
        self.FLAGCX_CHECK(self.handler.contents.devHandle.contents.streamFree(stream))

    def adaptor_stream_destroy(self, stream):
        self.FLAGCX_CHECK(self.handler.contents.devHandle.contents.streamDestroy(stream))

    def sync_stream(self, stream):
        self.FLAGCX_CHECK(self.handler.contents.devHandle.contents.streamSynchronize(stream))

    # ---- extensions
    def flagcxAllReduceCast(self, sendbuff, recvbuff, count, in_type, out_type, scale, op, comm, stream=None):
        self.call("flagcxAllReduceCast", sendbuff, recvbuff, count, in_type, out_type, ctypes.c_float(scale), op, comm, stream)

    def flagcxCommSplit(self, comm, color: int, key: int):
        out = flagcxComm_t()
        self.call("flagcxCommSplit", comm, color, key, ctypes.byref(out))
        return out if out.value else None

    def flagcxCommSplitSized(self, comm, color: int, key: int, stage_bytes: int = 0, user_bytes: int = 0):
        """Split with the new communicator's heap sized explicitly (bytes of a staging half, bytes for flagcxMemAlloc)."""
        out = flagcxComm_t()
        self.call("flagcxCommSplitSized", comm, color, key, stage_bytes, user_bytes, ctypes.byref(out))
        return out if out.value else None

    def set_cta_budget(self, comm, max_ctas: int):
        """Cap the CTAs of every collective of `comm` (0 lifts the cap); the same value on every rank."""
        self.call("flagcxCommSetCtaBudget", comm, max_ctas)

    def counters(self, comm) -> dict:
        c = flagcxCommCounters()
        self.call("flagcxCommGetCounters", comm, ctypes.byref(c))
        return {"calls": list(c.calls), "bytes": list(c.bytes), "launches": c.launches, "timeouts": c.timeouts,
                "kind_launches": list(c.kindLaunches)}

    def cluster_info(self, comm):
        n = self.flagcxCommCount(comm)
        nc, mine = ctypes.c_int(), ctypes.c_int()
        arr = (ctypes.c_int * n)()
        self.call("flagcxCommGetClusterInfo", comm, ctypes.byref(nc), ctypes.byref(mine), arr)
        return nc.value, mine.value, list(arr)

    def tuner_query(self, comm, op: int, nbytes: int, dtype: int, red: int = 0):
        buf = ctypes.create_string_buffer(64)
        nctas, us = ctypes.c_int(), ctypes.c_double()
        self.call("flagcxTunerQuery", comm, op, nbytes, dtype, red, buf, 64, ctypes.byref(nctas), ctypes.byref(us))
        return buf.value.decode(), nctas.value, us.value

    def tuner_query_ex(self, comm, op: int, nbytes: int, dtype: int, red: int = 0, zero_copy: bool = False):
        buf = ctypes.create_string_buffer(64)
        nctas, us = ctypes.c_int(), ctypes.c_double()
        self.call("flagcxTunerQueryEx", comm, op, nbytes, dtype, red, int(zero_copy), buf, 64, ctypes.byref(nctas), ctypes.byref(us))
        return buf.value.decode(), nctas.value, us.value

    def tuner_prior_plan(self, op: int, nbytes: int, dtype: int, nranks: int, multicast: bool = True):
        """(kind, CTAs, estimated microseconds) the cost model picks for `nranks` GPUs; works without a GPU."""
        buf = ctypes.create_string_buffer(64)
        nctas, us = ctypes.c_int(), ctypes.c_double()
        self.call("flagcxTunerPriorPlan", op, nbytes, dtype, nranks, int(multicast), buf, 64, ctypes.byref(nctas), ctypes.byref(us))
        return buf.value.decode(), nctas.value, us.value

    def tuner_prior_plan_ex(self, op: int, nbytes: int, dtype: int, nranks: int, multicast: bool = True, zero_copy: bool = True,
                            cta_budget: int = 0):
        """Like ``tuner_prior_plan`` for peer-visible buffers (zero-copy kinds allowed) and under a CTA budget."""
        buf = ctypes.create_string_buffer(64)
        nctas, us = ctypes.c_int(), ctypes.c_double()
        self.call("flagcxTunerPriorPlanEx", op, nbytes, dtype, nranks, int(multicast), int(zero_copy), cta_budget, buf, 64,
                  ctypes.byref(nctas), ctypes.byref(us))
        return buf.value.decode(), nctas.value, us.value

    def tuner_pin(self, comm, kind: Optional[str], nctas: int = 16):
        self.call("flagcxTunerPin", comm, kind.encode() if kind else None, nctas)


__all__ = ["FLAGCXLibrary", "FLAGCXError", "flagcxUniqueId", "flagcxDataTypeEnum", "flagcxRedOpTypeEnum",
           "flagcxCommCounters", "default_library_path"]
