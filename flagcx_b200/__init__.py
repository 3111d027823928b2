"""flagcx_b200: a Blackwell-native collective communication framework with the
public surface of FlagCX.

Layers (all native code lives under ``csrc/`` and is built in-tree into
``flagcx_b200/lib``):

* ``libflagcx.so``  - the C API of ``flagcx.h`` (bootstrap, symmetric heap,
  collective kernels, tuner, C2C planner, device API);
* ``_flagcx_torch`` - PyTorch ``ProcessGroup`` backend ``"flagcx"`` and the
  fused sm_100a ops used by the model code;
* ``flagcx_b200.wrapper``  - ctypes binding of the C API;
* ``flagcx_b200.models / ops / parallel / utils`` - model code, op wrappers,
  DDP / TP / EP helpers.

``import flagcx`` (the top-level shim) or ``flagcx_b200.register_backend()``
makes ``torch.distributed.init_process_group("cpu:flagcx,cuda:flagcx")`` work.
"""
from __future__ import annotations

import importlib.util
import os
import sys
from pathlib import Path

__version__ = "0.1.0"

_LIBDIR = Path(__file__).resolve().parent / "lib"
_native = None
_registered = False


def lib_path(name: str = "libflagcx.so") -> str:
    return str(_LIBDIR / name)


def native(build_if_missing: bool = True):
    """The ``_flagcx_torch`` extension module (imports torch)."""
    global _native
    if _native is not None:
        return _native
    import torch  # noqa: F401  (the extension links against libtorch)
    so = _LIBDIR / "_flagcx_torch.so"
    if not so.exists():
        if not build_if_missing:
            raise ImportError(f"{so} is missing; run `python -m flagcx_b200._build`")
        from . import _build
        _build.build_all(verbose=False)
    spec = importlib.util.spec_from_file_location("_flagcx_torch", str(so))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["_flagcx_torch"] = mod
    _native = mod
    return mod


def _create_backend(store, rank, size, timeout):
    return native().create_backend(store, rank, size, timeout)


def register_backend(name: str = "flagcx") -> None:
    """Register the c10d backend under ``name`` for CPU and CUDA tensors."""
    global _registered
    if _registered:
        return
    import torch.distributed as dist
    dist.Backend.register_backend(name, _create_backend, extended_api=False, devices=["cpu", "cuda"])
    _registered = True


def get_comm_handle(group=None, device="cuda") -> int:
    """Raw ``flagcxComm_t`` behind a process group (creating it if needed), for
    use with ``flagcx_b200.wrapper`` or the fused ops."""
    import torch
    import torch.distributed as dist
    group = group or dist.group.WORLD
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    backend = group._get_backend(dev)
    return backend.ensure_comm(dev)
