"""In-tree build of the native parts.

``libflagcx.so`` (C API, runtime, collective kernels) is built with nvcc/g++
directly; the PyTorch pieces (c10d backend and fused ops) are built with
``torch.utils.cpp_extension`` conventions but by the same explicit compiler
calls, so the shared objects land inside the package (``flagcx_b200/lib``)
and travel with the source tree.

Every CUDA source is compiled for sm_100a only:
``-gencode arch=compute_100a,code=sm_100a``.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shlex
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = ROOT / "flagcx_b200" / "lib"
OBJDIR = ROOT / "build" / "obj"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

COMMON_INC = [f"-I{CSRC / 'include'}", f"-I{CSRC}", f"-I{CUDA_HOME / 'include'}"]
CXXFLAGS = ["-O2", "-g", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread"]
NVCCFLAGS = ARCH + ["-O3", "-lineinfo", "-std=c++17", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
                    "-Xptxas", "-v"]


# FLAGCX_SANITIZE=address|thread builds a second copy of libflagcx.so with the host code instrumented
# (build/san/<kind>/libflagcx.so); the CPU tests then run against it with the sanitizer runtime preloaded.
SANITIZE = os.environ.get("FLAGCX_SANITIZE", "")
if SANITIZE:
    OBJDIR = ROOT / "build" / f"obj_{SANITIZE}"
    LIBDIR_NATIVE = ROOT / "build" / "san" / SANITIZE
    CXXFLAGS = CXXFLAGS + [f"-fsanitize={SANITIZE}", "-fno-omit-frame-pointer"]
    NVCCFLAGS = NVCCFLAGS + ["-Xcompiler", f"-fsanitize={SANITIZE}", "-Xcompiler", "-fno-omit-frame-pointer"]
else:
    LIBDIR_NATIVE = LIBDIR


def _run(cmd, log=None):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        Path(log).write_text(" ".join(shlex.quote(c) for c in cmd) + "\n" + proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout)
        raise RuntimeError("build step failed: " + " ".join(cmd[:6]) + " ...")
    return proc.stdout


def _stamp(src: Path, flags) -> str:
    h = hashlib.sha1()
    h.update(src.read_bytes())
    h.update(" ".join(flags).encode())
    # headers: cheap but safe - hash every header under csrc
    for hdr in sorted(CSRC.rglob("*.h")) + sorted(CSRC.rglob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()


def _compile(src: Path, extra_inc=(), extra_flags=(), force=False) -> Path:
    rel = src.relative_to(CSRC)
    obj = OBJDIR / (str(rel).replace("/", "__") + ".o")
    obj.parent.mkdir(parents=True, exist_ok=True)
    is_cu = src.suffix == ".cu"
    flags = (NVCCFLAGS if is_cu else CXXFLAGS) + list(extra_flags) + COMMON_INC + list(extra_inc)
    stamp_file = obj.with_suffix(".stamp")
    stamp = _stamp(src, flags)
    if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return obj
    cmd = ([NVCC] if is_cu else ["g++"]) + flags + ["-c", str(src), "-o", str(obj)]
    _run(cmd, log=obj.with_suffix(".log"))
    stamp_file.write_text(stamp)
    return obj


def native_sources():
    srcs = []
    for sub in ("core", "c2c", "kernels"):
        d = CSRC / sub
        if d.is_dir():
            srcs += sorted(p for p in d.iterdir() if p.suffix in (".cc", ".cu"))
    return srcs


def build_native(force=False, verbose=False) -> Path:
    """Build flagcx_b200/lib/libflagcx.so (or the sanitizer copy when FLAGCX_SANITIZE is set)."""
    LIBDIR_NATIVE.mkdir(parents=True, exist_ok=True)
    OBJDIR.mkdir(parents=True, exist_ok=True)
    srcs = native_sources()
    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(lambda s: _compile(s, force=force), srcs))
    out = LIBDIR_NATIVE / "libflagcx.so"
    newest = max(o.stat().st_mtime for o in objs)
    if force or not out.exists() or out.stat().st_mtime < newest:
        # the sanitizer runtime is preloaded by the process, so its symbols stay undefined at link time
        san = ["-Xcompiler", f"-fsanitize={SANITIZE}"] if SANITIZE else ["-Xlinker", "-z", "-Xlinker", "defs"]
        cmd = [NVCC, "-shared", "-o", str(out)] + [str(o) for o in objs] + ARCH + [
            "-cudart", "static", "-Xlinker", "--no-as-needed", "-lpthread", "-ldl", "-lrt"] + san
        _run(cmd)
    if verbose:
        print(f"built {out}")
    return out


def torch_flags():
    import torch
    from torch.utils import cpp_extension as ce
    inc = [f"-I{p}" for p in ce.include_paths()]
    import sysconfig
    inc.append(f"-I{sysconfig.get_paths()['include']}")
    abi = getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True)
    defs = [f"-D_GLIBCXX_USE_CXX11_ABI={int(bool(abi))}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    libdir = str(Path(torch.__file__).parent / "lib")
    return inc, defs, libdir


def build_torch_ext(force=False, verbose=False) -> Path:
    """Build flagcx_b200/lib/_flagcx_torch.so: the c10d backend and the fused ops."""
    lib = build_native(force=force, verbose=verbose)
    inc, defs, tlib = torch_flags()
    tdir = CSRC / "torch"
    srcs = sorted(p for p in tdir.iterdir() if p.suffix in (".cpp", ".cu")) if tdir.is_dir() else []
    objs = []

    def comp(src):
        rel = src.relative_to(CSRC)
        obj = OBJDIR / (str(rel).replace("/", "__") + ".o")
        is_cu = src.suffix == ".cu"
        base = (NVCCFLAGS if is_cu else CXXFLAGS + ["-Wno-sign-compare", "-Wno-unknown-pragmas"])
        flags = base + defs + COMMON_INC + inc + ["-DTORCH_EXTENSION_NAME=_flagcx_torch"]
        stamp_file = obj.with_suffix(".stamp")
        stamp = _stamp(src, flags)
        if not force and obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
            return obj
        cmd = ([NVCC] if is_cu else ["g++"]) + flags + ["-c", str(src), "-o", str(obj)]
        _run(cmd, log=obj.with_suffix(".log"))
        stamp_file.write_text(stamp)
        return obj

    with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(comp, srcs))
    out = LIBDIR / "_flagcx_torch.so"
    newest = max([o.stat().st_mtime for o in objs] + [lib.stat().st_mtime])
    if force or not out.exists() or out.stat().st_mtime < newest:
        cmd = [NVCC, "-shared", "-o", str(out)] + [str(o) for o in objs] + ARCH + [
            "-cudart", "shared", f"-L{LIBDIR}", "-lflagcx", f"-L{tlib}", "-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python",
            "-lc10_cuda", "-ltorch_cuda", "-Xlinker", "-rpath=$ORIGIN", "-Xlinker", f"-rpath={tlib}"]
        _run(cmd)
    if verbose:
        print(f"built {out}")
    return out


def build_tools(force=False, verbose=False) -> Path:
    """Build build/bin/flagcx_perf, the MPI-free perf binary with the reference's command line."""
    src = CSRC / "tools" / "flagcx_perf.cc"
    out = ROOT / "build" / "bin" / "flagcx_perf"
    out.parent.mkdir(parents=True, exist_ok=True)
    if force or not out.exists() or out.stat().st_mtime < src.stat().st_mtime:
        _run([NVCC, "-O2", "-std=c++17", "-x", "cu"] + ARCH + COMMON_INC + [str(src), "-o", str(out), "-ldl"])
    if verbose:
        print(f"built {out}")
    return out


def build_all(force=False, verbose=True):
    build_native(force=force, verbose=verbose)
    build_torch_ext(force=force, verbose=verbose)
    build_tools(force=force, verbose=verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
