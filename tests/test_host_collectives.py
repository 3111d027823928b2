"""CPU-only correctness of the host collective path: world_size 2..4 ranks as
processes, fp32 buffers of 1,048,576 elements per rank drawn from N(0,1) with
seed (seed, rank), compared elementwise with a numpy reference.

The reference library offers the same path (flagcx/flagcx.cc:1177-1229 with the
bootstrap host adaptor) but never checks it against an oracle."""
import ctypes

import numpy as np
import pytest

from tests.mp_util import run_ranks

N = 1 << 20
SEED = 1234


def _data(rank, n=N, dtype=np.float32):
    rng = np.random.default_rng([SEED, rank])
    return rng.standard_normal(n).astype(dtype)


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


def _worker(lib, uid, rank, world, which):
    comm = lib.flagcxCommInitRank(world, uid, rank)
    x = _data(rank)
    out = {}
    if which == "allreduce":
        y = np.empty_like(x)
        lib.flagcxAllReduce(_ptr(x), _ptr(y), N, 7, 0, comm)
        ref = sum(_data(r).astype(np.float64) for r in range(world))
        out["maxerr"] = float(np.abs(y - ref).max())
        # in place, max
        z = x.copy()
        lib.flagcxAllReduce(_ptr(z), _ptr(z), N, 7, 2, comm)
        refm = np.maximum.reduce([_data(r) for r in range(world)])
        out["max_exact"] = bool((z == refm).all())
    elif which == "allgather":
        cnt = N // world
        y = np.zeros(cnt * world, np.float32)
        lib.flagcxAllGather(_ptr(x), _ptr(y), cnt, 7, comm)
        ref = np.concatenate([_data(r)[:cnt] for r in range(world)])
        out["exact"] = bool((y == ref).all())
    elif which == "reducescatter":
        cnt = N // world
        y = np.zeros(cnt, np.float32)
        lib.flagcxReduceScatter(_ptr(x), _ptr(y), cnt, 7, 0, comm)
        ref = sum(_data(r).astype(np.float64)[rank * cnt:(rank + 1) * cnt] for r in range(world))
        out["maxerr"] = float(np.abs(y - ref).max())
    elif which == "broadcast":
        root = world - 1
        y = np.zeros(N, np.float32)
        lib.flagcxBroadcast(_ptr(x), _ptr(y), N, 7, root, comm)
        out["exact"] = bool((y == _data(root)).all())
    elif which == "others":
        cnt = 1000
        root = 0
        # reduce
        y = np.zeros(N, np.float32)
        lib.flagcxReduce(_ptr(x), _ptr(y), N, 7, 0, root, comm)
        if rank == root:
            ref = sum(_data(r).astype(np.float64) for r in range(world))
            out["reduce"] = float(np.abs(y - ref).max())
        # gather / scatter
        g = np.zeros(cnt * world, np.float32)
        lib.flagcxGather(_ptr(x), _ptr(g), cnt, 7, root, comm)
        if rank == root:
            out["gather"] = bool((g == np.concatenate([_data(r)[:cnt] for r in range(world)])).all())
        s = np.zeros(cnt, np.float32)
        lib.flagcxScatter(_ptr(x), _ptr(s), cnt, 7, root, comm)
        out["scatter"] = bool((s == _data(root)[rank * cnt:(rank + 1) * cnt]).all())
        # alltoall
        a = np.zeros(cnt * world, np.float32)
        lib.flagcxAlltoAll(_ptr(x), _ptr(a), cnt, 7, comm)
        out["alltoall"] = bool((a == np.concatenate([_data(r)[rank * cnt:(rank + 1) * cnt] for r in range(world)])).all())
        # alltoallv: rank r sends (p+1)*(r+1) elements to rank p
        sc = [(p + 1) * (rank + 1) for p in range(world)]
        sd = np.concatenate([[0], np.cumsum(sc)[:-1]]).tolist()
        rc = [(rank + 1) * (p + 1) for p in range(world)]
        rd = np.concatenate([[0], np.cumsum(rc)[:-1]]).tolist()
        v = np.zeros(sum(rc), np.float32)
        lib.flagcxAlltoAllv(_ptr(x), sc, sd, _ptr(v), rc, rd, 7, comm)
        exp = []
        for p in range(world):
            psc = [(q + 1) * (p + 1) for q in range(world)]
            psd = np.concatenate([[0], np.cumsum(psc)[:-1]])
            exp.append(_data(p)[psd[rank]:psd[rank] + psc[rank]])
        out["alltoallv"] = bool((v == np.concatenate(exp)).all())
        # grouped ring exchange + barrier
        nxt, prv = (rank + 1) % world, (rank - 1) % world
        r = np.zeros(N, np.float32)
        lib.flagcxGroupStart(comm)
        lib.flagcxSend(_ptr(x), N, 7, nxt, comm)
        lib.flagcxRecv(_ptr(r), N, 7, prv, comm)
        lib.flagcxGroupEnd(comm)
        out["sendrecv"] = bool((r == _data(prv)).all())
        lib.flagcxBarrier(comm)
        # 16-bit and 8-bit types go through fp32 on the host
        h = _data(rank, 4096).astype(np.float16)
        hy = np.zeros_like(h)
        lib.flagcxAllReduce(_ptr(h), _ptr(hy), h.size, 6, 0, comm)
        href = sum(_data(r, 4096).astype(np.float16).astype(np.float32) for r in range(world))
        out["half"] = float(np.abs(hy.astype(np.float32) - href).max())
        i8 = (np.arange(256) % 7 + rank).astype(np.int8)
        i8o = np.zeros_like(i8)
        lib.flagcxAllReduce(_ptr(i8), _ptr(i8o), i8.size, 0, 4, comm)  # avg
        iref = (sum((np.arange(256) % 7 + r) for r in range(world)) // world).astype(np.int8)
        out["int8avg"] = bool((i8o == iref).all())
    out["count"] = lib.flagcxCommCount(comm)
    out["rank"] = lib.flagcxCommUserRank(comm)
    lib.flagcxCommDestroy(comm)
    return out


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("which", ["allreduce", "allgather", "reducescatter", "broadcast"])
def test_headline_ops(native_lib, world, which):
    res, _ = run_ranks(_worker, world, args=(which,))
    for r in range(world):
        out = res[r][1]
        assert out["count"] == world and out["rank"] == r
        if "maxerr" in out:
            assert out["maxerr"] < 1e-5, out
        if "exact" in out:
            assert out["exact"], out
        if "max_exact" in out:
            assert out["max_exact"]


@pytest.mark.parametrize("world", [2, 4])
def test_remaining_ops(native_lib, world):
    res, _ = run_ranks(_worker, world, args=("others",))
    for r in range(world):
        out = res[r][1]
        for k in ("scatter", "alltoall", "alltoallv", "sendrecv", "int8avg"):
            assert out[k], (r, k, out)
        assert out["half"] < 0.05
        if r == 0:
            assert out["reduce"] < 1e-5 and out["gather"]
