"""Hierarchical (C2C) collectives on CPU ranks.

FLAGCX_CLUSTER_SPLIT_LIST=2 cuts a 4-rank communicator into two clusters of two,
the device the reference's CI uses to exercise its cross-cluster path on one box
(.github/workflows/unit-test.yml:89).  Every planned collective is compared with
numpy; plans are exported to the reference's XML format, re-imported with
FLAGCX_C2C_ALGO=XML_INPUT, and must give the same answer."""
import ctypes
import os

import numpy as np
import pytest

from tests.mp_util import run_ranks

N = 6000


def _d(rank, n=N):
    return np.random.default_rng([7, rank]).standard_normal(n).astype(np.float32)


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _worker(lib, uid, rank, world, mode, tmp):
    if mode == "export":
        os.environ["FLAGCX_ALGO_EXPORT_PREFIX"] = os.path.join(tmp, "plan")
    if mode == "import":
        os.environ["FLAGCX_C2C_ALGO"] = "XML_INPUT"
        os.environ["FLAGCX_ALGO_IMPORT_PREFIX"] = os.path.join(tmp, "plan")
    comm = lib.flagcxCommInitRank(world, uid, rank)
    nc, mine, table = lib.cluster_info(comm)
    out = {"nclusters": nc, "cluster": mine, "table": table}
    x = _d(rank)
    y = np.zeros(N, np.float32)
    lib.flagcxAllReduce(_p(x), _p(y), N, 7, 0, comm)
    out["allreduce"] = float(np.abs(y - sum(_d(r).astype(np.float64) for r in range(world))).max())
    if mode in ("export", "import"):
        lib.flagcxCommDestroy(comm)
        return out
    cnt = N // world
    y = np.zeros(cnt, np.float32)
    lib.flagcxReduceScatter(_p(x), _p(y), cnt, 7, 0, comm)
    out["reducescatter"] = float(np.abs(y - sum(_d(r).astype(np.float64) for r in range(world))[rank * cnt:(rank + 1) * cnt]).max())
    g = np.zeros(cnt * world, np.float32)
    lib.flagcxAllGather(_p(x), _p(g), cnt, 7, comm)
    out["allgather"] = bool((g == np.concatenate([_d(r)[:cnt] for r in range(world)])).all())
    for root in (0, world - 1):
        b = np.zeros(N, np.float32)
        lib.flagcxBroadcast(_p(x), _p(b), N, 7, root, comm)
        out[f"broadcast{root}"] = bool((b == _d(root)).all())
        r_ = np.zeros(N, np.float32)
        lib.flagcxReduce(_p(x), _p(r_), N, 7, 2, root, comm)  # max
        if rank == root:
            out[f"reduce{root}"] = bool((r_ == np.maximum.reduce([_d(q) for q in range(world)])).all())
    # an operation that is not planned hierarchically still works (flat)
    a = np.zeros(cnt * world, np.float32)
    lib.flagcxAlltoAll(_p(x), _p(a), cnt, 7, comm)
    out["alltoall"] = bool((a == np.concatenate([_d(r)[rank * cnt:(rank + 1) * cnt] for r in range(world)])).all())
    # split: even / odd ranks
    sub = lib.flagcxCommSplit(comm, rank % 2, rank)
    z = np.full(8, float(rank), np.float32)
    lib.flagcxAllReduce(_p(z), _p(z), 8, 7, 0, sub)
    out["split"] = float(z[0])
    out["split_size"] = lib.flagcxCommCount(sub)
    lib.flagcxCommDestroy(comm)
    return out


@pytest.mark.parametrize("algo", ["", "RING_PIPELINED"])
def test_c2c_collectives(native_lib, tmp_path, algo):
    env = {"FLAGCX_CLUSTER_SPLIT_LIST": "2"}
    if algo:
        env["FLAGCX_C2C_ALGO"] = algo
    res, _ = run_ranks(_worker, 4, args=("all", str(tmp_path)), env=env, timeout=180)
    for r in range(4):
        o = res[r][1]
        assert o["nclusters"] == 2 and o["table"] == [0, 0, 1, 1] and o["cluster"] == r // 2
        assert o["allreduce"] < 1e-5 and o["reducescatter"] < 1e-5
        assert o["allgather"] and o["alltoall"]
        assert o["broadcast0"] and o["broadcast3"]
        if r in (0, 3):
            assert o[f"reduce{r}"]
        assert o["split_size"] == 2 and o["split"] == (2.0 if r % 2 == 0 else 4.0)


def test_c2c_plan_xml_roundtrip(native_lib, tmp_path):
    env = {"FLAGCX_CLUSTER_SPLIT_LIST": "2"}
    res, _ = run_ranks(_worker, 4, args=("export", str(tmp_path)), env=env, timeout=120)
    files = sorted(p.name for p in tmp_path.iterdir())
    assert files == [f"plan_{r}.xml" for r in range(4)]
    text = (tmp_path / "plan_1.xml").read_text()
    for tag in ("<FlagcxC2cPlanner>", "<nChunks>", "<RefreshFunc>", "<PreHomoFuncSteps>", "<HeteroFuncSteps>", "<HomoInterFuncSteps>",
                "<PostHomoFuncSteps>", "<HomoFunc>", "<commOp>8</commOp>", "<commOp>6</commOp>", "<commOp>7</commOp>"):
        assert tag in text, tag
    res, _ = run_ranks(_worker, 4, args=("import", str(tmp_path)), env=env, timeout=120)
    for r in range(4):
        assert res[r][1]["allreduce"] < 1e-5
