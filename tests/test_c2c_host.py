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


def _worker_wide(lib, uid, rank, world, tmp):
    """Gather, scatter, all-to-all and all-to-all-v through the hierarchical planner, 2 clusters x 3 ranks."""
    comm = lib.flagcxCommInitRank(world, uid, rank)
    out = {}
    cnt = 501
    x = _d(rank, cnt * world)
    for root in (1, world - 1):
        g = np.zeros(cnt * world, np.float32)
        lib.flagcxGather(_p(x), _p(g), cnt, 7, root, comm)
        if rank == root:
            out[f"gather{root}"] = bool((g == np.concatenate([_d(r, cnt * world)[:cnt] for r in range(world)])).all())
        s = np.zeros(cnt, np.float32)
        lib.flagcxScatter(_p(x), _p(s), cnt, 7, root, comm)
        out[f"scatter{root}"] = bool((s == _d(root, cnt * world)[rank * cnt:(rank + 1) * cnt]).all())
    a = np.zeros(cnt * world, np.float32)
    lib.flagcxAlltoAll(_p(x), _p(a), cnt, 7, comm)
    out["alltoall"] = bool((a == np.concatenate([_d(r, cnt * world)[rank * cnt:(rank + 1) * cnt] for r in range(world)])).all())
    sc = [37 * ((rank + p) % 3) + p for p in range(world)]
    sd = [sum(sc[:p]) for p in range(world)]
    rc = [37 * ((p + rank) % 3) + rank for p in range(world)]
    rd = [sum(rc[:p]) for p in range(world)]
    dst = np.zeros(max(1, sum(rc)), np.float32)
    lib.flagcxAlltoAllv(_p(x), sc, sd, _p(dst), rc, rd, 7, comm)
    exp = []
    for p in range(world):
        psc = [37 * ((p + q) % 3) + q for q in range(world)]
        off = sum(psc[:rank])
        exp.append(_d(p, cnt * world)[off:off + psc[rank]])
    out["alltoallv"] = bool((dst[:sum(rc)] == np.concatenate(exp)).all())
    # all-gather, all-reduce, broadcast in whatever mode the environment selects
    g = np.zeros(cnt * world, np.float32)
    lib.flagcxAllGather(_p(x), _p(g), cnt, 7, comm)
    out["allgather"] = bool((g == np.concatenate([_d(r, cnt * world)[:cnt] for r in range(world)])).all())
    y = np.zeros(cnt * world, np.float32)
    lib.flagcxAllReduce(_p(x), _p(y), cnt * world, 7, 0, comm)
    out["allreduce"] = float(np.abs(y - sum(_d(r, cnt * world).astype(np.float64) for r in range(world))).max())
    b = np.zeros(cnt, np.float32)
    lib.flagcxBroadcast(_p(x), _p(b), cnt, 7, 4, comm)
    out["broadcast"] = bool((b == _d(4, cnt * world)[:cnt]).all())
    buf = ctypes.create_string_buffer(64)
    lib.call("flagcxCommGetNetOfRank", comm, rank, buf, 64)
    out["net"] = buf.value.decode()
    out["launches"] = lib.counters(comm)["calls"]
    lib.flagcxCommDestroy(comm)
    return out


@pytest.mark.parametrize("mode", ["each", "single", "multi_from_topo_file", "hetero_p2p"])
def test_c2c_all_collectives_and_inter_rank_modes(native_lib, tmp_path, mode):
    """2 clusters x 3 ranks.  `single`: one rank per cluster talks across clusters; `multi_from_topo_file`: the
    topology file attaches three distinct ports (one cluster-wide port would give `single`); `hetero_p2p`:
    the cross-cluster stage is a planner-built list of sends and receives."""
    env = {"FLAGCX_CLUSTER_SPLIT_LIST": "2"}
    if mode == "single":
        env["FLAGCX_C2C_INTER_RANKS"] = "1"
    if mode == "hetero_p2p":
        env["FLAGCX_C2C_HETERO_P2P"] = "1"
    if mode == "multi_from_topo_file":
        topo = tmp_path / "topo.xml"
        topo.write_text('<system version="1">\n' + "".join(f'  <gpu dev="{d}" net="port{d % 3}"></gpu>\n' for d in range(6)) + "</system>\n")
        env["FLAGCX_TOPO_FILE"] = str(topo)
    res, _ = run_ranks(_worker_wide, 6, args=(str(tmp_path),), env=env, timeout=240)
    for r in range(6):
        o = res[r][1]
        for k, v in o.items():
            if k in ("net", "launches"):
                continue
            if k == "allreduce":
                assert v < 1e-5, (r, k, v)
            else:
                assert v is True, (r, k, o)
        if mode == "multi_from_topo_file":
            assert o["net"] == f"port{r % 3}"


def test_nvlink_count_through_a_stand_in_management_library(native_lib, tmp_path):
    """The link probe loads the management library at run time; here a stand-in with 18 links, 16 of them up."""
    import subprocess
    src = tmp_path / "fake_nvml.c"
    src.write_text(r'''
int nvmlInit_v2(void) { return 0; }
int nvmlShutdown(void) { return 0; }
int nvmlDeviceGetHandleByPciBusId_v2(const char *id, void **dev) { *dev = (void *)1; return id && id[0] == '0' ? 0 : 2; }
int nvmlDeviceGetNvLinkState(void *dev, unsigned link, unsigned *up) { if (link >= 18) return 2; *up = link < 16; return 0; }
int nvmlDeviceGetNvLinkVersion(void *dev, unsigned link, unsigned *v) { *v = 5; return 0; }
''')
    so = tmp_path / "libfakenvml.so"
    subprocess.check_call(["gcc", "-shared", "-fPIC", "-o", str(so), str(src)])
    os.environ["FLAGCX_NVML_LIBRARY"] = str(so)
    try:
        from flagcx_b200.wrapper import FLAGCXLibrary
        lib = FLAGCXLibrary(native_lib)
        fn = lib.lib.flagcxTopoNvlinkCount
        fn.restype = ctypes.c_int
        fn.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        n, v = ctypes.c_int(), ctypes.c_int()
        assert fn(b"0000:1b:00.0", ctypes.byref(n), ctypes.byref(v)) == 0
        assert (n.value, v.value) == (16, 5)
        assert fn(b"ffff:00:00.0", ctypes.byref(n), ctypes.byref(v)) != 0  # unknown device
    finally:
        del os.environ["FLAGCX_NVML_LIBRARY"]
