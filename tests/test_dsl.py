"""The InterOp DSL: symbolic checking and XML generation, and the C2C
planner executing a DSL-written plan on four CPU ranks."""
import ctypes
import os

import numpy as np

from flagcx_b200.tools import (BuffRef, Collective, FlagcxWorkflow, Param, Primitive, Stage, add_opr, check, explain, init_buffer,
                               set_pipeline, set_refresh, RedOp, to_xml)
from tests.mp_util import run_ranks


def _allreduce_2x2(outdir=None, break_it=False, use_p2p=False):
    """All-reduce over 2 clusters x 2 ranks: reduce-scatter inside, exchange across, all-gather inside.
    With use_p2p the cross-cluster step is a pair of send/recv plus a local-cluster reduce written as
    a second all-reduce... kept simple: p2p variant swaps partial sums and re-reduces inside the cluster."""
    with FlagcxWorkflow("ar", Collective.AllReduce, [], [], 4, clusters=[[0, 1], [2, 3]]) as wf:
        send = [init_buffer(r, 0, 2) for r in range(4)]
        recv = [init_buffer(r, 1, 2) for r in range(4)]
        scr = [init_buffer(r, 2, 1) for r in range(4)]
        set_pipeline(1, 0, 1, 0, 1)
        for r in range(4):
            set_refresh(r, -1, 0, 0, 0, 0, RedOp.sum)
            add_opr(r, Stage.PreHomoFunc, 0, {Param.send_buff: BuffRef(send[r], 0, 2), Param.recv_buff: BuffRef(scr[r], 0, 1),
                                              Param.count: 1, Param.homo_type: 0, Param.comm_op: Primitive.ReduceScatter})
            add_opr(r, Stage.HeteroFunc, 0, None)
            if not break_it:
                add_opr(r, Stage.HomoInterFunc, 0, {Param.send_buff: BuffRef(scr[r], 0, 1), Param.recv_buff: BuffRef(scr[r], 0, 1),
                                                    Param.count: 1, Param.homo_type: 1, Param.comm_op: Primitive.AllReduce})
            else:
                add_opr(r, Stage.HomoInterFunc, 0, None)
            add_opr(r, Stage.PostHomoFunc, 0, {Param.send_buff: BuffRef(scr[r], 0, 1), Param.recv_buff: BuffRef(recv[r], 0, 1),
                                               Param.count: 1, Param.homo_type: 2, Param.comm_op: Primitive.AllGather})
        ok = check()
        msgs = explain()
        texts = [to_xml(r, outdir) if outdir else to_xml(r) for r in range(4)]
    return ok, msgs, texts


def test_checker_accepts_correct_and_rejects_broken_plan():
    ok, msgs, texts = _allreduce_2x2()
    assert ok, msgs
    assert "<commOp>8</commOp>" in texts[0] and "<nChunks>2</nChunks>" in texts[0] and "<homoType>1</homoType>" in texts[0]
    ok, msgs, _ = _allreduce_2x2(break_it=True)
    assert not ok and any("expected" in m for m in msgs)


def test_checker_models_p2p_exchange():
    # two clusters of one rank: all-reduce by swapping buffers and ... each rank ends with only the peer's data: must fail
    with FlagcxWorkflow("swap", Collective.AllReduce, [], [], 2, clusters=[[0], [1]]):
        send = [init_buffer(r, 0, 1) for r in range(2)]
        recv = [init_buffer(r, 1, 2) for r in range(2)]
        set_pipeline(1, 0, 0, 0, 0)
        for r in range(2):
            # copy own input into the receive buffer with a one-rank broadcast, then swap chunk 0 into the peer's chunk 1
            add_opr(r, Stage.PreHomoFunc, 0, {Param.send_buff: BuffRef(send[r], 0, 1), Param.recv_buff: BuffRef(recv[r], 0, 1),
                                              Param.count: 1, Param.homo_type: 0, Param.comm_op: Primitive.Broadcast,
                                              Param.peer_or_root_rank: 0})
            add_opr(r, Stage.HeteroFunc, 0, {Param.peer_or_root_rank: 1 - r, Param.send_offset: 0, Param.recv_offset: 1, Param.count: 1})
        assert not check()  # chunk 1 holds the peer's chunk 0, not a sum
        assert any("receive chunk" in m for m in explain())


def _run_plan(lib, uid, rank, world, prefix):
    os.environ["FLAGCX_C2C_ALGO"] = "XML_INPUT"
    os.environ["FLAGCX_ALGO_IMPORT_PREFIX"] = prefix
    comm = lib.flagcxCommInitRank(world, uid, rank)
    n = 4096
    x = np.random.default_rng([3, rank]).standard_normal(n).astype(np.float32)
    y = np.zeros(n, np.float32)
    lib.flagcxAllReduce(ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(y.ctypes.data), n, 7, 0, comm)
    ref = sum(np.random.default_rng([3, r]).standard_normal(n).astype(np.float64) for r in range(world))
    lib.flagcxCommDestroy(comm)
    return float(np.abs(y - ref).max())


def test_planner_executes_dsl_plan(native_lib, tmp_path):
    ok, msgs, _ = _allreduce_2x2(outdir=str(tmp_path))
    assert ok, msgs
    res, _ = run_ranks(_run_plan, 4, args=(str(tmp_path / "ar"),), env={"FLAGCX_CLUSTER_SPLIT_LIST": "2"}, timeout=120)
    for r in range(4):
        assert res[r][1] < 1e-5
