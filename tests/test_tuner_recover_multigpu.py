"""Two multi-GPU behaviours that only show with real ranks:

* the online tuner (FLAGCX_USE_TUNER=1) searches per call signature, so a decision found for bf16 sums is never
  applied to a call it cannot serve (an int32 or an fp32-max all-reduce in the same size bucket);
* a collective that gives up on one rank (its peer's host never launches the matching call; the wait runs
  into a short time-out and the kernel returns an error status, no GPU faults or hangs) leaves the ranks
  disagreeing on their sequence numbers, and flagcxCommRecover brings the communicator back.
"""
import ctypes

import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _setup(lib, uid, rank, world):
    torch.cuda.set_device(rank)
    torch.zeros(1, device="cuda")
    comm = lib.flagcxCommInitRank(world, uid, rank)
    return comm, lib.adaptor_stream_copy(torch.cuda.current_stream())


def _search_then_other_types(lib, uid, rank, world):
    comm, st = _setup(lib, uid, rank, world)
    n = 200000  # 400 KB of bf16: a bucket in which the switch kinds, the one-shot and the two-shot kinds all compete
    out = {}
    x = torch.full((n,), float(rank + 1), device="cuda", dtype=torch.bfloat16)
    y = torch.empty_like(x)
    for _ in range(120):  # enough calls for the search over this signature to finish (5 rounds x candidates)
        lib.flagcxAllReduce(x.data_ptr(), y.data_ptr(), n, 9, 0, comm, st)
    torch.cuda.synchronize()
    out["bf16"] = float(y.float().max().item())
    # same byte size, other signatures: int32 sum (no switch reduction for integers), fp32 max (the switch only adds fp32)
    xi = torch.full((n // 2,), rank + 1, device="cuda", dtype=torch.int32)
    yi = torch.zeros_like(xi)
    xf = torch.full((n // 2,), float(rank + 1), device="cuda")
    yf = torch.zeros_like(xf)
    for _ in range(3):
        lib.flagcxAllReduce(xi.data_ptr(), yi.data_ptr(), n // 2, 2, 0, comm, st)
        lib.flagcxAllReduce(xf.data_ptr(), yf.data_ptr(), n // 2, 7, 2, comm, st)
    torch.cuda.synchronize()
    out["int32"] = int(yi.min().item()), int(yi.max().item())
    out["fp32max"] = float(yf.min().item()), float(yf.max().item())
    # fused cast in the same bucket: bf16 in, fp32 out
    yc = torch.zeros(n, device="cuda")
    lib.flagcxAllReduceCast(x.data_ptr(), yc.data_ptr(), n, 9, 7, 1.0, 0, comm, st)
    torch.cuda.synchronize()
    out["cast"] = float(yc.min().item()), float(yc.max().item())
    out["async"] = lib.flagcxCommGetAsyncError(comm)
    lib.flagcxCommDestroy(comm)
    return out


def test_online_search_never_applies_a_decision_to_a_call_it_cannot_serve(native_lib):
    world = min(torch.cuda.device_count(), 4)
    res, _ = run_ranks(_search_then_other_types, world, timeout=300,
                       env={"FLAGCX_USE_TUNER": "1", "FLAGCX_KERNEL_TIMEOUT_MS": "20000"})
    total = world * (world + 1) // 2
    for r in range(world):
        o = res[r][1]
        assert o["async"] == 0
        assert o["bf16"] == float(total)
        assert o["int32"] == (total, total)
        assert o["fp32max"] == (float(world), float(world))
        assert o["cast"] == (float(total), float(total))


def _timeout_then_recover(lib, uid, rank, world):
    comm, st = _setup(lib, uid, rank, world)
    out = {}
    x = torch.ones(5000, device="cuda")
    lib.flagcxAllReduce(x.data_ptr(), x.data_ptr(), 5000, 7, 0, comm, st)
    torch.cuda.synchronize()
    out["first"] = float(x[0].item())
    lib.call("flagcxCommSetTimeoutMs", comm, 400)
    if rank == 0:
        # rank 0 launches a collective that nobody matches: its waits run out, the kernel returns with an error
        # record and the context stays usable (nothing traps, nothing hangs)
        z = torch.ones(5000, device="cuda")
        lib.flagcxAllReduce(z.data_ptr(), z.data_ptr(), 5000, 7, 0, comm, st)
        torch.cuda.synchronize()
        out["async_after_timeout"] = lib.flagcxCommGetAsyncError(comm)
        out["gpu_alive"] = float(torch.ones(4, device="cuda").sum().item())
    lib.call("flagcxCommSetTimeoutMs", comm, 20000)
    lib.call("flagcxCommRecover", comm)  # collective over the bootstrap network: also lines the two ranks up again
    out["async_after_recover"] = lib.flagcxCommGetAsyncError(comm)
    for i in range(3):  # both parities of every protocol word
        y = torch.full((70001,), float(rank + 1), device="cuda")
        lib.flagcxAllReduce(y.data_ptr(), y.data_ptr(), 70001, 7, 0, comm, st)
        torch.cuda.synchronize()
        out[f"sum{i}"] = float(y.min().item()), float(y.max().item())
    s = torch.full((1000,), float(rank), device="cuda")
    r_ = torch.zeros(1000, device="cuda")
    lib.flagcxGroupStart(comm)
    lib.flagcxSend(s.data_ptr(), 1000, 7, (rank + 1) % world, comm, st)
    lib.flagcxRecv(r_.data_ptr(), 1000, 7, (rank - 1) % world, comm, st)
    lib.flagcxGroupEnd(comm)
    torch.cuda.synchronize()
    out["p2p"] = float(r_[0].item())
    lib.flagcxCommDestroy(comm)
    return out


def test_recover_after_a_collective_timed_out_on_one_rank(native_lib):
    world = 2
    res, _ = run_ranks(_timeout_then_recover, world, timeout=300, env={"NCCL_NVLS_ENABLE": "0", "FLAGCX_NVLS_ENABLE": "0"})
    assert res[0][1]["async_after_timeout"] == 6 and res[0][1]["gpu_alive"] == 4.0
    for r in range(world):
        o = res[r][1]
        assert o["first"] == 2.0 and o["async_after_recover"] == 0
        for i in range(3):
            assert o[f"sum{i}"] == (3.0, 3.0)
        assert o["p2p"] == float((r - 1) % world)
