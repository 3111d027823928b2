"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels across real GPUs,
compared with fp32 references assembled from every rank's inputs, plus the
in-kernel ring exchange of the device API."""
import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _x(rank, rows, k):
    g = torch.Generator(device="cpu").manual_seed(50 + rank)
    return (torch.randn(rows, k, generator=g) * 0.5).bfloat16()


def _worker(lib, uid, rank, world):
    import flagcx_b200
    from flagcx_b200.parallel.tp import TensorParallelContext
    torch.cuda.set_device(rank)
    torch.zeros(1, device="cuda")
    nat = flagcx_b200.native()
    comm = lib.flagcxCommInitRank(world, uid, rank)
    rows, K, N = 128 * 4 * world, 1024, 1536
    tp = TensorParallelContext(comm.value, world, rank, max_rows=rows, max_k=K, max_n=N)
    g = torch.Generator(device="cpu").manual_seed(7)
    w = (torch.randn(N, K, generator=g) * 0.5).bfloat16().cuda()
    w2 = (torch.randn(K, N, generator=g) * 0.5).bfloat16().cuda()
    out = {"fails": []}
    full = torch.cat([_x(r, rows // world, K) for r in range(world)]).float()
    for rep in range(4):
        xl = _x(rank, rows // world, K).cuda()
        y = tp.ag_gemm(xl, w)
        torch.cuda.synchronize()
        ref = full @ w.float().cpu().t()
        e = (y.float().cpu() - ref).abs().max() / ref.abs().max()
        if e > 2e-2:
            out["fails"].append(("ag_gemm", rep, float(e)))
        # exit side: every rank multiplies its own [rows, N] activation by its weight shard; outputs are summed and scattered
        a = (y * (0.01 * (rank + 1))).bfloat16()
        z = tp.gemm_rs(a, w2)
        torch.cuda.synchronize()
        acc = None
        for r in range(world):
            ar = (y.float().cpu() * (0.01 * (r + 1))).bfloat16().float()
            part = ar @ w2.float().cpu().t()
            acc = part if acc is None else acc + part
        refz = acc[rank * rows // world:(rank + 1) * rows // world]
        e = (z.float().cpu() - refz).abs().max() / refz.abs().max()
        if e > 3e-2:
            out["fails"].append(("gemm_rs", rep, float(e)))
        zu = tp.unfused_gemm_rs(a, w2)
        torch.cuda.synchronize()
        e = (zu.float().cpu() - refz).abs().max() / refz.abs().max()
        if e > 3e-2:
            out["fails"].append(("unfused_gemm_rs", rep, float(e)))
    tp.check()
    # ring exchange with the in-kernel API: two inboxes used alternately
    slot = nat.alloc_signals(comm.value, 2)  # data-ready signal and consumed acknowledgement
    inbox = [nat.heap_tensor(comm.value, [1 << 20], torch.float32) for _ in range(2)]
    for epoch in range(1, 5):
        src = torch.full((1 << 20,), float(rank * 10 + epoch), device="cuda")
        dst = torch.zeros(1 << 20, device="cuda")
        nat.ring_exchange(comm.value, src, inbox[epoch & 1], dst, slot, epoch)
        torch.cuda.synchronize()
        if not bool((dst == ((rank - 1) % world) * 10 + epoch).all()):
            out["fails"].append(("ring", epoch))
    lib.flagcxBarrier(comm, lib.adaptor_stream_copy(torch.cuda.current_stream()))
    del tp, inbox
    lib.flagcxCommDestroy(comm)
    return out


def test_fused_tp_kernels(native_lib):
    world = min(torch.cuda.device_count(), 8)
    res, _ = run_ranks(_worker, world, timeout=600, env={"FLAGCX_KERNEL_TIMEOUT_MS": "20000"})
    for r in range(world):
        assert res[r][1]["fails"] == [], res[r][1]["fails"]
