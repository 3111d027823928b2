"""Fused expert-parallel MoE layer across real GPUs (one expert per rank, and two):
every rank checks its own tokens against an fp32 reference computed from all
experts' weights, and against the all-to-all-v based unfused path."""
import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

T, H, F, K = 768, 512, 1024, 2


def _inputs(rank, world, rep):
    g = torch.Generator(device="cpu").manual_seed(1000 + 17 * rank + rep)
    x = torch.randn(T, H, generator=g).bfloat16()
    logits = torch.randn(T, world, generator=g)
    k = min(K, world)
    w, idx = torch.topk(torch.softmax(logits, -1), k, dim=-1)
    if k < K:
        idx = torch.cat([idx, idx], 1)[:, :K]
        w = torch.cat([w, w], 1)[:, :K] * 0.5
    return x, idx.int().contiguous(), w.float().contiguous()


def _weights(e):
    g = torch.Generator(device="cpu").manual_seed(5000 + e)
    return (torch.randn(2 * F, H, generator=g) * 0.05).bfloat16(), (torch.randn(H, F, generator=g) * 0.05).bfloat16()


def _worker(lib, uid, rank, world):
    import flagcx_b200
    from flagcx_b200.parallel.ep import ExpertParallelContext, moe_reference
    torch.cuda.set_device(rank)
    torch.zeros(1, device="cuda")
    comm = lib.flagcxCommInitRank(world, uid, rank)
    ep = ExpertParallelContext(comm.value, world, rank, T, H, F, K, capacity_factor=2.0, dispatch_ctas=16)
    allw = [_weights(e) for e in range(world)]
    w1, w2 = (t.cuda() for t in allw[rank])
    out = {"fails": []}
    for rep in range(4):
        x, idx, wts = (t.cuda() for t in _inputs(rank, world, rep))
        y = ep.forward(x, idx, wts, w1, w2)
        torch.cuda.synchronize()
        ref = moe_reference(x, idx, wts, [w[0].cuda() for w in allw], [w[1].cuda() for w in allw])
        e = float((y.float() - ref).abs().max() / ref.abs().max())
        if not e < 3e-2:
            out["fails"].append(("fused", rep, e))
        u = ep.unfused_forward(x, idx, wts, w1, w2)
        torch.cuda.synchronize()
        e = float((u.float() - ref).abs().max() / ref.abs().max())
        if not e < 3e-2:
            out["fails"].append(("unfused", rep, e))
    try:
        ep.check()
    except RuntimeError as ex:
        out["fails"].append(("check", str(ex)))
    lib.flagcxBarrier(comm, lib.adaptor_stream_copy(torch.cuda.current_stream()))
    del ep
    lib.flagcxCommDestroy(comm)
    return out


def test_fused_moe_layer(native_lib):
    world = min(torch.cuda.device_count(), 8)
    res, _ = run_ranks(_worker, world, timeout=600, env={"FLAGCX_KERNEL_TIMEOUT_MS": "20000"})
    for r in range(world):
        assert res[r][1]["fails"] == [], res[r][1]["fails"]


def _worker_two_experts(lib, uid, rank, world):
    """Two experts per rank (expert e on rank e // 2): routing over 2 * world experts, fused output against fp32."""
    from flagcx_b200.parallel.ep import ExpertParallelContext, moe_reference
    torch.cuda.set_device(rank)
    torch.zeros(1, device="cuda")
    comm = lib.flagcxCommInitRank(world, uid, rank)
    L, E = 2, 2 * world
    ep = ExpertParallelContext(comm.value, world, rank, T, H, F, K, capacity_factor=2.0, dispatch_ctas=16, experts_per_rank=L)
    allw = [_weights(e) for e in range(E)]
    w1 = [allw[rank * L + l][0].cuda() for l in range(L)]
    w2 = [allw[rank * L + l][1].cuda() for l in range(L)]
    out = {"fails": []}
    for rep in range(3):
        g = torch.Generator(device="cpu").manual_seed(3000 + 17 * rank + rep)
        x = torch.randn(T, H, generator=g).bfloat16().cuda()
        w, idx = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), K, dim=-1)
        idx, wts = idx.int().contiguous().cuda(), w.float().contiguous().cuda()
        y = ep.forward(x, idx, wts, w1, w2)
        torch.cuda.synchronize()
        ref = moe_reference(x, idx, wts, [w[0].cuda() for w in allw], [w[1].cuda() for w in allw])
        e = float((y.float() - ref).abs().max() / ref.abs().max())
        if not e < 3e-2:
            out["fails"].append(("fused", rep, e))
    try:
        ep.check()
    except RuntimeError as ex:
        out["fails"].append(("check", str(ex)))
    lib.flagcxBarrier(comm, lib.adaptor_stream_copy(torch.cuda.current_stream()))
    del ep
    lib.flagcxCommDestroy(comm)
    return out


def test_fused_moe_layer_two_experts_per_rank(native_lib):
    world = min(torch.cuda.device_count(), 8)
    res, _ = run_ranks(_worker_two_experts, world, timeout=600, env={"FLAGCX_KERNEL_TIMEOUT_MS": "20000"})
    for r in range(world):
        assert res[r][1]["fails"] == [], res[r][1]["fails"]
