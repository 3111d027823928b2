"""Expert-parallel MoE pieces on one GPU against fp32 PyTorch references:
the device-row-count GEMM, SiLU-mul, and the whole fused layer on a one-rank
communicator (dispatch kernel, ROWMAP GEMM epilogue, combine kernel)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    import flagcx_b200
    return flagcx_b200.native()


@pytest.fixture(scope="module")
def comm1():
    from flagcx_b200.wrapper import FLAGCXLibrary
    lib = FLAGCXLibrary()
    torch.zeros(1, device="cuda")
    uid = lib.flagcxGetUniqueId()
    comm = lib.flagcxCommInitRank(1, uid, 0)
    yield lib, comm
    torch.cuda.synchronize()
    lib.flagcxCommDestroy(comm)


@pytest.mark.parametrize("rows", [0, 1, 127, 128, 300, 512])
def test_gemm_with_device_row_count(nat, rows):
    torch.manual_seed(rows)
    a = (torch.randn(512, 256, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(384, 256, device="cuda") * 0.5).bfloat16()
    c = torch.full((512, 384), 7.0, device="cuda", dtype=torch.bfloat16)
    m = torch.tensor([rows], dtype=torch.int32, device="cuda")
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    nat.gemm_dyn_m(a, b, c, m, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = a.float() @ b.float().t()
    if rows:
        e = (c[:rows].float() - ref[:rows]).abs().max() / ref.abs().max()
        assert e < 2e-2
    assert bool((c[rows:] == 7.0).all())  # rows beyond the count stay untouched


def test_silu_mul(nat):
    torch.manual_seed(3)
    gu = torch.randn(300, 2 * 512, device="cuda").bfloat16()
    h = torch.zeros(300, 512, device="cuda", dtype=torch.bfloat16)
    rows = torch.tensor([257], dtype=torch.int32, device="cuda")
    nat.silu_mul(gu, h, rows)
    torch.cuda.synchronize()
    ref = torch.nn.functional.silu(gu[:, :512].float()) * gu[:, 512:].float()
    assert ((h[:257].float() - ref[:257]).abs() / (ref[:257].abs() + 1.0)).max() < 2e-2
    assert bool((h[257:] == 0).all())
    nat.silu_mul(gu, h)
    torch.cuda.synchronize()
    assert ((h.float() - ref).abs() / (ref.abs() + 1.0)).max() < 2e-2


def test_fused_layer_on_one_rank(nat, comm1):
    from flagcx_b200.parallel.ep import ExpertParallelContext, moe_reference
    lib, comm = comm1
    T, H, F, K = 640, 512, 1024, 2
    ep = ExpertParallelContext(comm.value, 1, 0, T, H, F, K, dispatch_ctas=8)
    torch.manual_seed(4)
    w1 = (torch.randn(2 * F, H, device="cuda") * 0.05).bfloat16()
    w2 = (torch.randn(H, F, device="cuda") * 0.05).bfloat16()
    for rep in range(3):  # both buffer parities and a reused one
        x = torch.randn(T, H, device="cuda").bfloat16()
        idx = torch.zeros(T, K, dtype=torch.int32, device="cuda")
        idx[rep::7, 1] = -1  # a choice that is not dispatched
        wts = torch.rand(T, K, device="cuda")
        wts[idx < 0] = 0
        out = ep.forward(x, idx, wts, w1, w2)
        torch.cuda.synchronize()
        ep.check()
        assert int(ep.recv_total.item()) == int((idx == 0).sum().item())
        ref = moe_reference(x, idx, wts, [w1], [w2])
        e = (out.float() - ref).abs().max() / ref.abs().max()
        assert e < 3e-2, (rep, float(e))
        un = ep.unfused_forward(x, idx.clamp(min=0), wts, w1, w2)
        e = (un.float() - ref).abs().max() / ref.abs().max()
        assert e < 3e-2, ("unfused", rep, float(e))


def test_fused_layer_with_four_experts_on_one_rank(nat, comm1):
    """Several experts per rank: the dispatch kernel sorts the rows into one segment per local expert and every
    expert's GEMMs size themselves from their own device-resident row count."""
    from flagcx_b200.parallel.ep import ExpertParallelContext, moe_reference
    lib, comm = comm1
    T, H, F, K, L = 768, 512, 768, 2, 4
    ep = ExpertParallelContext(comm.value, 1, 0, T, H, F, K, dispatch_ctas=8, experts_per_rank=L, capacity_factor=1.5)
    torch.manual_seed(5)
    w1 = [(torch.randn(2 * F, H, device="cuda") * 0.05).bfloat16() for _ in range(L)]
    w2 = [(torch.randn(H, F, device="cuda") * 0.05).bfloat16() for _ in range(L)]
    for rep in range(3):
        x = torch.randn(T, H, device="cuda").bfloat16()
        first = torch.randint(0, L, (T,), device="cuda")
        idx = torch.stack([first, (first + 1 + torch.randint(0, L - 1, (T,), device="cuda")) % L], dim=1).int().contiguous()
        idx[rep::11, 1] = -1  # a choice that is not dispatched
        wts = torch.rand(T, K, device="cuda")
        wts[idx < 0] = 0
        out = ep.forward(x, idx, wts, w1, w2)
        torch.cuda.synchronize()
        ep.check()
        assert ep.recv_total.tolist() == [int((idx == e).sum().item()) for e in range(L)]
        ref = moe_reference(x, idx, wts, w1, w2)
        e = (out.float() - ref).abs().max() / ref.abs().max()
        assert e < 3e-2, (rep, float(e))
