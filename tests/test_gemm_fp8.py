"""Block-scaled fp8 GEMM (tcgen05 kind::f8f6f4 with per-128 promotion) and its quantisation kernels
against fp32 PyTorch references on one GPU."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    import flagcx_b200
    return flagcx_b200.native()


def _dequant_act(q, sa):
    m, k = q.shape
    return q.float() * sa.t().repeat_interleave(128, dim=1)[:, :k]


def _dequant_weight(q, sb):
    n, k = q.shape
    return q.float() * sb.repeat_interleave(128, dim=0)[:n].repeat_interleave(128, dim=1)[:, :k]


def test_quantisation_matches_reference(nat):
    torch.manual_seed(0)
    x = (torch.randn(300, 512, device="cuda") * 3).bfloat16()
    q, sa = nat.quant_fp8_act(x)
    assert q.dtype == torch.float8_e4m3fn and sa.shape == (4, 300)
    amax = x.float().view(300, 4, 128).abs().amax(-1)
    torch.testing.assert_close(sa.t(), amax / 448.0, rtol=1e-6, atol=0)
    back = _dequant_act(q, sa)
    assert ((back - x.float()).abs() <= 0.07 * amax.repeat_interleave(128, dim=1) + 1e-6).all()  # e4m3: 3 mantissa bits
    w = (torch.randn(200, 384, device="cuda")).bfloat16()
    qw, sb = nat.quant_fp8_weight(w)
    assert sb.shape == (2, 3)
    pad = torch.zeros(256, 384, device="cuda")
    pad[:200] = w.float()
    amaxw = pad.view(2, 128, 3, 128).abs().amax((1, 3))
    torch.testing.assert_close(sb, amaxw / 448.0, rtol=1e-6, atol=0)
    backw = _dequant_weight(qw, sb)
    assert ((backw - w.float()).abs() <= 0.07 * amaxw.repeat_interleave(128, 0)[:200].repeat_interleave(128, 1) + 1e-6).all()


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (256, 384, 512), (1000, 200, 1024), (4096, 2048, 4096), (77, 72, 256)])
def test_blockwise_fp8_gemm(nat, M, N, K):
    torch.manual_seed(M + N + K)
    # rows and blocks with very different magnitudes: per-block scales matter
    x = (torch.randn(M, K, device="cuda") * torch.logspace(-2, 2, M, device="cuda").unsqueeze(1)).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    q, sa = nat.quant_fp8_act(x)
    qw, sb = nat.quant_fp8_weight(w)
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = nat.gemm_fp8_nt(q, sa, qw, sb, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = _dequant_act(q, sa) @ _dequant_weight(qw, sb).t()  # same quantised inputs, fp32 math
    rel = ((c.float() - ref).abs() / (ref.abs().amax(1, keepdim=True) + 1e-9)).max().item()
    assert rel < 1e-2, rel
    # and the quantised product stays close to the bf16 one
    full = x.float() @ w.float().t()
    rel2 = ((c.float() - full).abs() / (full.abs().amax(1, keepdim=True) + 1e-9)).max().item()
    assert rel2 < 0.1, rel2
