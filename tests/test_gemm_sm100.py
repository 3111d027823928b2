"""tcgen05 GEMM family against fp32 PyTorch references, on one GPU.

The fused all-gather/reduce-scatter forms run here on a one-rank communicator:
that still exercises the comm CTAs, the per-block flags, the proxy fence in
front of the TMA loads, the staging/counter path and the reduction phase."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    import flagcx_b200
    return flagcx_b200.native()


def _ref(a, b):
    return a.float() @ b.float().t()


def _close(got, ref, k):
    tol = 2e-2 * (k ** 0.5) * 0.05 + 2e-2
    err = (got.float() - ref).abs().max().item()
    scale = ref.abs().max().item() + 1e-6
    assert err / scale < 2e-2, (err, scale)
    return err


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1024, 768, 4096), (8192, 3584, 4096), (384, 200, 136), (100, 72, 8)])
def test_plain_gemm(nat, M, N, K):
    torch.manual_seed(0)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = nat.gemm_nt(a, b, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _close(c, _ref(a, b), K)


def test_plain_gemm_strided_operands(nat):
    torch.manual_seed(1)
    big_a = (torch.randn(512, 1024, device="cuda")).bfloat16()
    big_b = (torch.randn(512, 1024, device="cuda")).bfloat16()
    a, b = big_a[:, 256:768], big_b[:384, 256:768]  # row stride 1024, 512-byte offset
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = nat.gemm_nt(a, b, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _close(c, _ref(a, b), 512)


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


def test_fused_forms_on_one_rank(nat, comm1):
    from flagcx_b200.parallel.tp import TensorParallelContext
    lib, comm = comm1
    tp = TensorParallelContext(comm.value, 1, 0, max_rows=1024, max_k=1024, max_n=1024, comm_ctas=4)
    torch.manual_seed(2)
    for rep in range(3):  # both workspace parities and a reused one
        x = (torch.randn(1024, 512, device="cuda") * 0.5).bfloat16()
        w = (torch.randn(768, 512, device="cuda") * 0.5).bfloat16()
        y = tp.ag_gemm(x, w)
        z = tp.gemm_rs(x, w)
        torch.cuda.synchronize()
        tp.check()
        ref = _ref(x, w)
        _close(y, ref, 512)
        _close(z, ref, 512)


def test_tensor_parallel_linears_forward_and_backward(nat, comm1):
    """Autograd wrappers of the fused kernels against plain PyTorch autograd (one rank: gather and scatter are identities)."""
    from flagcx_b200.parallel.tp import TensorParallelContext, column_parallel_linear, row_parallel_linear
    lib, comm = comm1
    tp = TensorParallelContext(comm.value, 1, 0, max_rows=512, max_k=1024, max_n=1024)
    torch.manual_seed(5)
    x = (torch.randn(512, 256, device="cuda") * 0.5).bfloat16().requires_grad_()
    w1 = (torch.randn(1024, 256, device="cuda") * 0.05).bfloat16().requires_grad_()
    w2 = (torch.randn(256, 1024, device="cuda") * 0.05).bfloat16().requires_grad_()
    h = column_parallel_linear(x, w1, tp)
    z = row_parallel_linear(torch.nn.functional.gelu(h), w2, tp)
    z.float().square().mean().backward()
    torch.cuda.synchronize()
    tp.check()
    got = [t.grad.float().clone() for t in (x, w1, w2)]
    xr, w1r, w2r = (t.detach().float().requires_grad_() for t in (x, w1, w2))
    hr = (xr @ w1r.t()).bfloat16().float()
    zr = torch.nn.functional.gelu(hr) @ w2r.t()
    zr.square().mean().backward()
    _close(z.detach(), zr.detach(), 1024)
    for g, r in zip(got, (xr.grad, w1r.grad, w2r.grad)):
        assert (g - r).abs().max() / (r.abs().max() + 1e-12) < 5e-2


@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (1024, 3072, 8192), (384, 200, 136), (1000, 72, 24)])
def test_gemm_with_transposed_operands(nat, a_mn, b_mn, M, N, K):
    """The backward GEMMs of a linear layer read an operand transposed where it lies (MN-major tiles)."""
    torch.manual_seed(2)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    ref = _ref(a, b)
    a_st = a.t().contiguous() if a_mn else a   # stored [K, M]
    b_st = b.t().contiguous() if b_mn else b   # stored [K, N]
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = nat.gemm(a_st, b_st, a_mn, b_mn, None, 1, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _close(c, ref, K)


@pytest.mark.parametrize("split_k", [0, 2, 5])
def test_gemm_bias_and_split_k(nat, split_k):
    torch.manual_seed(3)
    M, N, K = 256, 512, 4096  # 4 tiles: the launcher's own choice (split_k = 0) splits K as well
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = nat.gemm(a, b, False, False, bias, split_k, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _close(c, _ref(a, b) + bias.float(), K)
    # weight-gradient shape: few tiles, K = tokens, both operands transposed
    T, O, I = 8192, 256, 384
    dy = (torch.randn(T, O, device="cuda") * 0.3).bfloat16()
    x = (torch.randn(T, I, device="cuda") * 0.3).bfloat16()
    dw = nat.gemm(dy, x, True, True, None, split_k, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _close(dw, dy.float().t() @ x.float(), T)


def test_linear_autograd_matches_pytorch(nat):
    from flagcx_b200.ops import gemm_error, linear
    torch.manual_seed(4)
    B, T, I, O = 4, 256, 512, 768
    x = (torch.randn(B, T, I, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w = (torch.randn(O, I, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b = torch.randn(O, device="cuda").bfloat16().requires_grad_(True)
    g = (torch.randn(B, T, O, device="cuda") * 0.1).bfloat16()
    y = linear(x, w, b)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = torch.nn.functional.linear(xr, wr, br)
    yr.backward(g.float())
    assert gemm_error() == 0
    for got, ref, k in ((y, yr, I), (x.grad, xr.grad, O), (w.grad, wr.grad, B * T), (b.grad, br.grad, B * T)):
        _close(got, ref.detach(), k)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 768, 1024), (2048, 3072, 4096), (384, 200, 136), (104, 72, 24), (4096, 1024, 8192)])
def test_pair_kernel(nat, a_mn, b_mn, M, N, K):
    """The cta_group::2 kernel (two CTAs per 256 x 256 tile), forced for every shape: whole tiles, ragged edges,
    a row count that leaves the second CTA of a pair without rows, and all four operand orientations."""
    torch.manual_seed(6)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.5).bfloat16()
    ref = _ref(a, b)
    a_st = a.t().contiguous() if a_mn else a
    b_st = b.t().contiguous() if b_mn else b
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = nat.gemm(a_st, b_st, a_mn, b_mn, None, 1, err, 1)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _close(c, ref, K)


@pytest.mark.parametrize("split_k", [0, 3, 7])
def test_pair_kernel_bias_and_split_k(nat, split_k):
    torch.manual_seed(7)
    M, N, K = 512, 512, 4096
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    c = nat.gemm(a, b, False, False, bias, split_k, err, 1)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _close(c, _ref(a, b) + bias.float(), K)
    T, O, I = 8192, 1024, 384  # weight-gradient shape: K = tokens, both operands transposed
    dy = (torch.randn(T, O, device="cuda") * 0.3).bfloat16()
    x = (torch.randn(T, I, device="cuda") * 0.3).bfloat16()
    dw = nat.gemm(dy, x, True, True, None, split_k, err, 1)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    _close(dw, dy.float().t() @ x.float(), T)


def test_gemm_accumulates_into_out(nat):
    """C += A B^T into an existing matrix, with and without a split of K, on both kernels."""
    torch.manual_seed(8)
    M, N, K = 512, 768, 2048
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.3).bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    for pair in (0, 1):
        for split_k in (1, 4):
            base = torch.randn(M, N, device="cuda").bfloat16()
            out = base.clone()
            got = nat.gemm(a, b, False, False, None, split_k, err, pair, out, True)
            torch.cuda.synchronize()
            assert got.data_ptr() == out.data_ptr() and int(err.item()) == 0
            _close(out, _ref(a, b) + base.float(), K)


def test_direct_gradients_match_autograd(nat):
    """Parameters marked for direct gradients: the fused ops add into .grad and report readiness themselves."""
    from flagcx_b200.ops import add_layernorm, bias_gelu, enable_direct_grad, gemm_error, linear
    torch.manual_seed(9)
    T, I, O = 1024, 512, 768

    def make():
        torch.manual_seed(10)
        return [(torch.randn(O, I, device="cuda") * 0.05).bfloat16().requires_grad_(True),
                torch.randn(O, device="cuda").bfloat16().requires_grad_(True),
                torch.randn(O, device="cuda").bfloat16().requires_grad_(True),
                torch.ones(I, device="cuda").bfloat16().requires_grad_(True),
                torch.zeros(I, device="cuda").bfloat16().requires_grad_(True)]

    x = (torch.randn(T, I, device="cuda") * 0.5).bfloat16()
    g = (torch.randn(T, O, device="cuda") * 0.1).bfloat16()

    def run(params):
        w, b, gb, lw, lb = params
        _, h = add_layernorm(x, None, lw, lb)
        y = bias_gelu(linear(h, w, b), gb)
        y.backward(g)

    ref = make()
    run(ref)
    direct = make()
    seen = []
    for p in direct:
        p.grad = torch.zeros_like(p)
        enable_direct_grad(p, lambda q: seen.append(q.data_ptr()))
    run(direct)
    run(direct)  # a second pass accumulates on top of the first
    torch.cuda.synchronize()
    assert gemm_error() == 0
    assert sorted(seen) == sorted([p.data_ptr() for p in direct] * 2)
    for d, r in zip(direct, ref):
        want = 2 * r.grad.float()
        assert (d.grad.float() - want).abs().max() <= 3e-2 * want.abs().max() + 1e-3


@pytest.mark.parametrize("M,N,K", [(512, 1024, 256), (8192, 4096, 1024), (300, 200, 136)])
def test_gemm_with_gelu_epilogue(nat, M, N, K):
    """One launch writes a w^T and gelu_tanh(a w^T + bias); the autograd op on it matches PyTorch."""
    from flagcx_b200.ops import gemm_error, linear_bias_gelu
    torch.manual_seed(11)
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    b = torch.randn(N, device="cuda").bfloat16()
    err = torch.zeros(1, dtype=torch.int32, device="cuda")
    pre, act = nat.gemm_bias_gelu(a, w, b, err)
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    ref = _ref(a, w)
    _close(pre, ref, K)
    want = torch.nn.functional.gelu(ref + b.float(), approximate="tanh")
    assert (act.float() - want).abs().max() < 3e-2 * (want.abs().max() + 1.0)
    if N % 8 == 0 and M % 8 == 0:
        x = a.clone().requires_grad_(True)
        wp, bp = w.clone().requires_grad_(True), b.clone().requires_grad_(True)
        g = (torch.randn(M, N, device="cuda") * 0.1).bfloat16()
        linear_bias_gelu(x, wp, bp).backward(g)
        xr, wr, br = (t.detach().float().requires_grad_(True) for t in (a, w, b))
        torch.nn.functional.gelu(torch.nn.functional.linear(xr, wr, br), approximate="tanh").backward(g.float())
        assert gemm_error() == 0
        for got, refg, k in ((x.grad, xr.grad, N), (wp.grad, wr.grad, M), (bp.grad, br.grad, M)):
            _close(got, refg, k)
