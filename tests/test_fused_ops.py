"""Numerics of the fused training kernels against plain PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def nat():
    import flagcx_b200
    return flagcx_b200.native()


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


@pytest.mark.parametrize("M,C", [(64, 256), (1000, 1024), (4096, 1024), (33, 2048), (300, 768), (40, 1536)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_layernorm(nat, M, C, with_delta):
    from flagcx_b200.ops import add_layernorm
    torch.manual_seed(0)
    x, d = _bf(M, C), (_bf(M, C) if with_delta else None)
    g, b = _bf(C) + 1, _bf(C, scale=0.1)
    xr, dr = x.float().requires_grad_(), (d.float().requires_grad_() if with_delta else None)
    gr, br = g.float().requires_grad_(), b.float().requires_grad_()
    s = (xr + dr).bfloat16().float() if with_delta else xr
    yref = F.layer_norm(s, (C,), gr, br, 1e-5)
    xq, gq, bq = x.clone().requires_grad_(), g.clone().requires_grad_(), b.clone().requires_grad_()
    dq = d.clone().requires_grad_() if with_delta else None
    res, y = add_layernorm(xq, dq, gq, bq)
    torch.testing.assert_close(y.float(), yref, atol=3e-2, rtol=3e-2)
    if with_delta:
        torch.testing.assert_close(res.float(), (x.float() + d.float()), atol=2e-2, rtol=2e-2)
    dy, dres = _bf(M, C), _bf(M, C)
    (yref * dy.float()).sum().backward(retain_graph=True)
    if with_delta:
        (s * dres.float()).sum().backward()
    torch.autograd.backward([y, res] if with_delta else [y], [dy, dres] if with_delta else [dy])
    torch.testing.assert_close(xq.grad.float(), xr.grad, atol=6e-2, rtol=6e-2)
    if with_delta:
        torch.testing.assert_close(dq.grad.float(), dr.grad, atol=6e-2, rtol=6e-2)
    # parameter gradients are sums over M rows: compare relative to their scale
    for got, ref in ((gq.grad, gr.grad), (bq.grad, br.grad)):
        err = (got.float() - ref).abs().max() / (ref.abs().max() + 1e-6)
        assert err < 3e-2, err


@pytest.mark.parametrize("M,C", [(128, 1024), (8192, 4096), (77, 512)])
def test_bias_gelu(nat, M, C):
    from flagcx_b200.ops import bias_gelu
    torch.manual_seed(1)
    x, b = _bf(M, C), _bf(C)
    xr, br = x.float().requires_grad_(), b.float().requires_grad_()
    yref = F.gelu(xr + br, approximate="tanh")
    xq, bq = x.clone().requires_grad_(), b.clone().requires_grad_()
    y = bias_gelu(xq, bq)
    torch.testing.assert_close(y.float(), yref, atol=2e-2, rtol=2e-2)
    dy = _bf(M, C)
    yref.backward(dy.float())
    y.backward(dy)
    torch.testing.assert_close(xq.grad.float(), xr.grad, atol=3e-2, rtol=3e-2)
    err = (bq.grad.float() - br.grad).abs().max() / (br.grad.abs().max() + 1e-6)
    assert err < 3e-2, err


@pytest.mark.parametrize("M,V,Vpad", [(64, 1000, 1024), (512, 50257, 50304), (7, 33, 40)])
def test_cross_entropy(nat, M, V, Vpad):
    from flagcx_b200.ops import cross_entropy
    torch.manual_seed(2)
    logits = _bf(M, Vpad, scale=2.0)
    tgt = torch.randint(0, V, (M,), device="cuda")
    lr = logits[:, :V].float().requires_grad_()
    ref = F.cross_entropy(lr, tgt)
    ref.backward()
    lq = logits.clone().requires_grad_()
    work = lq * 1  # the op consumes its input buffer
    loss = cross_entropy(work, tgt, V)
    loss.backward()
    torch.testing.assert_close(loss.float(), ref, atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(lq.grad[:, :V].float(), lr.grad, atol=2e-3 / M + 1e-5, rtol=5e-2)
    assert float(lq.grad[:, V:].abs().max()) == 0.0


def test_adamw_matches_torch(nat):
    from flagcx_b200.ops import fused_adamw_step
    torch.manual_seed(3)
    n = 100003
    w = torch.randn(n, device="cuda")
    ref_p = w.clone().requires_grad_()
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    master, param = w.clone(), w.bfloat16()
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    step_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda").bfloat16()
        ref_p.grad = g.float()
        opt.step()
        grad = g.clone()
        step_dev.add_(1)
        fused_adamw_step(master, param, grad, m, v, lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, step=step,
                         step_dev=step_dev if step % 2 else None)
        assert float(grad.abs().max()) == 0.0
    torch.testing.assert_close(master, ref_p.detach(), atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(param.float(), master, atol=1e-2, rtol=1e-2)


def test_tiny_gpt2_trains_and_graph_matches_eager(nat):
    from flagcx_b200.models.gpt2 import GPT2, GPT2Config
    from flagcx_b200.parallel.ddp import DataParallelTrainer
    cfg = GPT2Config.tiny()
    losses = {}
    for graph in (False, True):
        torch.manual_seed(5)
        tr = DataParallelTrainer(GPT2(cfg), use_graph=graph, lr=1e-3)
        tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
        tgt = torch.randint(0, cfg.vocab, (4, cfg.seq_len), device="cuda", generator=torch.Generator("cuda").manual_seed(2))
        losses[graph] = [float(tr.step(tok, tgt).item()) for _ in range(8)]
    assert losses[False][-1] < losses[False][0]
    for a, b in zip(losses[False], losses[True]):
        assert abs(a - b) < 5e-2, (losses[False], losses[True])


def test_pipelined_step_hands_out_every_loss_one_step_late(nat):
    """step_pipelined from pinned host inputs: the same loss sequence as step + item, each loss one call later."""
    from flagcx_b200.models.gpt2 import GPT2, GPT2Config
    from flagcx_b200.parallel.ddp import DataParallelTrainer
    cfg = GPT2Config.tiny()
    g = torch.Generator().manual_seed(3)
    toks = [torch.randint(0, cfg.vocab, (4, cfg.seq_len), generator=g).pin_memory() for _ in range(3)]
    tgts = [torch.randint(0, cfg.vocab, (4, cfg.seq_len), generator=g).pin_memory() for _ in range(3)]
    seqs = []
    for pipelined in (False, True):
        torch.manual_seed(5)
        tr = DataParallelTrainer(GPT2(cfg), use_graph=True, lr=1e-3)
        got = []
        for i in range(7):
            if pipelined:
                prev = tr.step_pipelined(toks[i % 3], tgts[i % 3])
                assert (prev is None) == (i == 0)
                if prev is not None:
                    got.append(prev)
            else:
                got.append(float(tr.step(toks[i % 3], tgts[i % 3]).item()))
        if pipelined:
            got.append(tr.drain())
            assert tr.drain() is None
        seqs.append(got)
    assert len(seqs[0]) == len(seqs[1]) == 7
    for a, b in zip(*seqs):
        assert abs(a - b) < 5e-2, seqs


def test_trainer_checkpoint_resume(nat):
    """A trainer resumed from state_dict() continues like the one that wrote it."""
    from flagcx_b200.models.gpt2 import GPT2, GPT2Config
    from flagcx_b200.parallel.ddp import DataParallelTrainer
    cfg = GPT2Config.tiny()
    tok = torch.randint(0, cfg.vocab, (4, cfg.seq_len), device="cuda", generator=torch.Generator("cuda").manual_seed(1))
    tgt = torch.randint(0, cfg.vocab, (4, cfg.seq_len), device="cuda", generator=torch.Generator("cuda").manual_seed(2))
    torch.manual_seed(5)
    a = DataParallelTrainer(GPT2(cfg), use_graph=False, lr=1e-3)
    for _ in range(3):
        a.step(tok, tgt)
    state = a.state_dict()
    assert state["step"] == 3 and state["master"].device.type == "cpu"
    cont = [float(a.step(tok, tgt).item()) for _ in range(3)]
    torch.manual_seed(99)  # different initial weights: everything must come from the checkpoint
    b = DataParallelTrainer(GPT2(cfg), use_graph=False, lr=1e-3)
    b.load_state_dict(state)
    resumed = [float(b.step(tok, tgt).item()) for _ in range(3)]
    for x, y in zip(cont, resumed):
        assert abs(x - y) < 2e-3, (cont, resumed)
    bad = dict(state, specs=state["specs"][:-1])
    with pytest.raises(ValueError):
        b.load_state_dict(bad)


def test_gpt2_matches_plain_torch_forward(nat):
    """Loss of the fused model equals the loss of the same weights run through plain PyTorch ops."""
    from flagcx_b200.models.gpt2 import GPT2, GPT2Config
    cfg = GPT2Config.tiny()
    torch.manual_seed(6)
    model = GPT2(cfg).cuda().bfloat16()
    tok = torch.randint(0, cfg.vocab, (2, cfg.seq_len), device="cuda")
    tgt = torch.randint(0, cfg.vocab, (2, cfg.seq_len), device="cuda")
    loss = float(model(tok, tgt).item())
    with torch.no_grad():
        p = {k: v.float() for k, v in model.named_parameters()}
        x = p["wte"][tok] + p["wpe"][: cfg.seq_len]
        for i in range(cfg.n_layer):
            pre = f"blocks.{i}."
            h = F.layer_norm(x, (cfg.d_model,), p[pre + "ln1_w"], p[pre + "ln1_b"])
            B, T, C = x.shape
            q, k, v = F.linear(h, p[pre + "qkv_w"], p[pre + "qkv_b"]).view(B, T, 3, cfg.n_head, C // cfg.n_head).unbind(2)
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
            x = x + F.linear(a.transpose(1, 2).reshape(B, T, C), p[pre + "proj_w"], p[pre + "proj_b"])
            h = F.layer_norm(x, (cfg.d_model,), p[pre + "ln2_w"], p[pre + "ln2_b"])
            x = x + F.linear(F.gelu(F.linear(h, p[pre + "fc_w"], p[pre + "fc_b"]), approximate="tanh"), p[pre + "out_w"], p[pre + "out_b"])
        h = F.layer_norm(x, (cfg.d_model,), p["lnf_w"], p["lnf_b"])
        ref = float(F.cross_entropy(F.linear(h, p["wte"][: cfg.vocab]).view(-1, cfg.vocab), tgt.view(-1)).item())
    assert abs(loss - ref) < 3e-2, (loss, ref)
