from __future__ import annotations

import torch

import flagcx_b200


def _n():
    return flagcx_b200.native()


def enable_direct_grad(param: torch.Tensor, ready=None) -> None:
    """Let this library's backward kernels add a parameter's gradient straight into ``param.grad`` (which must
    exist, e.g. as a view of a flat gradient buffer that the optimizer zeroes) instead of returning a temporary
    that autograd then adds with a kernel of its own.  The backward function returns None for such a parameter;
    autograd still runs the parameter's accumulation node, so hooks registered with
    ``register_post_accumulate_grad_hook`` keep firing, after the kernel that wrote the gradient has been queued.
    ``ready(param)`` is for callers without such hooks: it is called once per contribution (do not use both, the
    parameter would be announced twice)."""
    param._fcx_direct_grad = True
    param._fcx_grad_ready = ready


def _direct(param):
    """The tensor to accumulate into, or None when the parameter's gradient goes through autograd."""
    if param is None or not getattr(param, "_fcx_direct_grad", False):
        return None
    g = param.grad
    if g is None or g.dtype != torch.bfloat16 or not g.is_contiguous():
        return None
    return g


def _done(param):
    cb = getattr(param, "_fcx_grad_ready", None)
    if cb is not None:
        cb(param)


class _AddLayerNorm(torch.autograd.Function):
    """(res, y) = (x + delta, LayerNorm(x + delta)); one pass over the row."""

    @staticmethod
    def forward(ctx, x, delta, gamma, beta, eps):
        res, y, mean, rstd = _n().layernorm_fwd(x, delta, gamma, beta, eps)
        ctx.save_for_backward(res, gamma, mean, rstd)
        ctx.has_delta = delta is not None
        ctx.params = (gamma, beta)
        return res, y

    @staticmethod
    def backward(ctx, dres, dy):
        res, gamma, mean, rstd = ctx.saved_tensors
        dres = dres.contiguous() if dres is not None else None
        pg, pb = ctx.params
        gg, gb = _direct(pg), _direct(pb)
        if gg is not None and gb is not None:
            dx, _, _ = _n().layernorm_bwd(dy.contiguous(), res, gamma, mean, rstd, dres, gg, gb)
            _done(pg)
            _done(pb)
            return dx, (dx if ctx.has_delta else None), None, None, None
        dx, dgamma, dbeta = _n().layernorm_bwd(dy.contiguous(), res, gamma, mean, rstd, dres)
        return dx, (dx if ctx.has_delta else None), dgamma, dbeta, None


def add_layernorm(x, delta, gamma, beta, eps: float = 1e-5):
    """Returns ``(x + delta, LayerNorm(x + delta))``; ``delta`` may be None."""
    return _AddLayerNorm.apply(x, delta, gamma, beta, eps)


class _BiasGelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        ctx.save_for_backward(x, bias)
        ctx.bias_param = bias
        return _n().bias_gelu_fwd(x, bias)

    @staticmethod
    def backward(ctx, dy):
        x, bias = ctx.saved_tensors
        gb = _direct(ctx.bias_param)
        if gb is not None:
            dx, _ = _n().bias_gelu_bwd(dy.contiguous(), x, bias, gb)
            _done(ctx.bias_param)
            return dx, None
        dx, dbias = _n().bias_gelu_bwd(dy.contiguous(), x, bias)
        return dx, dbias


def bias_gelu(x, bias):
    """gelu_tanh(x + bias) with the bias gradient reduced in the backward pass."""
    return _BiasGelu.apply(x, bias)


class _CrossEntropy(torch.autograd.Function):
    """Mean softmax cross-entropy over rows.  The logits tensor is consumed:
    it is overwritten with the gradient during the forward pass, so the loss
    must be the root of the backward pass (its incoming gradient is taken as 1)."""

    @staticmethod
    def forward(ctx, logits, targets, vocab):
        m = targets.numel()
        losses = _n().cross_entropy_(logits, targets.reshape(-1), vocab, 1.0 / m)
        ctx.save_for_backward(logits)
        return losses.mean()

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        return dlogits, None, None


def cross_entropy(logits, targets, vocab: int):
    return _CrossEntropy.apply(logits, targets, vocab)


def fused_adamw_step(master, param, grad, m, v, *, lr, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, step=1,
                     grad_scale=1.0, zero_grad=True, step_dev=None):
    """One AdamW update over flat buffers (fp32 master/m/v, bf16 param/grad).
    ``step_dev`` (int32 device scalar) overrides ``step`` and keeps the bias
    correction exact inside a replayed CUDA graph."""
    _n().adamw_(master, param, grad, m, v, lr, betas[0], betas[1], eps, weight_decay, step, grad_scale, zero_grad, step_dev)


# ---------------------------------------------------------------- linear layers on the tcgen05 GEMM

_gemm_err = {}


def _err_flag(device):
    """Device int the GEMM kernels set when one of their bounded waits gives up (checked by `gemm_error`)."""
    key = (device.type, device.index)
    if key not in _gemm_err:
        _gemm_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _gemm_err[key]


def gemm_error(device=None) -> int:
    """Non-zero when a tcgen05 GEMM on this device gave up waiting (reads the device flag back)."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    return int(_err_flag(device).item())


def gemm(a, b, a_mn: bool = False, b_mn: bool = False, bias=None, split_k: int = 0):
    """bf16 GEMM on the 5th-generation tensor cores.  ``a_mn`` / ``b_mn``: the operand is stored transposed
    ([K, M] / [K, N]) and is read where it lies.  Returns ``[M, N]`` bf16."""
    return _n().gemm(a, b, a_mn, b_mn, bias, split_k, _err_flag(a.device))


class _Linear(torch.autograd.Function):
    """y = x w^T (+ bias) with all three GEMMs (forward, input gradient, weight gradient) on the library's own
    tcgen05 kernel: the backward operands are read transposed in place, the weight gradient splits its long
    reduction over the tokens across CTAs, the bias gradient is the library's column-sum kernel."""

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        ctx.in_shape = x.shape
        ctx.params = (w, bias)
        y = gemm(x2, w, False, False, bias)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, False, True).view(ctx.in_shape)      # [T,O] x [O,I]: w read as the [K=O, N=I] operand
        pw, pb = ctx.params
        if ctx.needs_input_grad[1]:
            gw = _direct(pw)
            if gw is not None and gw.shape[1] % 2 == 0:
                # [O,T] x [T,I]: both read transposed, K = tokens; added into the parameter's gradient in place
                _n().gemm(dy2, x2, True, True, None, 0, _err_flag(dy2.device), -1, gw, True)
                _done(pw)
            else:
                dw = gemm(dy2, x2, True, True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = _direct(pb)
            if gb is not None:
                _n().col_sum(dy2, gb)
                _done(pb)
            else:
                db = _n().col_sum(dy2)
        return dx, dw, db


class _LinearBiasGelu(torch.autograd.Function):
    """gelu_tanh(x w^T + bias) with the activation computed in the GEMM's epilogue: one kernel writes the product
    (kept for the backward pass) and the activation.  Backward: bias+GELU gradient kernel, then the input and
    weight gradients on the tcgen05 GEMMs."""

    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        pre, act = _n().gemm_bias_gelu(x2, w, bias, _err_flag(x2.device))
        ctx.save_for_backward(x2, w, pre, bias)
        ctx.in_shape = x.shape
        ctx.params = (w, bias)
        return act.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w, pre, bias = ctx.saved_tensors
        pw, pb = ctx.params
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        db = None
        gb = _direct(pb)
        if gb is not None:
            dpre, _ = _n().bias_gelu_bwd(dy2, pre, bias, gb)
            _done(pb)
        else:
            dpre, db = _n().bias_gelu_bwd(dy2, pre, bias)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dpre, w, False, True).view(ctx.in_shape)
        if ctx.needs_input_grad[1]:
            gw = _direct(pw)
            if gw is not None and gw.shape[1] % 2 == 0:
                _n().gemm(dpre, x2, True, True, None, 0, _err_flag(dpre.device), -1, gw, True)
                _done(pw)
            else:
                dw = gemm(dpre, x2, True, True)
        return dx, dw, db


def linear_bias_gelu(x, w, bias):
    """``gelu_tanh(linear(x, w, bias))`` for bf16 CUDA tensors with the activation fused into the GEMM's epilogue
    (forward) and the usual fused kernels in the backward pass."""
    return _LinearBiasGelu.apply(x, w, bias)


def linear(x, w, bias=None):
    """``torch.nn.functional.linear`` for bf16 CUDA tensors on the library's tcgen05 GEMM (forward and backward).
    Shapes the kernel cannot take (inner sizes that are not multiples of 8) raise; there is no silent fallback."""
    return _Linear.apply(x, w, bias)
