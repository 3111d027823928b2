from __future__ import annotations

import torch

import flagcx_b200


def _n():
    return flagcx_b200.native()


class _AddLayerNorm(torch.autograd.Function):
    """(res, y) = (x + delta, LayerNorm(x + delta)); one pass over the row."""

    @staticmethod
    def forward(ctx, x, delta, gamma, beta, eps):
        res, y, mean, rstd = _n().layernorm_fwd(x, delta, gamma, beta, eps)
        ctx.save_for_backward(res, gamma, mean, rstd)
        ctx.has_delta = delta is not None
        return res, y

    @staticmethod
    def backward(ctx, dres, dy):
        res, gamma, mean, rstd = ctx.saved_tensors
        dres = dres.contiguous() if dres is not None else None
        dx, dgamma, dbeta = _n().layernorm_bwd(dy.contiguous(), res, gamma, mean, rstd, dres)
        return dx, (dx if ctx.has_delta else None), dgamma, dbeta, None


def add_layernorm(x, delta, gamma, beta, eps: float = 1e-5):
    """Returns ``(x + delta, LayerNorm(x + delta))``; ``delta`` may be None."""
    return _AddLayerNorm.apply(x, delta, gamma, beta, eps)


class _BiasGelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias):
        ctx.save_for_backward(x, bias)
        return _n().bias_gelu_fwd(x, bias)

    @staticmethod
    def backward(ctx, dy):
        x, bias = ctx.saved_tensors
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
