"""GPT-2 style decoder built on the fused sm_100a ops.

The data-parallel benchmark of this framework trains a GPT-2-medium shaped
decoder (24 layers, d_model 1024, 16 heads, FFN 4096, vocab 50257, sequence
1024) with random weights on random tokens.  The reference library has no
model code; its documentation only describes running third-party trainers on
top of the backend (docs/user_guide.md:137-297).

Per layer the model issues: fused residual-add + LayerNorm (one kernel), the
four projections on the library's own tcgen05 GEMM (forward with the bias
added in its epilogue, input-gradient and weight-gradient GEMMs reading their
operands transposed in place, the weight gradient with its token reduction
split across CTAs), attention through PyTorch's scaled_dot_product_attention
(a library flash-attention kernel: the one contraction this framework does not
supply itself), fused bias + GELU, and at the end one fused
softmax-cross-entropy kernel that also leaves the logit gradient in place.
``FLAGCX_MODEL_GEMM=library`` switches the projections back to the vendor GEMM
for comparison.  Parameters are bf16 views into one flat buffer so
that the optimizer and the gradient all-reduce work on contiguous memory.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from flagcx_b200.ops import add_layernorm, bias_gelu, cross_entropy, linear, linear_bias_gelu


def _linear_fn():
    return F.linear if os.environ.get("FLAGCX_MODEL_GEMM", "own") == "library" else linear


@dataclass
class GPT2Config:
    n_layer: int = 24
    n_head: int = 16
    d_model: int = 1024
    d_ff: int = 4096
    vocab: int = 50257
    seq_len: int = 1024

    @property
    def vocab_padded(self) -> int:
        return (self.vocab + 127) // 128 * 128

    @staticmethod
    def medium() -> "GPT2Config":
        return GPT2Config()

    @staticmethod
    def tiny() -> "GPT2Config":
        return GPT2Config(n_layer=2, n_head=4, d_model=256, d_ff=1024, vocab=1000, seq_len=64)


class Block(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        C = cfg.d_model
        self.n_head = cfg.n_head
        self.ln1_w = nn.Parameter(torch.ones(C))
        self.ln1_b = nn.Parameter(torch.zeros(C))
        self.qkv_w = nn.Parameter(torch.empty(3 * C, C))
        self.qkv_b = nn.Parameter(torch.zeros(3 * C))
        self.proj_w = nn.Parameter(torch.empty(C, C))
        self.proj_b = nn.Parameter(torch.zeros(C))
        self.ln2_w = nn.Parameter(torch.ones(C))
        self.ln2_b = nn.Parameter(torch.zeros(C))
        self.fc_w = nn.Parameter(torch.empty(cfg.d_ff, C))
        self.fc_b = nn.Parameter(torch.zeros(cfg.d_ff))
        self.out_w = nn.Parameter(torch.empty(C, cfg.d_ff))
        self.out_b = nn.Parameter(torch.zeros(C))
        std = 0.02
        nn.init.normal_(self.qkv_w, std=std)
        nn.init.normal_(self.fc_w, std=std)
        nn.init.normal_(self.proj_w, std=std / math.sqrt(2 * cfg.n_layer))
        nn.init.normal_(self.out_w, std=std / math.sqrt(2 * cfg.n_layer))

    def forward(self, x, delta):
        """x: residual stream [B, T, C]; delta: pending update not yet added."""
        B, T, C = x.shape
        lin = _linear_fn()
        x, h = add_layernorm(x, delta, self.ln1_w, self.ln1_b)
        qkv = lin(h, self.qkv_w, self.qkv_b).view(B, T, 3, self.n_head, C // self.n_head)
        q, k, v = qkv.unbind(2)
        att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        att = att.transpose(1, 2).reshape(B, T, C)
        a = lin(att, self.proj_w, self.proj_b)
        x, h = add_layernorm(x, a, self.ln2_w, self.ln2_b)
        if lin is linear and os.environ.get("FLAGCX_MODEL_FUSED_GELU", "1") != "0":
            f = linear_bias_gelu(h, self.fc_w, self.fc_b)  # the activation comes out of the GEMM's epilogue
        else:
            f = bias_gelu(lin(h, self.fc_w), self.fc_b)
        return x, lin(f, self.out_w, self.out_b)


class GPT2(nn.Module):
    def __init__(self, cfg: GPT2Config):
        super().__init__()
        self.cfg = cfg
        C = cfg.d_model
        self.wte = nn.Parameter(torch.empty(cfg.vocab_padded, C))  # rows >= vocab are padding (kept at zero)
        self.wpe = nn.Parameter(torch.empty(cfg.seq_len, C))
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.n_layer)])
        self.lnf_w = nn.Parameter(torch.ones(C))
        self.lnf_b = nn.Parameter(torch.zeros(C))
        nn.init.normal_(self.wte, std=0.02)
        nn.init.normal_(self.wpe, std=0.02)
        with torch.no_grad():
            self.wte[cfg.vocab:].zero_()

    def forward(self, tokens, targets):
        """tokens, targets: int64 [B, T] on the GPU.  Returns the mean loss."""
        B, T = tokens.shape
        x = F.embedding(tokens, self.wte) + self.wpe[:T]
        delta = None
        for blk in self.blocks:
            x, delta = blk(x, delta)
        _, h = add_layernorm(x, delta, self.lnf_w, self.lnf_b)
        logits = _linear_fn()(h.view(B * T, -1), self.wte)  # [B*T, vocab_padded]
        return cross_entropy(logits, targets, self.cfg.vocab)

    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    def direct_grad_parameters(self):
        """``(parameter, single_use)`` pairs for ``flagcx_b200.ops.enable_direct_grad``: parameters whose gradient this
        model's fused ops can add straight into ``.grad``.  ``single_use`` is False for the token embedding: it is tied
        to the output projection, whose weight gradient is added in place early in the backward pass, while the
        embedding lookup's own gradient arrives through autograd at the very end."""
        out = []
        for p in self.parameters():
            if p is self.wpe:
                continue
            out.append((p, p is not self.wte))
        return out


def flatten_parameters(model: nn.Module, dtype=torch.bfloat16, device="cuda", buffer: torch.Tensor | None = None):
    """Move every parameter into one flat ``dtype`` buffer (each parameter
    becomes a view) and return ``(flat_params, [(name, offset, numel)])``.
    Offsets are padded to 128 elements so that every view is 256-byte aligned."""
    specs, total = [], 0
    for name, p in model.named_parameters():
        specs.append((name, total, p.numel()))
        total += (p.numel() + 127) // 128 * 128
    flat = buffer if buffer is not None else torch.zeros(total, dtype=dtype, device=device)
    assert flat.numel() >= total
    with torch.no_grad():
        for (name, off, n), p in zip(specs, list(model.parameters())):
            view = flat[off:off + n].view(p.shape)
            view.copy_(p.detach().to(device=device, dtype=dtype))
            p.data = view
    return flat[:total] if flat.numel() != total else flat, specs
