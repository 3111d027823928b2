"""Reference arm of the benchmark: the UNMODIFIED reference installed under
``baseline/_ref`` (its PyTorch plugin ``flagcx`` on top of its ``libflagcx.so``,
i.e. FlagCX dispatching to NCCL), driven the way its documentation describes:
``init_process_group`` with the ``flagcx`` backend and stock
``torch.nn.parallel.DistributedDataParallel`` (25 MB buckets) around a plain
PyTorch GPT-2-medium.  Nothing of this framework is imported here.

The model is the textbook module (nn.LayerNorm, nn.Linear, tanh-GELU,
scaled_dot_product_attention, F.cross_entropy), bf16 parameters, fp32 master
weights updated by torch.optim.AdamW(fused=True).

``build_stock_ddp`` is the same model and loop on whatever process group is
already initialised; ``bench.py --impl ours-c10d`` uses it over this
framework's c10d backend, which isolates the communication library from the
model-side kernel fusion when the two arms are compared.
"""
from __future__ import annotations

import ctypes
import math
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

REF = Path(__file__).resolve().parent / "_ref"


class _Block(nn.Module):
    def __init__(self, C, H, FF, L):
        super().__init__()
        self.ln1 = nn.LayerNorm(C)
        self.qkv = nn.Linear(C, 3 * C)
        self.proj = nn.Linear(C, C)
        self.ln2 = nn.LayerNorm(C)
        self.fc = nn.Linear(C, FF)
        self.out = nn.Linear(FF, C)
        self.H = H
        for lin in (self.qkv, self.fc):
            nn.init.normal_(lin.weight, std=0.02)
        for lin in (self.proj, self.out):
            nn.init.normal_(lin.weight, std=0.02 / math.sqrt(2 * L))

    def forward(self, x):
        B, T, C = x.shape
        q, k, v = self.qkv(self.ln1(x)).view(B, T, 3, self.H, C // self.H).unbind(2)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, T, C))
        return x + self.out(F.gelu(self.fc(self.ln2(x)), approximate="tanh"))


class _GPT2(nn.Module):
    def __init__(self, L=24, H=16, C=1024, FF=4096, V=50257, T=1024):
        super().__init__()
        self.wte = nn.Embedding(V, C)
        self.wpe = nn.Embedding(T, C)
        self.blocks = nn.ModuleList([_Block(C, H, FF, L) for _ in range(L)])
        self.lnf = nn.LayerNorm(C)
        nn.init.normal_(self.wte.weight, std=0.02)
        nn.init.normal_(self.wpe.weight, std=0.02)

    def forward(self, tok, tgt):
        B, T = tok.shape
        x = self.wte(tok) + self.wpe.weight[:T]
        for b in self.blocks:
            x = b(x)
        logits = F.linear(self.lnf(x), self.wte.weight)
        return F.cross_entropy(logits.view(B * T, -1).float(), tgt.view(-1))


def build_stock_ddp(args, local_rank, device):
    """Plain PyTorch GPT-2 under stock DistributedDataParallel on whatever backend the process group has."""
    if args.model == "medium":
        model = _GPT2()
        name = "gpt2-medium"
    else:
        model = _GPT2(L=2, H=4, C=256, FF=1024, V=1000, T=64)
        name = "gpt2-tiny"
    model = model.to(device=device, dtype=torch.bfloat16)
    ddp = nn.parallel.DistributedDataParallel(model, device_ids=[local_rank], bucket_cap_mb=args.bucket_mb,
                                              gradient_as_bucket_view=True) if dist.is_initialized() else model
    params = [p for p in model.parameters()]
    master = [p.detach().float().clone().requires_grad_(True) for p in params]
    opt = torch.optim.AdamW(master, lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1, fused=True)

    class Runner:
        vocab = model.wte.weight.shape[0]

        def step(self, tok, tgt):
            if tok.device.type != "cuda":
                tok = tok.to(device, non_blocking=True)
                tgt = tgt.to(device, non_blocking=True)
            loss = ddp(tok, tgt)
            loss.backward()
            for m, p in zip(master, params):
                if m.grad is None:
                    m.grad = torch.empty_like(m)
            with torch.no_grad():
                torch._foreach_copy_([m.grad for m in master], [p.grad for p in params])
                opt.step()
                torch._foreach_copy_(params, master)
            model.zero_grad(set_to_none=False)
            return loss.detach()

        def launches_per_step(self):
            return 0

        def checksum(self):
            """Three numbers that are equal on every rank exactly when the ranks hold the same weights."""
            with torch.no_grad():
                return torch.stack([params[0].float().sum(), params[len(params) // 2].float().sum(),
                                    params[-1].float().sum()]).double().cpu()
    Runner.name = name
    return Runner()


def build_reference(args, rank, world, local_rank, device):
    # the plugin's _C extension was linked against a build-tree path; load the library by hand first
    ctypes.CDLL(str(REF / "libflagcx.so"), mode=ctypes.RTLD_GLOBAL)
    sys.path.insert(0, str(REF))
    for k in [k for k in sys.modules if k == "flagcx" or k.startswith("flagcx.")]:
        del sys.modules[k]
    import flagcx as ref_flagcx  # noqa: F401  (the reference plugin registers backend "flagcx")
    assert str(REF) in getattr(ref_flagcx, "__file__", ""), "the reference plugin must come from baseline/_ref"
    dist.init_process_group("cpu:gloo,cuda:flagcx", rank=rank, world_size=world)
    return build_stock_ddp(args, local_rank, device)
