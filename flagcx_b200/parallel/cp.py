"""Long-context attention over a process group, written on the c10d operations of this library's backend.

The reference ships no sequence-parallel strategy; its building blocks for one are the send/recv ring of its perf test
(test/perf/test_sendrecv.cpp:50-51, 110-113) and ``all_to_all_single`` of its torch plug-in
(plugin/torch/flagcx/src/backend_flagcx.cpp:624-683).  Two strategies on exactly those operations:

* ``ring_attention``     context parallelism: every rank keeps its slice of the queries and the key/value blocks travel
                         round the ring (grouped send + receive per step, ``batch_isend_irecv``), partial results are
                         merged with the running-maximum softmax; with a causal mask the blocks that lie entirely in the
                         future are skipped.
* ``ulysses_attention``  head parallelism: one all-to-all turns the sequence-sharded [B, T/n, H, D] tensors into
                         head-sharded [B, T, H/n, D] ones, attention runs locally on whole sequences, a second all-to-all
                         turns the result back.

Both are differentiable: the communication steps are autograd functions whose backward is the mirrored transfer.  On
CUDA tensors the transfers are this library's grouped send/recv and all-to-all kernels; on CPU tensors the TCP host path.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


class _RingShift(torch.autograd.Function):
    """y on rank r = x of rank r - 1 (one grouped send + receive); backward moves the gradient the other way."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _shift(x, group, +1)

    @staticmethod
    def backward(ctx, g):
        return _shift(g.contiguous(), ctx.group, -1), None


def _shift(x, group, direction):
    n, r = dist.get_world_size(group), dist.get_rank(group)
    if n == 1:
        return x.clone()
    to, frm = (r + direction) % n, (r - direction) % n
    x = x.contiguous()
    out = torch.empty_like(x)
    ops = [dist.P2POp(dist.isend, x, dist.get_global_rank(group, to) if group is not None else to, group),
           dist.P2POp(dist.irecv, out, dist.get_global_rank(group, frm) if group is not None else frm, group)]
    for req in dist.batch_isend_irecv(ops):
        req.wait()
    return out


def _block(q, k, v, scale, mask):
    """Scores of one key/value block in fp32 (fp64 inputs stay fp64): (row maximum, row sum of exp, unnormalised output)."""
    ct = torch.promote_types(q.dtype, torch.float32)
    q, k, v = q.to(ct), k.to(ct), v.to(ct)
    s = torch.matmul(q, k.transpose(-1, -2)) * scale
    if mask is not None:
        s = s.masked_fill(~mask, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)  # a fully masked row contributes nothing
    p = torch.exp(s - m)
    return m, p.sum(dim=-1, keepdim=True), torch.matmul(p, v)


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, causal: bool = False, scale: float | None = None):
    """Attention over a sequence sharded across the group.  ``q``, ``k``, ``v``: [B, H, T/n, D], rank r holding tokens
    [r T/n, (r+1) T/n).  Returns this rank's [B, H, T/n, D] slice of the output, in the dtype of ``q``."""
    n, r = dist.get_world_size(group), dist.get_rank(group)
    tl, d = q.shape[-2], q.shape[-1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    m_run = l_run = acc = None
    kv = torch.stack([k, v])  # one transfer per step
    tri = torch.ones(tl, tl, dtype=torch.bool, device=q.device).tril() if causal else None
    for step in range(n):
        owner = (r - step) % n  # whose keys and values are here now
        if not (causal and owner > r):  # a block that lies entirely in the future is skipped
            m_b, l_b, o_b = _block(q, kv[0], kv[1], scale, tri if (causal and owner == r) else None)
            if acc is None:
                m_run, l_run, acc = m_b, l_b, o_b
            else:
                m_new = torch.maximum(m_run, m_b)
                a, b = torch.exp(m_run - m_new), torch.exp(m_b - m_new)
                l_run, acc, m_run = a * l_run + b * l_b, a * acc + b * o_b, m_new
        else:
            # Skipped, but kept in the graph with weight zero: every rank's backward pass must run every ring step
            # (the transfer of the gradients is a grouped send + receive that all ranks take part in), whether or
            # not this rank used the block.
            acc = acc + 0.0 * kv.to(acc.dtype).sum()
        if step + 1 < n:
            kv = _RingShift.apply(kv, group)
    return (acc / l_run).to(q.dtype)


class _AllToAll(torch.autograd.Function):
    """Equal-split all-to-all along dimension 0 of a [n, ...] tensor; it is its own transpose, so is its backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        out = torch.empty_like(g)
        dist.all_to_all_single(out, g, group=ctx.group)
        return out, None


def _seq_to_heads(x, group):
    """[B, T/n, H, D] (sequence-sharded) -> [B, T, H/n, D] (head-sharded)."""
    n = dist.get_world_size(group)
    b, tl, h, d = x.shape
    x = x.view(b, tl, n, h // n, d).permute(2, 0, 1, 3, 4).contiguous()  # [n(dest), B, T/n, H/n, D]
    y = _AllToAll.apply(x, group)                                          # [n(source = sequence block), B, T/n, H/n, D]
    return y.permute(1, 0, 2, 3, 4).reshape(b, n * tl, h // n, d)


def _heads_to_seq(x, group):
    """[B, T, H/n, D] (head-sharded) -> [B, T/n, H, D] (sequence-sharded)."""
    n = dist.get_world_size(group)
    b, t, hl, d = x.shape
    x = x.view(b, n, t // n, hl, d).permute(1, 0, 2, 3, 4).contiguous()  # [n(dest = sequence block), B, T/n, H/n, D]
    y = _AllToAll.apply(x, group)                                          # [n(source = head block), B, T/n, H/n, D]
    return y.permute(1, 2, 0, 3, 4).reshape(b, t // n, n * hl, d)


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, causal: bool = False):
    """Attention over a sequence sharded across the group by re-sharding to heads.  ``q``, ``k``, ``v``: [B, T/n, H, D]
    with H divisible by the group size.  Returns [B, T/n, H, D]."""
    n = dist.get_world_size(group)
    if q.shape[2] % n:
        raise ValueError(f"{q.shape[2]} heads cannot be split over {n} ranks")
    qh, kh, vh = (_seq_to_heads(t, group).transpose(1, 2) for t in (q, k, v))  # [B, H/n, T, D]
    o = torch.nn.functional.scaled_dot_product_attention(qh, kh, vh, is_causal=causal)
    return _heads_to_seq(o.transpose(1, 2).contiguous(), group)
