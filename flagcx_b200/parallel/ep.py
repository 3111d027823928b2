"""Expert-parallel mixture-of-experts layer (one or several experts per rank, top-k routing).

Fused path (``ExpertParallelContext.forward``), five launches and no host
round trip:

1. ``moe_dispatch``  one cooperative kernel: per-expert counts, count-matrix
   exchange through the symmetric heap, token push over NVLink into the
   expert's segment of its rank's input buffer; the received row counts
   (one per local expert) stay on the device.  Steps 2-4 run once per
   local expert.
2. up/gate GEMM      tcgen05 GEMM whose row count is read on the device.
3. ``silu_mul``
4. down GEMM         tcgen05 GEMM in ROWMAP mode: the epilogue stores every
   output row straight into the combine buffer of the token's home rank
   (the combine all-to-all never exists as a separate step).
5. ``moe_combine``   waits for every expert's GEMM CTAs, then the weighted
   sum over the k choices.

Unfused path (``unfused_forward``): what a FlagCX user writes today:
``flagcxAlltoAllv`` needs host-side counts (flagcx/include/flagcx.h:397), so
the router output is copied to the host, counts are exchanged, tokens are
permuted, sent, multiplied with library GEMMs, sent back and un-permuted.
"""
from __future__ import annotations

import torch

import flagcx_b200


def moe_reference(x, topk_idx, topk_w, w_gate_up, w_down, expert: int | None = None):
    """fp32 math of the layer for ONE set of expert weights per expert id.

    ``w_gate_up``: list (one per expert) of [2F, H]; ``w_down``: list of [H, F].
    Returns fp32 [T, H].  Used by tests as the oracle.
    """
    T, H = x.shape
    out = torch.zeros(T, H, dtype=torch.float32, device=x.device)
    xf = x.float()
    for e in range(len(w_gate_up)):
        if expert is not None and e != expert:
            continue
        F = w_down[e].shape[1]
        for k in range(topk_idx.shape[1]):
            sel = (topk_idx[:, k] == e).nonzero().flatten()
            if sel.numel() == 0:
                continue
            gu = (xf[sel] @ w_gate_up[e].float().t()).bfloat16().float()
            h = (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]).bfloat16().float()
            y = (h @ w_down[e].float().t()).bfloat16().float()
            out[sel] += topk_w[sel, k].unsqueeze(1).float() * y
    return out


class ExpertParallelContext:
    def __init__(self, comm: int, nranks: int, rank: int, tokens: int, hidden: int, ffn: int, topk: int = 2,
                 capacity_factor: float = 1.25, dispatch_ctas: int = 64, device=None, experts_per_rank: int = 1):
        """``tokens``: tokens per rank; ``capacity_factor`` x the balanced load bounds the rows an expert accepts;
        ``experts_per_rank``: expert e lives on rank ``e // experts_per_rank`` (at most 64 experts in all)."""
        self.nat = flagcx_b200.native()
        self.comm, self.n, self.rank = comm, nranks, rank
        self.T, self.H, self.F, self.K = tokens, hidden, ffn, topk
        self.L = experts_per_rank
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.dispatch_ctas = dispatch_ctas
        total = nranks * tokens * topk          # routed (token, choice) entries of the whole job
        balanced = -(-total // (nranks * self.L))  # ... spread evenly over the experts
        cap_l = min(total, int(balanced * capacity_factor)) if nranks * self.L > 1 else balanced
        self.cap_l = (cap_l + 127) // 128 * 128  # rows of one local expert's segment
        self.cap = self.cap_l * self.L
        ht = self.nat.heap_tensor
        i32, i64, bf = torch.int32, torch.int64, torch.bfloat16
        self.count_mat = [ht(comm, [nranks * nranks * self.L], i32).zero_() for _ in range(2)]
        self.count_flags = [ht(comm, [8], i64).zero_() for _ in range(2)]
        self.recv = [ht(comm, [self.cap, hidden], bf) for _ in range(2)]
        self.info = [ht(comm, [self.cap, 4], i32).zero_() for _ in range(2)]
        self.disp_done = [ht(comm, [8], i64).zero_() for _ in range(2)]
        self.combine = [ht(comm, [tokens * topk, hidden], bf) for _ in range(2)]
        self.comb_done = [ht(comm, [2], i64).zero_() for _ in range(2)]
        dev = self.device
        self.slot = torch.zeros(tokens * topk, dtype=i32, device=dev)
        self.local_counts = torch.zeros(nranks * self.L, dtype=i32, device=dev)
        self.recv_total = torch.zeros(self.L, dtype=i32, device=dev)  # rows received per local expert
        self.err = torch.zeros(1, dtype=i32, device=dev)
        self.gu = torch.empty(self.cap, 2 * ffn, dtype=bf, device=dev)
        self.h = torch.empty(self.cap, ffn, dtype=bf, device=dev)
        self.calls = 0
        self.comb_want = [0, 0]
        torch.cuda.synchronize()
        if nranks > 1:  # nobody may write into a workspace that its owner has not cleared yet
            t = torch.zeros(1, device=dev)
            self.nat.comm_all_reduce(comm, t, t, 0, 1.0)
            torch.cuda.synchronize()

    def forward(self, x, topk_idx, topk_w, w_gate_up, w_down, out=None):
        """x bf16 [T, H]; topk_idx int32 [T, K] (global expert ids); topk_w fp32 [T, K]; w_gate_up bf16 [2F, H] and
        w_down bf16 [H, F] of THIS rank's expert, or lists / stacked tensors of ``experts_per_rank`` of them.
        Returns bf16 [T, H]."""
        nat, par = self.nat, self.calls & 1
        epoch = (self.calls >> 1) + 1
        self.calls += 1
        if out is None:
            out = torch.empty_like(x)
        if self.L == 1 and torch.is_tensor(w_gate_up) and w_gate_up.dim() == 2:
            w_gate_up, w_down = [w_gate_up], [w_down]
        assert len(w_gate_up) == self.L and len(w_down) == self.L, "one weight pair per local expert"
        nat.moe_dispatch(self.comm, x, topk_idx, self.count_mat[par], self.count_flags[par], self.recv[par], self.info[par],
                         self.disp_done[par], epoch, self.slot, self.local_counts, self.recv_total, self.err, self.dispatch_ctas,
                         self.L)
        for l in range(self.L):  # every local expert works on its own segment, sized on the device by its row count
            seg = slice(l * self.cap_l, (l + 1) * self.cap_l)
            rows = self.recv_total[l:l + 1]
            nat.gemm_dyn_m(self.recv[par][seg], w_gate_up[l], self.gu[seg], rows, self.err)
            nat.silu_mul(self.gu[seg], self.h[seg], rows)
            grid = nat.gemm_rowmap(self.comm, self.h[seg], w_down[l], rows, self.info[par][seg], self.combine[par], self.comb_done[par],
                                   self.K, self.err)
            self.comb_want[par] += grid * self.n  # every rank launches the same grids
        nat.moe_combine(self.comm, self.combine[par], topk_w, out, self.comb_done[par], self.comb_want[par], self.err)
        return out

    def check(self):
        """Raise if a kernel gave up on a wait or dropped tokens (call after a synchronize)."""
        code = int(self.err.item())
        if code == 1:
            raise RuntimeError("a MoE kernel gave up waiting (peer missing or too slow)")
        if code == 2:
            raise RuntimeError("an expert received more tokens than its capacity; raise capacity_factor")

    # ---- the unfused baseline on the same library: host counts + all-to-all-v + library GEMMs
    def unfused_forward(self, x, topk_idx, topk_w, w_gate_up, w_down):
        n, K, H = self.n, self.K, self.H
        flat = topk_idx.flatten().long()
        order = torch.argsort(flat, stable=True)
        send = x[order // K]
        scounts_dev = torch.bincount(flat, minlength=n).to(torch.int64)
        rcounts_dev = torch.empty_like(scounts_dev)
        if n > 1:
            self.nat.comm_all_to_all(self.comm, scounts_dev, rcounts_dev)
        else:
            rcounts_dev.copy_(scounts_dev)
        scounts = scounts_dev.cpu().tolist()  # the host round trip the fused path avoids
        rcounts = rcounts_dev.cpu().tolist()
        sdis = [sum(scounts[:i]) for i in range(n)]
        rdis = [sum(rcounts[:i]) for i in range(n)]
        rows = sum(rcounts)
        recv = torch.empty(rows, H, dtype=x.dtype, device=x.device)
        if n > 1:
            self.nat.comm_all_to_all_v(self.comm, send, [c * H for c in scounts], [d * H for d in sdis], recv,
                                       [c * H for c in rcounts], [d * H for d in rdis])
        else:
            recv.copy_(send)
        gu = recv @ w_gate_up.t()
        F = w_down.shape[1]
        h = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
        y = h @ w_down.t()
        back = torch.empty_like(send)
        if n > 1:
            self.nat.comm_all_to_all_v(self.comm, y, [c * H for c in rcounts], [d * H for d in rdis], back,
                                       [c * H for c in scounts], [d * H for d in sdis])
        else:
            back.copy_(y)
        ret = torch.empty_like(back)
        ret[order] = back
        ret = ret.view(self.T, K, H)
        return (ret.float() * topk_w.unsqueeze(2)).sum(1).to(x.dtype)
