"""Tensor-parallel (sequence-parallel) building blocks on the fused tcgen05
kernels: all-gather -> GEMM on entry of a sharded block and GEMM ->
reduce-scatter on exit, each ONE kernel that moves the data over NVLink while
the tensor cores work (csrc/torch/gemm_sm100.cu).

``TensorParallelContext`` owns the symmetric-heap workspaces (gathered
activations, partial-tile staging, flags and counters), double-buffered by
call parity so that a rank that runs one call ahead of a peer never touches
memory the peer still reads.

The unfused equivalents (library all-gather / reduce-scatter followed by a
library GEMM) are what a FlagCX user runs today; ``unfused_ag_gemm`` and
``unfused_gemm_rs`` implement exactly that on this library's collectives for
comparison.
"""
from __future__ import annotations

import torch

import flagcx_b200


class TensorParallelContext:
    def __init__(self, comm: int, nranks: int, rank: int, max_rows: int, max_k: int, max_n: int, comm_ctas: int | None = None,
                 device=None):
        """``max_rows``: tokens of the full (gathered) sequence; ``max_k``: widest gathered activation;
        ``max_n``: widest reduce-scattered output; ``comm_ctas``: CTAs that move data in the all-gather GEMM
        (default: sized per call so that the transfer takes about half the GEMM's time)."""
        self.nat = flagcx_b200.native()
        self.comm, self.n, self.rank = comm, nranks, rank
        self.comm_ctas = comm_ctas
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        ht = self.nat.heap_tensor
        self.gathered = [ht(comm, [max_rows, max_k], torch.bfloat16) for _ in range(2)]
        self.ag_flags = [ht(comm, [max(1, max_rows // 128)], torch.int64).zero_() for _ in range(2)]
        self.rs_stage = [ht(comm, [nranks, max_rows // nranks, max_n], torch.bfloat16) for _ in range(2)]
        self.rs_counters = [ht(comm, [max(1, max_rows // nranks // 128) * ((max_n + 255) // 256)], torch.int64).zero_() for _ in range(2)]
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.ag_calls = 0
        self.rs_calls = 0
        torch.cuda.synchronize()
        # nobody may push into a workspace that its owner has not cleared yet
        if nranks > 1:
            t = torch.zeros(1, device=self.device)
            self.nat.comm_all_reduce(comm, t, t, 0, 1.0)
            torch.cuda.synchronize()

    def ag_gemm(self, x_local: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``all_gather(x_local) @ w.T``; x_local [rows/n, K], w [N, K] -> [rows, N]."""
        par = self.ag_calls & 1
        epoch = (self.ag_calls >> 1) + 1
        self.ag_calls += 1
        rows, k = x_local.shape[0] * self.n, x_local.shape[1]
        gathered = self.gathered[par].view(-1)[: rows * k].view(rows, k)
        return self.nat.ag_gemm(self.comm, x_local, gathered, self.ag_flags[par], w, epoch, self._comm_ctas(rows, k, w.shape[0]), self.err)

    def _comm_ctas(self, rows: int, k: int, n_out: int) -> int:
        """One data-moving CTA sustains about 40 GB/s over NVLink and 16 saturate the link; use as few as hide the
        transfer of the remote rows behind the GEMM (estimated at 1.4 PFLOP/s)."""
        if self.comm_ctas is not None:
            return self.comm_ctas
        if self.n == 1:
            return 1
        remote_bytes = (self.n - 1) * (rows // self.n) * k * 2
        gemm_s = 2.0 * rows * k * n_out / 1.4e15
        want = remote_bytes / (0.5 * gemm_s) / 40e9
        return int(min(20, max(2, -(-want // 1))))

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """``reduce_scatter(a @ w.T)`` over rows; a [rows, K], w [N, K] -> [rows/n, N]."""
        par = self.rs_calls & 1
        epoch = (self.rs_calls >> 1) + 1
        self.rs_calls += 1
        rows, n_out = a.shape[0], w.shape[0]
        stage = self.rs_stage[par].view(-1)[: rows * n_out]
        return self.nat.gemm_rs(self.comm, a, w, stage, self.rs_counters[par], epoch, self.err)

    def check(self):
        """Raise if a kernel of this context gave up on a wait (call after a synchronize)."""
        if int(self.err.item()) != 0:
            raise RuntimeError("a fused GEMM kernel gave up waiting (peer missing or too slow)")

    # ---- the unfused baselines on the same library
    def unfused_ag_gemm(self, x_local, w):
        full = torch.empty(x_local.shape[0] * self.n, x_local.shape[1], dtype=x_local.dtype, device=x_local.device)
        if self.n > 1:
            self.nat.comm_all_gather(self.comm, x_local, full)
        else:
            full.copy_(x_local)
        return full @ w.t()

    def unfused_gemm_rs(self, a, w):
        part = a @ w.t()
        if self.n == 1:
            return part
        out = torch.empty(a.shape[0] // self.n, w.shape[0], dtype=a.dtype, device=a.device)
        self.nat.comm_reduce_scatter(self.comm, part, out, 0)
        return out


class _ColumnParallel(torch.autograd.Function):
    """y = all_gather(x_local) @ w.T with sequence-parallel input (rows sharded) and column-sharded weight.

    forward  : one fused all-gather -> GEMM kernel
    backward : dx_local = reduce_scatter(dy @ w)   one fused GEMM -> reduce-scatter kernel
               dw       = dy.T @ all_gather(x)     library GEMM on the rows gathered by the forward kernel
    """

    @staticmethod
    def forward(ctx, x_local, w, tp):
        par = tp.ag_calls & 1
        y = tp.ag_gemm(x_local, w)
        rows, k = x_local.shape[0] * tp.n, x_local.shape[1]
        # the forward kernel left every rank's rows in the workspace (the local block is only read in place)
        gathered = tp.gathered[par].view(-1)[: rows * k].view(rows, k)
        full = gathered.clone()
        r0 = tp.rank * x_local.shape[0]
        full[r0:r0 + x_local.shape[0]] = x_local
        ctx.save_for_backward(full, w)
        ctx.tp = tp
        return y

    @staticmethod
    def backward(ctx, dy):
        full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        dx_local = tp.gemm_rs(dy, w.t().contiguous())  # [rows, N] @ [N, K] -> rows/n x K
        dw = dy.t() @ full
        return dx_local, dw, None


class _RowParallel(torch.autograd.Function):
    """z_local = reduce_scatter(a @ w.T) with row-sharded weight (K sharded) and sequence-parallel output.

    forward  : one fused GEMM -> reduce-scatter kernel
    backward : da = all_gather(dz_local) @ w       one fused all-gather -> GEMM kernel
               dw = all_gather(dz_local).T @ a     library GEMM on the rows gathered by that kernel
    """

    @staticmethod
    def forward(ctx, a, w, tp):
        ctx.save_for_backward(a, w)
        ctx.tp = tp
        return tp.gemm_rs(a, w)

    @staticmethod
    def backward(ctx, dz_local):
        a, w = ctx.saved_tensors
        tp = ctx.tp
        dz_local = dz_local.contiguous()
        par = tp.ag_calls & 1
        da = tp.ag_gemm(dz_local, w.t().contiguous())  # [rows, N] @ [N, K_local]
        rows, ncols = dz_local.shape[0] * tp.n, dz_local.shape[1]
        gathered = tp.gathered[par].view(-1)[: rows * ncols].view(rows, ncols)
        full = gathered.clone()
        r0 = tp.rank * dz_local.shape[0]
        full[r0:r0 + dz_local.shape[0]] = dz_local
        dw = full.t() @ a
        return da, dw, None


def column_parallel_linear(x_local: torch.Tensor, w: torch.Tensor, tp: TensorParallelContext) -> torch.Tensor:
    """Differentiable ``all_gather(x_local) @ w.T`` on the fused kernels (entry of a tensor-parallel block)."""
    return _ColumnParallel.apply(x_local, w, tp)


def row_parallel_linear(a: torch.Tensor, w: torch.Tensor, tp: TensorParallelContext) -> torch.Tensor:
    """Differentiable ``reduce_scatter(a @ w.T)`` on the fused kernels (exit of a tensor-parallel block)."""
    return _RowParallel.apply(a, w, tp)
