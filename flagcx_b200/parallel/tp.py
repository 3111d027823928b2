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
                 device=None, buffers: int = 2):
        """``max_rows``: tokens of the full (gathered) sequence; ``max_k``: widest gathered activation;
        ``max_n``: widest reduce-scattered output; ``comm_ctas``: CTAs that move data in the all-gather GEMM
        (default: sized per call so that the transfer takes about half the GEMM's time); ``buffers``: workspaces
        the calls rotate through (at least 2; a layer whose backward pass re-reads the rows gathered by its
        forward pass needs one per all-gather of the layer, forward and backward, so that none is overwritten)."""
        self.nat = flagcx_b200.native()
        self.comm, self.n, self.rank = comm, nranks, rank
        self.comm_ctas = comm_ctas
        self.nbuf = max(2, buffers)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        ht = self.nat.heap_tensor
        self.gathered = [ht(comm, [max_rows, max_k], torch.bfloat16) for _ in range(self.nbuf)]
        self.ag_flags = [ht(comm, [max(1, max_rows // 128)], torch.int64).zero_() for _ in range(self.nbuf)]
        self.rs_stage = [ht(comm, [nranks, max_rows // nranks, max_n], torch.bfloat16) for _ in range(2)]
        self.rs_counters = [ht(comm, [max(1, max_rows // nranks // 128) * ((max_n + 255) // 256)], torch.int64).zero_() for _ in range(2)]
        self._wt = {}
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
        par = self.ag_calls % self.nbuf
        epoch = self.ag_calls // self.nbuf + 1
        self.ag_calls += 1
        rows, k = x_local.shape[0] * self.n, x_local.shape[1]
        gathered = self.gathered[par].view(-1)[: rows * k].view(rows, k)
        return self.nat.ag_gemm(self.comm, x_local, gathered, self.ag_flags[par], w, epoch, self._comm_ctas(rows, k, w.shape[0]), self.err)

    def last_gathered(self, x_local: torch.Tensor) -> torch.Tensor:
        """The full [rows, K] matrix that the most recent ``ag_gemm`` call gathered: the remote rows are where the
        kernel put them, the local rows (which the kernel reads in place) are copied in.  Valid until ``buffers``
        further all-gather calls have been made."""
        par = (self.ag_calls - 1) % self.nbuf
        rows, k = x_local.shape[0] * self.n, x_local.shape[1]
        full = self.gathered[par].view(-1)[: rows * k].view(rows, k)
        r0 = self.rank * x_local.shape[0]
        full[r0:r0 + x_local.shape[0]].copy_(x_local)
        return full

    def transposed(self, w: torch.Tensor) -> torch.Tensor:
        """``w.T`` as a contiguous matrix, cached until ``w`` is modified in place (the fused kernels take their
        weight operand K-major; the backward pass needs the other orientation once per optimizer step)."""
        key = (w.data_ptr(), tuple(w.shape))
        hit = self._wt.get(key)
        if hit is None or hit[0] != w._version:
            hit = (w._version, w.t().contiguous())
            self._wt[key] = hit
        return hit[1]

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
        epoch = (self.rs_calls >> 1) + 1  # two staging areas suffice: a result is read out before the kernel ends
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
               dw       = dy.T @ all_gather(x)     tcgen05 GEMM (both operands read transposed in place, K = tokens
                                                   split across CTAs) on the rows gathered by the forward kernel
    """

    @staticmethod
    def forward(ctx, x_local, w, tp):
        y = tp.ag_gemm(x_local, w)
        full = tp.last_gathered(x_local)
        if tp.nbuf < 4:
            full = full.clone()  # too few workspaces to keep the gathered rows until the backward pass
        ctx.save_for_backward(full, w)
        ctx.tp = tp
        return y

    @staticmethod
    def backward(ctx, dy):
        from flagcx_b200.ops import gemm
        full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        # The weight gradient first: it reads the rows gathered by the forward pass from a workspace that the
        # peers will push into again a few calls from now, and they cannot get there before this rank has
        # contributed to the reduce-scatter below.
        dw = gemm(dy, full, True, True)              # [N, rows] @ [rows, K]
        dx_local = tp.gemm_rs(dy, tp.transposed(w))  # [rows, N] @ [N, K] -> rows/n x K
        return dx_local, dw, None


class _RowParallel(torch.autograd.Function):
    """z_local = reduce_scatter(a @ w.T) with row-sharded weight (K sharded) and sequence-parallel output.

    forward  : one fused GEMM -> reduce-scatter kernel
    backward : da = all_gather(dz_local) @ w       one fused all-gather -> GEMM kernel
               dw = all_gather(dz_local).T @ a     tcgen05 GEMM on the rows gathered by that kernel
    """

    @staticmethod
    def forward(ctx, a, w, tp):
        ctx.save_for_backward(a, w)
        ctx.tp = tp
        return tp.gemm_rs(a, w)

    @staticmethod
    def backward(ctx, dz_local):
        from flagcx_b200.ops import gemm
        a, w = ctx.saved_tensors
        tp = ctx.tp
        dz_local = dz_local.contiguous()
        da = tp.ag_gemm(dz_local, tp.transposed(w))  # [rows, N] @ [N, K_local]
        full = tp.last_gathered(dz_local)
        dw = gemm(full, a, True, True)               # [N, rows] @ [rows, K_local]
        return da, dw, None


def column_parallel_linear(x_local: torch.Tensor, w: torch.Tensor, tp: TensorParallelContext) -> torch.Tensor:
    """Differentiable ``all_gather(x_local) @ w.T`` on the fused kernels (entry of a tensor-parallel block)."""
    return _ColumnParallel.apply(x_local, w, tp)


def row_parallel_linear(a: torch.Tensor, w: torch.Tensor, tp: TensorParallelContext) -> torch.Tensor:
    """Differentiable ``reduce_scatter(a @ w.T)`` on the fused kernels (exit of a tensor-parallel block)."""
    return _RowParallel.apply(a, w, tp)
