"""Data-parallel training engine.

One process per GPU.  Parameters, gradients and optimizer state live in flat
buffers; gradients are all-reduced in ~25 MB buckets as soon as the backward
pass has finished writing a bucket, on a side stream, by the library's own
NVLink kernels (average fused into the reduction); one fused AdamW kernel
updates fp32 master weights and refreshes the bf16 parameters.  The whole
step (forward, backward, bucket all-reduces, optimizer) is captured once in a
CUDA graph and replayed, which removes the per-kernel launch cost of an
eager step.  The collective kernels keep their sequence numbers in device
memory, which is what makes them replayable.

The engine owns a communicator of its own (split off the process group's), for
two reasons: a communicator serves one stream at a time, and this one launches
on the engine's side stream while the process group's may be busy with the
caller's collectives; and its heap is sized for the gradients.  Gradients and
parameters live in that communicator's symmetric heap, so each bucket is
reduced in place through the zero-copy kernel (in-switch reduction, nothing
staged) with a small CTA budget (``FLAGCX_DDP_CTAS``, default 16) that leaves
the SMs to the backward pass it overlaps.

This is the framework's counterpart of running ``DistributedDataParallel``
over the reference's process-group backend (plugin/torch/flagcx/src/backend_flagcx.cpp:505-532);
stock ``DistributedDataParallel`` over this library's backend works as well
(``bench.py --impl ours-c10d`` and the c10d backend tests run it).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

import flagcx_b200
from flagcx_b200.models.gpt2 import flatten_parameters
from flagcx_b200.ops import fused_adamw_step


@dataclass
class _Bucket:
    start: int
    end: int
    nparams: int
    pending: int = 0


class DataParallelTrainer:
    def __init__(self, model: torch.nn.Module, *, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, bucket_mb: float = 25.0, group=None, use_graph: bool = True,
                 device: Optional[torch.device] = None):
        self.model = model
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.native = flagcx_b200.native()
        self.comm = 0
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.step_no = 0
        self.launches_per_step = 0
        self.step_dev = torch.zeros(1, dtype=torch.int32, device=self.device)

        # ---- flat buffers (in the engine's own symmetric heap when there is anything to exchange)
        n = sum((p.numel() + 127) // 128 * 128 for p in model.parameters())
        if self.world > 1:
            parent = flagcx_b200.get_comm_handle(group, self.device)
            heap_bytes = 2 * (2 * n) + (64 << 20)
            self.comm = self.native.comm_split(parent, 0, self.rank, stage_bytes=64 << 20, user_bytes=heap_bytes)
            self.cta_budget = int(os.environ.get("FLAGCX_DDP_CTAS", "16"))
            self.native.comm_set_cta_budget(self.comm, self.cta_budget)
            # under a small CTA budget the switch's own reduction is worth its extra bytes even with two ranks
            self.native.comm_set_zc_multicast(self.comm, int(os.environ.get("FLAGCX_DDP_ZC_MC", "2")))
            buf = self.native.heap_tensor(self.comm, [n], torch.bfloat16)
            self.flat_params, self.specs = flatten_parameters(model, torch.bfloat16, self.device, buffer=buf)
            self.flat_grads = self.native.heap_tensor(self.comm, [n], torch.bfloat16)
            self.flat_grads.zero_()
        else:
            self.flat_params, self.specs = flatten_parameters(model, torch.bfloat16, self.device)
            self.flat_grads = torch.zeros(n, dtype=torch.bfloat16, device=self.device)
        self.master = self.flat_params.float()
        self.m = torch.zeros_like(self.master)
        self.v = torch.zeros_like(self.master)
        params = list(model.parameters())
        for (name, off, cnt), p in zip(self.specs, params):
            p.grad = self.flat_grads[off:off + cnt].view(p.shape)
        if self.world > 1:
            # all ranks start from rank 0's weights
            self.native.comm_broadcast(self.comm, self.flat_params, 0)
            self.master.copy_(self.flat_params)

        # ---- buckets, built from the end of the buffer (gradients arrive roughly in reverse order)
        self.buckets: List[_Bucket] = []
        self.bucket_of = {}
        cap = int(bucket_mb * (1 << 20) / 2)
        end = n
        cur_params = []
        for i in range(len(self.specs) - 1, -1, -1):
            name, off, cnt = self.specs[i]
            cur_params.append(i)
            if end - off >= cap or i == 0:
                b = _Bucket(off, end, len(cur_params))
                for j in cur_params:
                    self.bucket_of[j] = len(self.buckets)
                self.buckets.append(b)
                end = off
                cur_params = []
        for i, p in enumerate(params):
            p.register_post_accumulate_grad_hook(self._make_hook(i))
        # Gradients that the fused backward kernels add straight into the flat buffer come back from the backward
        # functions as None.  Autograd still runs the parameter's accumulation node then (with nothing to add) and
        # with it the post-accumulate hook above, after the kernel that wrote the gradient has been queued: the
        # bucket bookkeeping needs no second signal (a second one would close buckets early).
        self.direct_grads = 0
        if os.environ.get("FLAGCX_DDP_DIRECT_GRAD", "1") != "0" and hasattr(model, "direct_grad_parameters"):
            from flagcx_b200.ops import enable_direct_grad
            for p, _counted in model.direct_grad_parameters():
                enable_direct_grad(p)
                self.direct_grads += 1
        # Side stream: a bucket's all-reduce and its share of the optimizer step run here, beside the rest of
        # the backward pass.  A parameter whose gradient is complete is no longer read by this step's backward
        # (the tied embedding sits in the bucket that closes last), so updating it early is safe.
        self.side_stream = torch.cuda.Stream(device=self.device, priority=-1)
        self.comm_stream = self.side_stream
        self.ready_event = torch.cuda.Event()
        self.done_event = torch.cuda.Event()
        self.pre_tail_event = torch.cuda.Event()
        self.split_tail = os.environ.get("FLAGCX_DDP_SPLIT_TAIL", "1") != "0"
        # Measured on one B200: the per-bucket optimizer beside the backward pass gains nothing (26.7 against
        # 26.5 ms per step; the AdamW blocks and the GEMMs compete for the same SMs), so it is off by default.
        self.overlap_optimizer = os.environ.get("FLAGCX_DDP_OVERLAP_OPT", "0") != "0"
        # the bucket that closes last has nothing left to overlap with: it may take more of the GPU
        self.tail_ctas = int(os.environ.get("FLAGCX_DDP_TAIL_CTAS", "64"))
        self._budget_now = getattr(self, "cta_budget", 0)

        self._loss_host = None
        self._loss_pending = None
        self.snapshot_grads = False
        self.grad_snapshot = None
        self.use_graph = use_graph
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_tokens = None
        self.static_targets = None
        self.static_loss = None
        self.eager_steps = 0

    # ---- gradient bucket hooks
    def _make_hook(self, idx):
        def hook(_param):
            b = self.buckets[self.bucket_of[idx]]
            b.pending -= 1
            if b.pending == 0:
                self._bucket_ready(b)
        return hook

    def _adamw(self, lo: int, hi: int):
        fused_adamw_step(self.master[lo:hi], self.flat_params[lo:hi], self.flat_grads[lo:hi], self.m[lo:hi], self.v[lo:hi],
                         lr=self.lr, betas=self.betas, eps=self.eps, weight_decay=self.wd, step=self.step_no + 1, zero_grad=True,
                         step_dev=self.step_dev)

    def _bucket_ready(self, b: _Bucket):
        early_opt = self.overlap_optimizer and not self.snapshot_grads
        if self.world == 1 and not early_opt:
            return
        cur = torch.cuda.current_stream(self.device)
        self.ready_event.record(cur)
        self.side_stream.wait_event(self.ready_event)
        with torch.cuda.stream(self.side_stream):
            if self.world > 1:
                if b is self.buckets[-1]:
                    self.pre_tail_event.record(self.side_stream)  # every earlier bucket is reduced at this point
                want = self.tail_ctas if b is self.buckets[-1] else self.cta_budget
                if want != self._budget_now:
                    self.native.comm_set_cta_budget(self.comm, want)
                    self._budget_now = want
                g = self.flat_grads[b.start:b.end]
                self.native.comm_all_reduce(self.comm, g, g, 4, 1.0)  # 4 = average
                self.launches_per_step += 1
            if early_opt:
                self._adamw(b.start, b.end)
                self.launches_per_step += 1

    # ---- one optimisation step on tensors that already live on the device
    def _step_device(self, tokens, targets):
        for b in self.buckets:
            b.pending = b.nparams
        self.launches_per_step = 0
        early_opt = self.overlap_optimizer and not self.snapshot_grads
        self.step_dev.add_(1)  # before the backward pass: every bucket's optimizer share reads it
        loss = self.model(tokens, targets)
        loss.backward()
        if self.world > 1 or early_opt:
            self.done_event.record(self.side_stream)
            if self.world > 1 and not early_opt and not self.snapshot_grads and self.split_tail:
                self._finish_step_split()
                return loss.detach()
            torch.cuda.current_stream(self.device).wait_event(self.done_event)
        if self.snapshot_grads:  # for tests: the averaged gradients as the optimizer is about to see them
            self.grad_snapshot = self.flat_grads.clone()
        if not early_opt:
            self._adamw(0, self.flat_grads.numel())
            self.launches_per_step += 1
        return loss.detach()

    def _finish_step_split(self):
        """More than one rank: the all-reduce of the bucket that closes last (the tied embedding, the largest
        tensor of the model) has no backward work left to hide behind, so the optimizer hides it instead: the
        update of everything outside that bucket runs while the bucket is still being reduced."""
        cur = torch.cuda.current_stream(self.device)
        tail = self.buckets[-1]
        cur.wait_event(self.pre_tail_event)
        n = self.flat_grads.numel()
        if tail.end < n:
            self._adamw(tail.end, n)
            self.launches_per_step += 1
        cur.wait_event(self.done_event)
        self._adamw(tail.start, tail.end)
        self.launches_per_step += 1

    def _capture(self, tokens, targets):
        self.static_tokens = tokens.clone()
        self.static_targets = targets.clone()
        self.graph = torch.cuda.CUDAGraph()
        # the AdamW step counter lives on the device, so replays stay exact
        with torch.cuda.graph(self.graph):
            self.static_loss = self._step_device(self.static_tokens, self.static_targets)

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """One training step.  ``tokens``/``targets`` may be pinned host tensors
        (they are copied to the device on the current stream) or device tensors.
        Returns the loss as a device scalar; call ``.item()`` to read it back."""
        if tokens.device.type != "cuda":
            tokens = tokens.to(self.device, non_blocking=True)
            targets = targets.to(self.device, non_blocking=True)
        if not self.use_graph:
            loss = self._step_device(tokens, targets)
        elif self.graph is None and self.eager_steps < 2:
            # warm-up on a side stream, as graph capture requires
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(s):
                loss = self._step_device(tokens, targets)
            torch.cuda.current_stream(self.device).wait_stream(s)
            self.eager_steps += 1
        else:
            if self.graph is None:
                self._capture(tokens, targets)
            self.static_tokens.copy_(tokens, non_blocking=True)
            self.static_targets.copy_(targets, non_blocking=True)
            self.graph.replay()
            loss = self.static_loss
        self.step_no += 1
        return loss

    # ---- checkpoint / resume (the reference, a communication library, holds no training state and has no counterpart)
    def state_dict(self) -> dict:
        """Everything the next step depends on, as CPU tensors: fp32 master weights, both AdamW moments, the step
        count, and the layout of the flat buffers (name, offset, count per parameter) to check a resume against."""
        torch.cuda.synchronize(self.device)
        return {"master": self.master.detach().cpu(), "m": self.m.detach().cpu(), "v": self.v.detach().cpu(),
                "step": int(self.step_no), "specs": [tuple(s) for s in self.specs],
                "hyper": {"lr": self.lr, "betas": tuple(self.betas), "eps": self.eps, "weight_decay": self.wd}}

    def load_state_dict(self, state: dict) -> None:
        """Resume from ``state_dict()`` of a trainer over the same model (same parameter layout).  Every rank loads the
        same state; the bf16 working weights are re-derived from the fp32 master copy."""
        if [tuple(s) for s in state["specs"]] != [tuple(s) for s in self.specs]:
            raise ValueError("the checkpoint was written for a different parameter layout")
        torch.cuda.synchronize(self.device)
        self.master.copy_(state["master"])
        self.m.copy_(state["m"])
        self.v.copy_(state["v"])
        self.flat_params.copy_(self.master)  # fp32 -> bf16
        self.flat_grads.zero_()
        self.step_no = int(state["step"])
        self.step_dev.fill_(self.step_no)
        torch.cuda.synchronize(self.device)

    def step_pipelined(self, tokens: torch.Tensor, targets: torch.Tensor):
        """``step`` for a training loop that reads every loss on the host without stalling the GPU: the step is
        queued, its loss is copied into pinned host memory behind it, and the call returns the loss of the PREVIOUS
        step as a float (None on the first call) - by then that copy has long finished, so the host is back at
        once to queue the next step while this one runs.  ``drain()`` returns the loss of the last step."""
        if self._loss_host is None:
            self._loss_host = [torch.zeros(1, dtype=torch.float32).pin_memory() for _ in range(2)]
            self._loss_event = [torch.cuda.Event(), torch.cuda.Event()]
            self._loss_pending = None
        loss = self.step(tokens, targets)  # queued; the host does not wait for it
        slot = 0 if self._loss_pending == 1 else 1
        self._loss_host[slot].copy_(loss.detach().reshape(1).float(), non_blocking=True)
        self._loss_event[slot].record(torch.cuda.current_stream(self.device))
        prev = self.drain()  # the step before this one: finished (or about to) while this one is already queued
        self._loss_pending = slot
        return prev

    def drain(self):
        """Loss of the most recent ``step_pipelined`` call that has not been handed out yet (None if there is none)."""
        if self._loss_host is None or self._loss_pending is None:
            return None
        slot, self._loss_pending = self._loss_pending, None
        self._loss_event[slot].synchronize()
        return float(self._loss_host[slot][0])

    def kernels_per_step(self) -> int:
        """Launches of this framework's own kernels in one step: per layer 2
        fused LayerNorm forward, 2 x 2 backward (dx; parameter gradients with
        their reduction), bias-GELU forward + 2 backward (dx; bias gradient);
        the tcgen05 GEMMs of the projections and the LM head; the final
        LayerNorm (1 + 2), the loss kernel, and per bucket one all-reduce
        kernel (more than one rank) and one AdamW kernel (one AdamW kernel in
        all when the optimizer is not overlapped)."""
        L = len(getattr(self.model, "blocks", []))
        own = L * (2 + 4 + 1 + 2) + (1 + 2) + 1
        if os.environ.get("FLAGCX_MODEL_GEMM", "own") != "library" and os.environ.get("FLAGCX_MODEL_FUSED_GELU", "1") != "0":
            own -= L  # the GELU of the forward pass runs in the epilogue of the up-projection GEMM
        if os.environ.get("FLAGCX_MODEL_GEMM", "own") != "library":
            # tcgen05 GEMMs: four projections per layer and the LM head, each forward + input gradient + weight
            # gradient; the three biased projections' bias gradients take one column-sum kernel each
            own += L * (4 * 3 + 3) + 3
        nb = len(self.buckets)
        adamw = nb if self.overlap_optimizer else (2 if self.world > 1 and self.split_tail else 1)
        return own + (nb if self.world > 1 else 0) + adamw
