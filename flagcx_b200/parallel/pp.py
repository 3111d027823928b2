"""Pipeline parallelism on the send/recv operations of this library's backend.

The reference offers pipeline parallelism only as "send/recv and ``batch_isend_irecv`` work through the plug-in"
(plugin/torch/flagcx/__init__.py:40-66, flagcx/core/group.cc for the grouped launch).  ``PipelineStage`` is the
schedule on top: rank s of the group owns stage s of the model, micro-batches flow forward as activations and backward
as activation gradients, either all-forward-then-all-backward (``schedule="gpipe"``) or one-forward-one-backward
(``"1f1b"``, which bounds the activations a stage keeps alive to the number of stages after it).

On CUDA tensors every transfer is one launch of this library's device-buffer send/recv kernel (zero-copy when the
receiver's buffer is visible to the sender); on CPU tensors it is the TCP host path.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist


class PipelineStage:
    def __init__(self, module: torch.nn.Module, group=None, activation_shape: Optional[Sequence[int]] = None,
                 dtype: torch.dtype = torch.float32, device=None):
        """``module``: this rank's stage.  ``activation_shape``: shape of the tensor that travels between stages for
        one micro-batch (every boundary carries the same shape here, as in a stack of equal transformer blocks)."""
        self.module, self.group = module, group
        self.n, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.shape, self.dtype = tuple(activation_shape or ()), dtype
        self.device = device or next(module.parameters()).device
        self.first, self.last = self.rank == 0, self.rank == self.n - 1

    def _peer(self, r):
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _exchange(self, send=None, send_to=None, recv_from=None):
        """One grouped launch: optionally send ``send`` to stage ``send_to`` and/or receive an activation-shaped tensor
        from stage ``recv_from``.  A stage that must send one way and receive the other in the same step does both in ONE
        group, so two neighbours that are both about to send can never wait for each other."""
        ops, out = [], None
        if send is not None:
            ops.append(dist.P2POp(dist.isend, send.contiguous(), self._peer(send_to), self.group))
        if recv_from is not None:
            out = torch.empty(self.shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, out, self._peer(recv_from), self.group))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()
        return out

    def _forward(self, x_in, inputs, targets, loss_fn, i):
        x = inputs[i] if self.first else x_in.requires_grad_(True)
        y = self.module(x)
        if self.last:
            y = loss_fn(y, targets[i]) / len(targets)
        return x, y

    def _backward(self, x, y, grad):
        if self.last:
            y.backward()
        else:
            y.backward(grad)
        return None if self.first else x.grad

    def run(self, inputs: Optional[List[torch.Tensor]], targets: Optional[List[torch.Tensor]], loss_fn: Optional[Callable] = None,
            micro_batches: Optional[int] = None, schedule: str = "1f1b"):
        """One optimisation step's forward and backward over all micro-batches; gradients accumulate in the stage's
        parameters.  ``inputs`` is used on the first stage, ``targets`` and ``loss_fn`` on the last; the other ranks pass
        ``micro_batches``.  Returns the mean loss on the last stage, None elsewhere."""
        m = micro_batches or len(inputs if self.first else targets)
        if self.last and targets is None:
            raise ValueError("the last stage needs the targets")
        prev, nxt = (None if self.first else self.rank - 1), (None if self.last else self.rank + 1)
        live, losses = [], []

        def run_forward(i, x_in):
            x, y = self._forward(x_in, inputs, targets, loss_fn, i)
            live.append((x, y))
            if self.last:
                losses.append(y.detach())
            return None if self.last else y.detach()

        if schedule == "gpipe":
            for i in range(m):
                out = run_forward(i, self._exchange(recv_from=prev))
                self._exchange(send=out, send_to=nxt)
            for _ in range(m):
                x, y = live.pop(0)
                dx = self._backward(x, y, self._exchange(recv_from=nxt))
                self._exchange(send=dx, send_to=prev)
        elif schedule == "1f1b":
            warm = min(m, self.n - 1 - self.rank)  # forwards this stage runs before its first backward
            steady = m - warm
            for i in range(warm):
                out = run_forward(i, self._exchange(recv_from=prev))
                self._exchange(send=out, send_to=nxt)
            x_in = self._exchange(recv_from=prev) if steady > 0 else None
            for j in range(steady):
                out = run_forward(warm + j, x_in)
                grad = self._exchange(send=out, send_to=nxt, recv_from=nxt)  # forward out, gradient in: one group
                x, y = live.pop(0)
                dx = self._backward(x, y, grad)
                if j + 1 < steady:
                    x_in = self._exchange(send=dx, send_to=prev, recv_from=prev)  # gradient out, next input in
                else:
                    self._exchange(send=dx, send_to=prev)
            for _ in range(warm):
                x, y = live.pop(0)
                dx = self._backward(x, y, self._exchange(recv_from=nxt))
                self._exchange(send=dx, send_to=prev)
        else:
            raise ValueError(f"unknown schedule {schedule!r}")
        return torch.stack(losses).sum() if self.last else None
