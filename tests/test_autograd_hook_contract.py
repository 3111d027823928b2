"""The PyTorch behaviour the data-parallel trainer's bucket bookkeeping rests on, pinned on CPU: a parameter whose
backward function returns None (because the gradient was written straight into ``.grad``) still runs its accumulation
node once per backward pass, and with it the post-accumulate hook - exactly once, also when the parameter is used
twice and only one use returns a gradient through autograd."""
import torch


class _WritesGradItself(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        ctx.param = w
        return x * w

    @staticmethod
    def backward(ctx, g):
        x, w = ctx.saved_tensors
        ctx.param.grad.add_(g * x)  # what the fused kernels do on the GPU
        return g * w, None


def test_hook_fires_once_for_a_gradient_returned_as_none():
    w = torch.full((3,), 2.0, requires_grad=True)
    w.grad = torch.zeros(3)
    x = torch.ones(3, requires_grad=True)
    fired = []
    w.register_post_accumulate_grad_hook(lambda p: fired.append(p.grad.clone()))
    for step in range(2):
        _WritesGradItself.apply(x, w).sum().backward()
        assert len(fired) == step + 1
        assert torch.equal(fired[-1], torch.full((3,), float(step + 1)))  # the direct write is visible to the hook


def test_hook_fires_once_for_a_tied_parameter_with_one_direct_use():
    w = torch.full((3,), 2.0, requires_grad=True)
    w.grad = torch.zeros(3)
    x = torch.ones(3, requires_grad=True)
    fired = []
    w.register_post_accumulate_grad_hook(lambda p: fired.append(p.grad.clone()))
    (_WritesGradItself.apply(x, w) + 3.0 * w).sum().backward()  # one direct use, one ordinary use
    assert len(fired) == 1
    assert torch.equal(fired[0], torch.full((3,), 4.0))  # 1 (direct) + 3 (autograd), both there when the hook runs
