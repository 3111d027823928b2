"""Context-parallel attention (ring and Ulysses) and a 1F1B pipeline over the "flagcx" PyTorch backend in one script:
the strategies a framework builds from the reference's send/recv ring (test/perf/test_sendrecv.cpp:50-51) and
``all_to_all_single`` (plugin/torch/flagcx/src/backend_flagcx.cpp:624-683), here as library functions.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m flagcx_b200.examples.parallel_strategies

Runs on the GPUs when there is one per rank, otherwise on CPU tensors over the TCP host path.  Every rank checks its
slice against whole-sequence attention (every rank builds the same full tensors from one seed) and the pipeline's loss
against the unsplit model; the script exits non-zero on a mismatch."""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist


def main() -> int:
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29534")
    os.environ.setdefault("FLAGCX_SOCKET_IFNAME", "lo")
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    import flagcx  # noqa: F401  registers the backend
    from flagcx_b200.parallel.cp import ring_attention, ulysses_attention
    from flagcx_b200.parallel.pp import PipelineStage
    if use_cuda:
        torch.cuda.set_device(local)
        dev = torch.device("cuda", local)
        dist.init_process_group("cpu:gloo,cuda:flagcx", rank=rank, world_size=world)
    else:
        dev = torch.device("cpu")
        dist.init_process_group("flagcx", rank=rank, world_size=world)
    bad = []

    def check(name, ok):
        if not bool(ok):
            bad.append(name)
        if rank == 0:
            print(f"{name:34s} {'ok' if ok else 'MISMATCH'}", flush=True)

    # ---- long-context attention: 2 x 4 heads, 64 tokens per rank
    B, H, D, tl = 2, 4 * world, 32, 64
    T = tl * world
    g = torch.Generator().manual_seed(7)
    q, k, v = (torch.randn(B, H, T, D, generator=g).to(dev) for _ in range(3))
    mine = slice(rank * tl, (rank + 1) * tl)
    for causal in (False, True):
        ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)[:, :, mine]
        o = ring_attention(q[:, :, mine], k[:, :, mine], v[:, :, mine], causal=causal)
        check(f"ring attention causal={causal}", torch.allclose(o, ref, atol=2e-5, rtol=1e-4))
        o = ulysses_attention(*(t[:, :, mine].transpose(1, 2).contiguous() for t in (q, k, v)), causal=causal)
        check(f"ulysses attention causal={causal}", torch.allclose(o.transpose(1, 2), ref, atol=2e-5, rtol=1e-4))

    # ---- pipeline: one residual MLP block per rank, 8 micro-batches, 1F1B
    width, mb, m = 64, 8, 8
    torch.manual_seed(3)
    blocks = [torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.GELU(), torch.nn.Linear(width, width)).to(dev) for _ in range(world)]
    xs = [torch.randn(mb, width, generator=g).to(dev) for _ in range(m)]
    ys = [torch.randn(mb, width, generator=g).to(dev) for _ in range(m)]
    with torch.no_grad():
        whole = sum(torch.nn.functional.mse_loss(torch.nn.Sequential(*blocks)(x), y) for x, y in zip(xs, ys)) / m
    stage = PipelineStage(blocks[rank], activation_shape=(mb, width), device=dev)
    loss = stage.run(xs if rank == 0 else None, ys if rank == world - 1 else None, torch.nn.functional.mse_loss, micro_batches=m)
    ok = torch.tensor([1.0 if (loss is None or torch.allclose(loss, whole, atol=1e-5)) else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    check("1F1B pipeline loss", ok.item() == 1.0)
    grads = all(p.grad is not None and torch.isfinite(p.grad).all() for p in blocks[rank].parameters())
    check("1F1B pipeline gradients", grads)

    flag = torch.tensor([float(len(bad))], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print("all strategies agree" if flag.item() == 0 else f"MISMATCHES: {bad}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    return 0 if flag.item() == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
