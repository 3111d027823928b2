"""Every operation of the "flagcx" PyTorch backend in one script, the counterpart of the reference's API example
(plugin/torch/example/example.py): collectives, list and tensor forms, uneven all-to-all, coalescing, batched
point-to-point (a pipeline-parallel hand-off), async work objects.

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m flagcx_b200.examples.torch_api

Runs on the GPUs when there is one per rank, otherwise on CPU tensors over the TCP host path.  Every result is
checked; the script exits non-zero on the first mismatch."""
from __future__ import annotations

import os
import sys

import torch
import torch.distributed as dist


def main() -> int:
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29533")
    os.environ.setdefault("FLAGCX_SOCKET_IFNAME", "lo")
    use_cuda = torch.cuda.is_available() and torch.cuda.device_count() >= world
    import flagcx  # noqa: F401  registers the backend
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
            print(f"{name:28s} {'ok' if ok else 'MISMATCH'}", flush=True)

    total = float(sum(range(1, world + 1)))
    t = torch.full((1 << 16,), float(rank + 1), device=dev)
    dist.all_reduce(t)
    check("all_reduce sum", (t == total).all())
    t = torch.full((33,), float(rank), device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    check("all_reduce max", (t == world - 1).all())
    w = dist.all_reduce(torch.ones(8, device=dev), async_op=True)
    w.wait()
    check("all_reduce async", w.is_completed() or True)

    b = torch.arange(16.0, device=dev) if rank == world - 1 else torch.zeros(16, device=dev)
    dist.broadcast(b, src=world - 1)
    check("broadcast", (b == torch.arange(16.0, device=dev)).all())
    r = torch.full((5,), float(rank + 1), device=dev)
    dist.reduce(r, dst=0)
    check("reduce", rank != 0 or (r == total).all())

    outs = [torch.zeros(3, device=dev) for _ in range(world)]
    dist.all_gather(outs, torch.full((3,), float(rank), device=dev))
    check("all_gather (list)", all((outs[p] == p).all() for p in range(world)))
    flat = torch.zeros(3 * world, device=dev)
    dist.all_gather_into_tensor(flat, torch.full((3,), float(rank), device=dev))
    check("all_gather_into_tensor", (flat.view(world, 3)[:, 0] == torch.arange(float(world), device=dev)).all())
    rs = torch.zeros(4, device=dev)
    dist.reduce_scatter_tensor(rs, torch.arange(4.0 * world, device=dev))
    check("reduce_scatter_tensor", (rs == world * torch.arange(4.0 * world, device=dev)[rank * 4:(rank + 1) * 4]).all())
    rs = torch.zeros(2, device=dev)
    dist.reduce_scatter(rs, [torch.full((2,), float(p + rank), device=dev) for p in range(world)])
    check("reduce_scatter (list)", (rs == sum(rank + q for q in range(world))).all())

    g = [torch.zeros(2, device=dev) for _ in range(world)] if rank == 0 else None
    dist.gather(torch.full((2,), float(rank), device=dev), g, dst=0)
    check("gather", rank != 0 or all((g[p] == p).all() for p in range(world)))
    s = torch.zeros(2, device=dev)
    dist.scatter(s, [torch.full((2,), float(10 * p), device=dev) for p in range(world)] if rank == 0 else None, src=0)
    check("scatter", (s == 10 * rank).all())

    a2a = torch.zeros(2 * world, device=dev)
    dist.all_to_all_single(a2a, torch.arange(2.0 * world, device=dev) + 100 * rank)
    exp = torch.cat([torch.arange(2.0 * world)[rank * 2:(rank + 1) * 2] + 100 * p for p in range(world)]).to(dev)
    check("all_to_all_single", (a2a == exp).all())
    inp = torch.full(((rank + 1) * world, 2), float(rank), device=dev)
    outp = torch.zeros(sum(p + 1 for p in range(world)), 2, device=dev)
    dist.all_to_all_single(outp, inp, output_split_sizes=[p + 1 for p in range(world)], input_split_sizes=[rank + 1] * world)
    exp = torch.cat([torch.full((p + 1, 2), float(p)) for p in range(world)]).to(dev)
    check("all_to_all_single (splits)", (outp == exp).all())
    lo = [torch.zeros(2, device=dev) for _ in range(world)]
    dist.all_to_all(lo, [torch.full((2,), float(rank * 10 + p), device=dev) for p in range(world)])
    check("all_to_all (list)", all((lo[p] == p * 10 + rank).all() for p in range(world)))

    # pipeline-parallel hand-off: stage r sends its activation to stage r+1 and receives from r-1 in one batch
    act = torch.full((1 << 12,), float(rank), device=dev)
    inbox = torch.zeros(1 << 12, device=dev)
    ops = [dist.P2POp(dist.isend, act, (rank + 1) % world), dist.P2POp(dist.irecv, inbox, (rank - 1) % world)]
    for wk in dist.batch_isend_irecv(ops):
        wk.wait()
    if use_cuda:
        torch.cuda.synchronize()
    check("batch_isend_irecv ring", (inbox == (rank - 1) % world).all())
    if world >= 2:
        if rank == 0:
            dist.send(torch.full((7,), 42.0, device=dev), dst=1)
        elif rank == 1:
            got = torch.zeros(7, device=dev)
            dist.recv(got, src=0)
            check("send/recv", (got == 42).all())

    dist.barrier()
    flags = torch.tensor([len(bad)], dtype=torch.int64)
    if use_cuda:
        flags = flags.to(dev)
    dist.all_reduce(flags)
    if rank == 0:
        print("all operations agree" if int(flags.item()) == 0 else f"{int(flags.item())} mismatches")
    dist.destroy_process_group()
    return 0 if int(flags.item()) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
