"""Ring attention, Ulysses attention and the pipeline schedules on the "flagcx" backend with CPU tensors (TCP host
path): forward results and gradients against one process that sees the whole sequence / the whole model."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

B, H, D = 2, 6, 8


def _full_attention(q, k, v, causal):
    return torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=causal)


def _worker(rank, world, port, q_out):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), FLAGCX_SOCKET_IFNAME="lo")
        import flagcx  # noqa: F401
        from flagcx_b200.parallel.cp import ring_attention, ulysses_attention
        from flagcx_b200.parallel.pp import PipelineStage
        dist.init_process_group("flagcx", rank=rank, world_size=world)
        out = {}
        tl = 5
        T = tl * world
        g = torch.Generator().manual_seed(11)
        q, k, v, go = (torch.randn(B, H, T, D, generator=g, dtype=torch.float64) for _ in range(4))
        mine = slice(rank * tl, (rank + 1) * tl)
        for causal in (False, True):
            # the oracle: one process, whole sequence
            qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
            ref = _full_attention(qr, kr, vr, causal)
            ref.backward(go)
            # ring: [B, H, T/n, D] shards
            ql, kl, vl = (t[:, :, mine].clone().requires_grad_(True) for t in (q, k, v))
            o = ring_attention(ql, kl, vl, causal=causal)
            o.backward(go[:, :, mine])
            tag = "causal" if causal else "full"
            out[f"ring {tag} fwd"] = bool(torch.allclose(o, ref[:, :, mine].detach(), atol=1e-9))
            for name, got, want in (("dq", ql.grad, qr.grad), ("dk", kl.grad, kr.grad), ("dv", vl.grad, vr.grad)):
                out[f"ring {tag} {name}"] = bool(torch.allclose(got, want[:, :, mine], atol=1e-9))
            # Ulysses: [B, T/n, H, D] shards, H divisible by the world
            if H % world == 0:
                qu, ku, vu = (t[:, :, mine].transpose(1, 2).clone().requires_grad_(True) for t in (q, k, v))
                o = ulysses_attention(qu, ku, vu, causal=causal)
                o.backward(go[:, :, mine].transpose(1, 2))
                out[f"ulysses {tag} fwd"] = bool(torch.allclose(o.transpose(1, 2), ref[:, :, mine].detach(), atol=1e-9))
                for name, got, want in (("dq", qu.grad, qr.grad), ("dk", ku.grad, kr.grad), ("dv", vu.grad, vr.grad)):
                    out[f"ulysses {tag} {name}"] = bool(torch.allclose(got.transpose(1, 2), want[:, :, mine], atol=1e-9))
        # pipeline: stage s = layer s of an MLP stack; micro-batches against the same stack in one process
        width, mb, m = 16, 4, 5
        torch.manual_seed(3)
        layers = [torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.Tanh()).double() for _ in range(world)]
        xs = [torch.randn(mb, width, dtype=torch.float64) for _ in range(m)]
        ys = [torch.randn(mb, width, dtype=torch.float64) for _ in range(m)]
        loss_fn = torch.nn.functional.mse_loss
        ref_model = torch.nn.Sequential(*[torch.nn.Sequential(torch.nn.Linear(width, width), torch.nn.Tanh()).double() for _ in range(world)])
        for a, b in zip(ref_model, layers):
            a.load_state_dict(b.state_dict())
        ref_loss = sum(loss_fn(ref_model(x), y) for x, y in zip(xs, ys)) / m
        ref_loss.backward()
        for schedule in ("gpipe", "1f1b"):
            stage = layers[rank]
            stage.zero_grad()
            pipe = PipelineStage(stage, activation_shape=(mb, width), dtype=torch.float64, device=torch.device("cpu"))
            loss = pipe.run(xs if rank == 0 else None, ys if rank == world - 1 else None, loss_fn, micro_batches=m, schedule=schedule)
            if rank == world - 1:
                out[f"pipeline {schedule} loss"] = bool(torch.allclose(loss, ref_loss.detach(), atol=1e-12))
            for (n1, p1), (n2, p2) in zip(stage.named_parameters(), ref_model[rank].named_parameters()):
                out[f"pipeline {schedule} grad {n1}"] = bool(torch.allclose(p1.grad, p2.grad, atol=1e-12))
        dist.barrier()
        dist.destroy_process_group()
        q_out.put((rank, "ok", out))
    except BaseException:  # noqa
        import traceback
        q_out.put((rank, "err", traceback.format_exc()))


@pytest.mark.parametrize("world", [2, 3])
def test_sequence_and_pipeline_parallel_cpu(native_lib, world):
    from flagcx_b200 import _build
    _build.build_torch_ext()
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        rank, status, out = q.get(timeout=240)
        res[rank] = (status, out)
    for p in procs:
        p.join(timeout=20)
    for r in range(world):
        assert res[r][0] == "ok", res[r][1]
        assert len(res[r][1]) > 8
        for k, v in res[r][1].items():
            assert v, (r, k)
