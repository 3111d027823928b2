"""Zero-copy collectives on real GPUs: buffers in the symmetric heap (flagcxMemAlloc) and buffers made
peer-visible with flagcxCommRegister, one process per GPU, results against PyTorch references.

Covered: every collective on heap buffers with the plan the tuner picks (which must be a zero-copy kind: the
per-kind launch counters are checked), in place and out of place, through the switch (multimem) and with it
turned off, heap offsets that differ between ranks (which rules the multicast alias out), registered
cudaMalloc buffers, a CTA budget, and a mix of zero-copy and staged calls on one communicator."""
import ctypes
import os

import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

K_AR_ZC, K_RS_ZC, K_REDUCE_ZC, K_MOVE_ZC, K_MOVE_CE = 18, 19, 20, 21, 22


def _world():
    return min(torch.cuda.device_count(), 8)


def _copy_engine_supported(world):
    return world == 2 or os.environ.get("FLAGCX_COPY_ENGINE") == "1"


def _seeded(rank, n, dtype, device="cuda", salt=0):
    g = torch.Generator(device="cpu").manual_seed(100 + rank + 1000 * salt)
    return (torch.rand(n, generator=g) * 2 - 1).to(dtype).to(device)


def _zero_copy(lib, uid, rank, world, skew):
    import flagcx_b200
    torch.cuda.set_device(rank)
    torch.zeros(1, device="cuda")
    native = flagcx_b200.native(build_if_missing=False)
    comm = lib.flagcxCommInitRank(world, uid, rank)
    st = lib.adaptor_stream_copy(torch.cuda.current_stream())
    h = comm.value
    fails = []

    def check(name, got, ref, atol, rtol=1e-2):
        if not torch.allclose(got.float().cpu(), ref.float(), atol=atol, rtol=rtol):
            fails.append((name, float((got.float().cpu() - ref.float()).abs().max())))

    pad = None
    if skew:  # push this rank's later allocations to a rank-dependent offset: no common multicast address
        pad = native.heap_tensor(h, [4096 * (rank + 1)], torch.uint8)

    def heap(n, dtype):
        return native.heap_tensor(h, [n], dtype)

    DT = {torch.float32: 7, torch.bfloat16: 9}
    for dtype, atol in ((torch.float32, 1e-5), (torch.bfloat16, 0.03 * world)):
        for count in (1, 257, 4099, (1 << 20) + 3, 1 << 23):
            xs = [_seeded(r, count, dtype, "cpu").float() for r in range(world)]
            x, y = heap(count, dtype), heap(count, dtype)
            x.copy_(_seeded(rank, count, dtype))
            for _ in range(3):
                lib.flagcxAllReduce(x.data_ptr(), y.data_ptr(), count, DT[dtype], 0, comm, st)
            torch.cuda.synchronize()
            check(f"allreduce {dtype} {count}", y, torch.stack(xs).sum(0), atol)
            lib.flagcxAllReduce(x.data_ptr(), x.data_ptr(), count, DT[dtype], 4, comm, st)  # in place, average
            torch.cuda.synchronize()
            check(f"allreduce avg in place {dtype} {count}", x, torch.stack(xs).mean(0), atol)
            del x, y
    # max on bf16 (the switch can do it) and on fp32 (it cannot: plain loads), pinned CTA counts
    for dtype in (torch.bfloat16, torch.float32):
        for nctas in (1, 5, 32):
            lib.tuner_pin(comm, "ar_zc", nctas)
            x, y = heap(100001, dtype), heap(100001, dtype)
            x.copy_(_seeded(rank, 100001, dtype))
            lib.flagcxAllReduce(x.data_ptr(), y.data_ptr(), 100001, DT[dtype], 2, comm, st)
            torch.cuda.synchronize()
            ref = torch.stack([_seeded(r, 100001, dtype, "cpu").float() for r in range(world)]).max(0).values
            check(f"allreduce max {dtype} x{nctas}", y, ref, 0)
            del x, y
    lib.tuner_pin(comm, None)
    # fused cast
    x, y = heap(50000, torch.bfloat16), heap(50000, torch.float8_e4m3fn)
    x.copy_(_seeded(rank, 50000, torch.bfloat16))
    lib.flagcxAllReduceCast(x.data_ptr(), y.data_ptr(), 50000, 9, 10, 0.25, 0, comm, st)
    torch.cuda.synchronize()
    ref = torch.stack([_seeded(r, 50000, torch.bfloat16, "cpu").float() for r in range(world)]).sum(0) * 0.25
    check("allreduce cast fp8", y.float(), ref.to(torch.float8_e4m3fn).float(), 0.07 * world, 0.13)
    del x, y

    for count in (1, 1000, (1 << 20) + 8):
        xs = [_seeded(r, count * world, torch.float32, "cpu") for r in range(world)]
        tot = torch.stack(xs).sum(0)
        x, y, z = heap(count * world, torch.float32), heap(count, torch.float32), heap(count * world, torch.float32)
        x.copy_(xs[rank])
        lib.flagcxReduceScatter(x.data_ptr(), y.data_ptr(), count, 7, 0, comm, st)
        torch.cuda.synchronize()
        check(f"reducescatter {count}", y, tot[rank * count:(rank + 1) * count], 1e-5)
        lib.flagcxAllGather(y.data_ptr(), z.data_ptr(), count, 7, comm, st)
        torch.cuda.synchronize()
        check(f"allgather {count}", z, tot, 1e-5)
        # in place: the piece already sits at its place in the receive buffer
        z.zero_()
        z[rank * count:(rank + 1) * count] = y
        lib.flagcxAllGather(z[rank * count:].data_ptr(), z.data_ptr(), count, 7, comm, st)
        torch.cuda.synchronize()
        check(f"allgather in place {count}", z, tot, 1e-5)
        for root in (0, world - 1):
            b = heap(count, torch.float32)
            b.copy_(xs[rank][:count])
            lib.flagcxBroadcast(b.data_ptr(), b.data_ptr(), count, 7, root, comm, st)
            torch.cuda.synchronize()
            check(f"broadcast {count} root {root}", b, xs[root][:count], 0)
            r_ = heap(count, torch.float32)
            r_.zero_()
            lib.flagcxReduce(x.data_ptr(), r_.data_ptr(), count, 7, 0, root, comm, st)
            torch.cuda.synchronize()
            if rank == root:
                check(f"reduce {count} root {root}", r_, torch.stack([t[:count] for t in xs]).sum(0), 1e-5)
            g = heap(count * world, torch.float32)
            g.zero_()
            lib.flagcxGather(x.data_ptr(), g.data_ptr(), count, 7, root, comm, st)
            torch.cuda.synchronize()
            if rank == root:
                check(f"gather {count} root {root}", g, torch.cat([t[:count] for t in xs]), 0)
            s = heap(count, torch.float32)
            s.zero_()
            lib.flagcxScatter(x.data_ptr(), s.data_ptr(), count, 7, root, comm, st)
            torch.cuda.synchronize()
            check(f"scatter {count} root {root}", s, xs[root][rank * count:(rank + 1) * count], 0)
            del b, r_, g, s
        a = heap(count * world, torch.float32)
        a.zero_()
        lib.flagcxAlltoAll(x.data_ptr(), a.data_ptr(), count, 7, comm, st)
        torch.cuda.synchronize()
        check(f"alltoall {count}", a, torch.cat([xs[p][rank * count:(rank + 1) * count] for p in range(world)]), 0)
        del x, y, z, a
    # all-to-all-v: the send buffers are peer-visible, the receive buffer is ordinary memory
    big = [_seeded(r, 4000 * world, torch.float32, "cpu", salt=3) for r in range(world)]
    sc = [1000 * ((rank + p) % 3) + 5 * p for p in range(world)]
    sd = [sum(sc[:p]) for p in range(world)]
    rc = [1000 * ((p + rank) % 3) + 5 * rank for p in range(world)]
    rd = [sum(rc[:p]) for p in range(world)]
    src = heap(max(1, sum(sc)), torch.float32)
    src.copy_(big[rank][:max(1, sum(sc))])
    dst = torch.zeros(max(1, sum(rc)), device="cuda")
    lib.flagcxAlltoAllv(src.data_ptr(), sc, sd, dst.data_ptr(), rc, rd, 7, comm, st)
    torch.cuda.synchronize()
    exp = []
    for p in range(world):
        psc = [1000 * ((p + q) % 3) + 5 * q for q in range(world)]
        off = sum(psc[:rank])
        exp.append(big[p][off:off + psc[rank]])
    check("alltoallv", dst[:sum(rc)], torch.cat(exp), 0)
    del src, dst  # their sizes differ between the ranks: freed, so that what follows sits at one heap offset everywhere
    # The copy-engine form needs one heap offset on all ranks (checked on the device).  It is a supported choice on two
    # ranks; beyond that the tuner offers it only with FLAGCX_COPY_ENGINE=1, and so does this test.
    if not skew and _copy_engine_supported(world):
        # copy-engine form of the push movers: two one-CTA kernels around peer copies queued by the host
        lib.tuner_pin(comm, "move_ce", 1)
        cnt = (1 << 19) + 64
        xs = [_seeded(r, cnt * world, torch.float32, "cpu", salt=8) for r in range(world)]
        x, g = heap(cnt * world, torch.float32), heap(cnt * world, torch.float32)
        x.copy_(xs[rank])
        for rep in range(2):
            g.zero_()
            lib.flagcxAllGather(x.data_ptr(), g.data_ptr(), cnt, 7, comm, st)
            torch.cuda.synchronize()
            check(f"allgather copy-engine {rep}", g, torch.cat([t[:cnt] for t in xs]), 0)
        g.zero_()
        lib.flagcxAlltoAll(x.data_ptr(), g.data_ptr(), cnt, 7, comm, st)
        torch.cuda.synchronize()
        check("alltoall copy-engine", g, torch.cat([xs[p][rank * cnt:(rank + 1) * cnt] for p in range(world)]), 0)
        b = heap(cnt, torch.float32)
        b.copy_(xs[rank][:cnt])
        lib.flagcxBroadcast(b.data_ptr(), b.data_ptr(), cnt, 7, world - 1, comm, st)
        torch.cuda.synchronize()
        check("broadcast copy-engine", b, xs[world - 1][:cnt], 0)
        sc_ = heap(cnt, torch.float32)
        sc_.zero_()
        lib.flagcxScatter(x.data_ptr(), sc_.data_ptr(), cnt, 7, 0, comm, st)
        torch.cuda.synchronize()
        check("scatter copy-engine", sc_, xs[0][rank * cnt:(rank + 1) * cnt], 0)
        lib.tuner_pin(comm, None)
        del x, g, b, sc_
    kinds_heap = lib.counters(comm)["kind_launches"]

    # registered cudaMalloc buffers (not in the heap): same kernels through the segment table
    n = 300007
    lib.call("flagcxCommSetCtaBudget", comm, 8)
    # registration needs the base of an allocation: without a communicator flagcxMemAlloc is a plain cudaMalloc
    ps = lib.flagcxMemAlloc(n * 4, None)
    pr = lib.flagcxMemAlloc(n * 4, None)
    hs = lib.flagcxCommRegister(comm, ps, n * 4)
    hr = lib.flagcxCommRegister(comm, pr, n * 4)
    src = _seeded(rank, n, torch.float32, salt=5)
    dh = lib.handler.contents.devHandle.contents
    dh.deviceMemcpy(ps, src.data_ptr(), n * 4, 2, st)
    before = lib.counters(comm)["kind_launches"][K_AR_ZC]
    lib.flagcxAllReduce(ps, pr, n, 7, 0, comm, st)
    out = torch.empty(n, device="cuda")
    dh.deviceMemcpy(out.data_ptr(), pr, n * 4, 2, st)
    torch.cuda.synchronize()
    check("allreduce registered", out, torch.stack([_seeded(r, n, torch.float32, "cpu", salt=5) for r in range(world)]).sum(0), 1e-5)
    registered_zc = lib.counters(comm)["kind_launches"][K_AR_ZC] - before
    # a staged call (ordinary tensors) in between, then zero-copy again
    t = _seeded(rank, 70001, torch.float32, salt=6)
    lib.flagcxAllReduce(t.data_ptr(), t.data_ptr(), 70001, 7, 0, comm, st)
    torch.cuda.synchronize()
    check("allreduce staged between", t, torch.stack([_seeded(r, 70001, torch.float32, "cpu", salt=6) for r in range(world)]).sum(0), 1e-5)
    lib.flagcxAllReduce(ps, ps, n, 7, 4, comm, st)
    dh.deviceMemcpy(out.data_ptr(), ps, n * 4, 2, st)
    torch.cuda.synchronize()
    check("allreduce registered in place", out, torch.stack([_seeded(r, n, torch.float32, "cpu", salt=5) for r in range(world)]).mean(0), 1e-5)
    lib.flagcxBarrier(comm, st)
    lib.flagcxCommDeregister(comm, hs)
    lib.flagcxCommDeregister(comm, hr)
    lib.flagcxMemFree(ps, None)
    lib.flagcxMemFree(pr, None)
    res = {"fails": fails, "async": lib.flagcxCommGetAsyncError(comm), "kinds": kinds_heap, "registered_zc": registered_zc}
    del pad
    lib.flagcxCommDestroy(comm)
    return res


@pytest.mark.parametrize("mode", ["switch", "plain", "skewed"])
def test_zero_copy_collectives(native_lib, mode):
    world = _world()
    # the cost model decides here (no measured table): it is what sends peer-visible buffers to the zero-copy kinds
    env = {"FLAGCX_KERNEL_TIMEOUT_MS": "20000", "FLAGCX_HEAP_USER_BYTES": str(1 << 30), "FLAGCX_TUNER_DEFAULTS": "0"}
    if mode == "plain":
        env["FLAGCX_ZC_MC"] = "0"
    res, _ = run_ranks(_zero_copy, world, args=(mode == "skewed",), timeout=900, env=env)
    for r in range(world):
        out = res[r][1]
        assert out["fails"] == [], out["fails"][:10]
        assert out["async"] == 0
        k = out["kinds"]
        assert k[K_AR_ZC] > 0 and k[K_RS_ZC] > 0 and k[K_MOVE_ZC] > 0, k
        assert k[K_MOVE_CE] == (5 if mode != "skewed" and _copy_engine_supported(world) else 0), k
        assert out["registered_zc"] == 1


def _ddp_matches_single_process(lib, uid, rank, world, port):
    """N ranks x micro-batch b through DataParallelTrainer against one fp32 PyTorch model on the N*b batch."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import flagcx  # noqa: F401
    from flagcx_b200.models.gpt2 import GPT2, GPT2Config
    from flagcx_b200.parallel.ddp import DataParallelTrainer
    dist.init_process_group("cpu:gloo,cuda:flagcx", rank=rank, world_size=world)
    cfg = GPT2Config.tiny()
    b, T, steps = 2, cfg.seq_len, 3
    g = torch.Generator().manual_seed(7)
    toks = torch.randint(0, cfg.vocab, (steps, world * b, T), generator=g)
    tgts = torch.randint(0, cfg.vocab, (steps, world * b, T), generator=g)

    torch.manual_seed(0)
    model = GPT2(cfg)
    ref = GPT2(cfg)
    ref.load_state_dict(model.state_dict())
    trainer = DataParallelTrainer(model, lr=1e-3, use_graph=False, device=torch.device("cuda", rank))
    trainer.snapshot_grads = True

    # the oracle: same architecture in plain fp32 PyTorch on the concatenated batch, bf16-rounded start weights
    import torch.nn.functional as F
    ref = ref.cuda().float()
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(p.to(torch.bfloat16).float())
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-3, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)

    def ref_loss(tok, tgt):
        B, T_ = tok.shape
        x = F.embedding(tok, ref.wte) + ref.wpe[:T_]
        for blk in ref.blocks:
            C = x.shape[-1]
            h = F.layer_norm(x, (C,), blk.ln1_w, blk.ln1_b)
            qkv = F.linear(h, blk.qkv_w, blk.qkv_b).view(B, T_, 3, blk.n_head, C // blk.n_head)
            q, k, v = qkv.unbind(2)
            att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
            x = x + F.linear(att.transpose(1, 2).reshape(B, T_, C), blk.proj_w, blk.proj_b)
            h = F.layer_norm(x, (C,), blk.ln2_w, blk.ln2_b)
            x = x + F.linear(F.gelu(F.linear(h, blk.fc_w, blk.fc_b), approximate="tanh"), blk.out_w, blk.out_b)
        h = F.layer_norm(x, (x.shape[-1],), ref.lnf_w, ref.lnf_b)
        logits = F.linear(h.view(B * T_, -1), ref.wte)[:, :cfg.vocab]
        return F.cross_entropy(logits, tgt.view(-1))

    out = {"loss": [], "ref_loss": [], "grad_rel": None}
    for s in range(steps):
        mine = slice(rank * b, (rank + 1) * b)
        loss = trainer.step(toks[s, mine].cuda(), tgts[s, mine].cuda())
        lt = loss.detach().float().cpu().reshape(1)
        dist.all_reduce(lt)  # gloo: the mean of the ranks' losses is the loss of the global batch
        out["loss"].append(float(lt / world))
        opt.zero_grad()
        rl = ref_loss(toks[s].cuda(), tgts[s].cuda())
        rl.backward()
        if s == 0:
            got = trainer.grad_snapshot.float()
            want = torch.zeros_like(got)
            for (name, off, cnt), p in zip(trainer.specs, ref.parameters()):
                want[off:off + cnt] = p.grad.reshape(-1)
            out["grad_rel"] = float((got - want).norm() / want.norm())
            out["grad_cos"] = float(torch.nn.functional.cosine_similarity(got, want, dim=0))
        opt.step()
        out["ref_loss"].append(float(rl))
    # all ranks hold the same weights, bit for bit
    w = trainer.flat_params.detach().clone()
    ws = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(ws, w)
    out["same"] = all(bool(torch.equal(ws[0], t)) for t in ws)
    out["kinds"] = trainer.native.comm_counters(trainer.comm)["kind_launches"]
    torch.cuda.synchronize()
    dist.barrier(device_ids=[rank])
    dist.destroy_process_group()
    return out


def test_ddp_trainer_matches_single_process_on_the_global_batch(native_lib):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = _world()
    res, _ = run_ranks(_ddp_matches_single_process, world, args=(port,), timeout=600, env={"FLAGCX_TUNER_DEFAULTS": "0"})
    for r in range(world):
        out = res[r][1]
        assert out["same"]
        assert out["kinds"][K_AR_ZC] > 0, out["kinds"]  # the buckets went through the zero-copy kernel
        # gradients of step 1: bf16 model and bf16 all-reduce against fp32 autograd on the global batch
        assert out["grad_cos"] > 0.995 and out["grad_rel"] < 0.1, out
        for a, b_ in zip(out["loss"], out["ref_loss"]):
            assert abs(a - b_) < 0.03 * abs(b_), (out["loss"], out["ref_loss"])
