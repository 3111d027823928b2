"""Real multi-GPU tests: one process per GPU, the C API through ctypes, results
compared with PyTorch references.  Run with as many ranks as there are GPUs
(capped at 8).  Covers every collective, the tuner-selectable variants
(including the NVSwitch multimem ones when the box has a multicast object),
heap-resident buffers, grouped send/recv, the c10d backend under
DistributedDataParallel, and the bounded-wait error path."""
import ctypes
import os

import pytest
import torch

from tests.mp_util import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    return min(torch.cuda.device_count(), 8)


def _stream(lib):
    return lib.adaptor_stream_copy(torch.cuda.current_stream())


def _setup(lib, uid, rank, world):
    torch.cuda.set_device(rank)
    torch.zeros(1, device="cuda")
    comm = lib.flagcxCommInitRank(world, uid, rank)
    return comm, _stream(lib)


def _seeded(rank, n, dtype, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(100 + rank)
    return (torch.rand(n, generator=g) * 2 - 1).to(dtype).to(device)


def _collectives(lib, uid, rank, world):
    comm, st = _setup(lib, uid, rank, world)
    DT = {torch.float32: 7, torch.bfloat16: 9, torch.float16: 6, torch.float8_e4m3fn: 10, torch.int32: 2}
    res = {"mc": False}
    bases = (ctypes.c_void_p * world)()
    mc = ctypes.c_void_p()
    hb = ctypes.c_size_t()
    lib.call("flagcxCommHeapInfo", comm, bases, ctypes.byref(mc), ctypes.byref(hb))
    res["mc"] = bool(mc.value)
    fails = []

    def check(name, got, ref, atol, rtol=1e-2):
        if not torch.allclose(got.float(), ref.float(), atol=atol, rtol=rtol):
            fails.append((name, float((got.float() - ref.float()).abs().max())))

    variants = [None, ("ar_ll", 2), ("ar_oneshot", 8), ("ar_twoshot", 16)]
    if res["mc"]:
        variants.append(("ar_nvls", 16))
    for dtype, atol in ((torch.float32, 1e-5), (torch.bfloat16, 0.03 * world)):
        for count in (1, 257, 4096, 1 << 16, (1 << 20) + 3, 1 << 24):
            xs = [_seeded(r, count, dtype, "cpu").float() for r in range(world)]
            ref = torch.stack(xs).sum(0)
            for var in variants:
                if var and var[0] == "ar_ll" and count * dtype.itemsize > 32768:
                    continue
                if var and var[0] == "ar_oneshot" and count * dtype.itemsize > (8 << 20):
                    continue
                lib.tuner_pin(comm, var[0] if var else None, var[1] if var else 1)
                x = _seeded(rank, count, dtype)
                y = torch.empty_like(x)
                for _ in range(3):
                    lib.flagcxAllReduce(x.data_ptr(), y.data_ptr(), count, DT[dtype], 0, comm, st)
                torch.cuda.synchronize()
                check(f"allreduce {dtype} {count} {var}", y.cpu(), ref, atol)
    lib.tuner_pin(comm, None)
    # max on bf16 and avg on fp32 through the default path (and NVLS when present)
    for var in [None] + ([("ar_nvls", 8)] if res["mc"] else []):
        lib.tuner_pin(comm, var[0] if var else None, var[1] if var else 1)
        x = _seeded(rank, 100000, torch.bfloat16)
        y = torch.empty_like(x)
        lib.flagcxAllReduce(x.data_ptr(), y.data_ptr(), x.numel(), 9, 2, comm, st)
        torch.cuda.synchronize()
        ref = torch.stack([_seeded(r, 100000, torch.bfloat16, "cpu").float() for r in range(world)]).max(0).values
        check(f"allreduce max {var}", y.cpu(), ref, 0)
        x = _seeded(rank, 100000, torch.float32)
        lib.flagcxAllReduce(x.data_ptr(), x.data_ptr(), x.numel(), 7, 4, comm, st)
        torch.cuda.synchronize()
        ref = torch.stack([_seeded(r, 100000, torch.float32, "cpu") for r in range(world)]).mean(0)
        check(f"allreduce avg in place {var}", x.cpu(), ref, 1e-5)
    lib.tuner_pin(comm, None)
    # fused cast: bf16 in, fp8 out, scaled
    x = _seeded(rank, 50000, torch.bfloat16)
    y = torch.empty(50000, dtype=torch.float8_e4m3fn, device="cuda")
    lib.flagcxAllReduceCast(x.data_ptr(), y.data_ptr(), 50000, 9, 10, 0.25, 0, comm, st)
    torch.cuda.synchronize()
    ref = (torch.stack([_seeded(r, 50000, torch.bfloat16, "cpu").float() for r in range(world)]).sum(0) * 0.25)
    check("allreduce cast fp8", y.cpu().float(), ref.to(torch.float8_e4m3fn).float(), 0.07 * world, 0.13)

    # reduce-scatter / all-gather, default and NVLS variants
    for count in (1, 1000, 1 << 18, (1 << 22) + 8):
        for var in [None] + ([("nvls", 16)] if res["mc"] else []):
            xs = [_seeded(r, count * world, torch.float32, "cpu") for r in range(world)]
            x = xs[rank].cuda()
            y = torch.empty(count, device="cuda")
            lib.tuner_pin(comm, "rs_nvls" if var else None, 16)
            lib.flagcxReduceScatter(x.data_ptr(), y.data_ptr(), count, 7, 0, comm, st)
            torch.cuda.synchronize()
            check(f"reducescatter {count} {var}", y.cpu(), torch.stack(xs).sum(0)[rank * count:(rank + 1) * count], 1e-5)
            z = torch.empty(count * world, device="cuda")
            lib.tuner_pin(comm, "ag_nvls" if var else None, 16)
            lib.flagcxAllGather(y.data_ptr(), z.data_ptr(), count, 7, comm, st)
            torch.cuda.synchronize()
            check(f"allgather {count} {var}", z.cpu(), torch.stack(xs).sum(0), 1e-5)
    lib.tuner_pin(comm, None)
    # rooted ops and all-to-all
    count = 70001
    for root in (0, world - 1):
        xs = [_seeded(r, count * world, torch.float32, "cpu") for r in range(world)]
        x = xs[rank].cuda()
        b = x[:count].clone()
        lib.flagcxBroadcast(b.data_ptr(), b.data_ptr(), count, 7, root, comm, st)
        torch.cuda.synchronize()
        check(f"broadcast root {root}", b.cpu(), xs[root][:count], 0)
        r = torch.zeros(count, device="cuda")
        lib.flagcxReduce(x.data_ptr(), r.data_ptr(), count, 7, 0, root, comm, st)
        torch.cuda.synchronize()
        if rank == root:
            check(f"reduce root {root}", r.cpu(), torch.stack([t[:count] for t in xs]).sum(0), 1e-5)
        g = torch.zeros(count * world, device="cuda")
        lib.flagcxGather(x.data_ptr(), g.data_ptr(), count, 7, root, comm, st)
        torch.cuda.synchronize()
        if rank == root:
            check(f"gather root {root}", g.cpu(), torch.cat([t[:count] for t in xs]), 0)
        s = torch.zeros(count, device="cuda")
        lib.flagcxScatter(x.data_ptr(), s.data_ptr(), count, 7, root, comm, st)
        torch.cuda.synchronize()
        check(f"scatter root {root}", s.cpu(), xs[root][rank * count:(rank + 1) * count], 0)
    xs = [_seeded(r, count * world, torch.float32, "cpu") for r in range(world)]
    a = torch.zeros(count * world, device="cuda")
    lib.flagcxAlltoAll(xs[rank].cuda().data_ptr(), a.data_ptr(), count, 7, comm, st)
    torch.cuda.synchronize()
    check("alltoall", a.cpu(), torch.cat([xs[p][rank * count:(rank + 1) * count] for p in range(world)]), 0)
    sc = [1000 * ((rank + p) % 3) + 5 * p for p in range(world)]
    sd = [sum(sc[:p]) for p in range(world)]
    rc = [1000 * ((p + rank) % 3) + 5 * rank for p in range(world)]
    rd = [sum(rc[:p]) for p in range(world)]
    src = xs[rank][:max(1, sum(sc))].cuda()
    dst = torch.zeros(max(1, sum(rc)), device="cuda")
    lib.flagcxAlltoAllv(src.data_ptr(), sc, sd, dst.data_ptr(), rc, rd, 7, comm, st)
    torch.cuda.synchronize()
    exp = []
    for p in range(world):
        psc = [1000 * ((p + q) % 3) + 5 * q for q in range(world)]
        off = sum(psc[:rank])
        exp.append(xs[p][off:off + psc[rank]])
    check("alltoallv", dst.cpu()[:sum(rc)], torch.cat(exp), 0)

    # grouped ring send/recv: staged (ordinary memory) and zero-copy (heap memory), several sizes
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for n in (0, 5, 100000, (9 << 20) + 7):
        s = _seeded(rank, max(n, 1), torch.float32)
        r = torch.zeros(max(n, 1), device="cuda")
        lib.flagcxGroupStart(comm)
        lib.flagcxSend(s.data_ptr(), n, 7, nxt, comm, st)
        lib.flagcxRecv(r.data_ptr(), n, 7, prv, comm, st)
        lib.flagcxGroupEnd(comm)
        torch.cuda.synchronize()
        if n:
            check(f"sendrecv staged {n}", r.cpu(), _seeded(prv, n, torch.float32, "cpu"), 0)
    n = 1 << 20
    hp = lib.flagcxMemAlloc(n * 4, comm)
    src = _seeded(rank, n, torch.float32)
    lib.handler.contents.devHandle.contents.deviceMemcpy(hp, src.data_ptr(), n * 4, 2, st)
    r = torch.zeros(n, device="cuda")
    lib.flagcxGroupStart(comm)
    lib.flagcxSend(hp, n, 7, nxt, comm, st)
    lib.flagcxRecv(r.data_ptr(), n, 7, prv, comm, st)
    lib.flagcxGroupEnd(comm)
    torch.cuda.synchronize()
    check("sendrecv zero-copy", r.cpu(), _seeded(prv, n, torch.float32, "cpu"), 0)
    lib.flagcxMemFree(hp, comm)
    lib.flagcxBarrier(comm, st)
    res["async_error"] = lib.flagcxCommGetAsyncError(comm)
    res["counters"] = lib.counters(comm)["launches"]
    res["fails"] = fails
    lib.flagcxCommDestroy(comm)
    return res


def test_collectives_all_ranks(native_lib):
    world = _world()
    res, _ = run_ranks(_collectives, world, timeout=900, env={"FLAGCX_KERNEL_TIMEOUT_MS": "20000", "FLAGCX_P2P_ZEROCOPY": "1"})
    for r in range(world):
        out = res[r][1]
        assert out["fails"] == [], out["fails"][:10]
        assert out["async_error"] == 0
        assert out["counters"] > 0


def _timeout_path(lib, uid, rank, world):
    comm, st = _setup(lib, uid, rank, world)
    out = {}
    if rank == 0:
        lib.call("flagcxCommSetTimeoutMs", comm, 300)
        # a wait that nothing satisfies: returns after the deadline with an error record, context stays usable
        lib.call("flagcxCommWaitTest", comm, st)
        torch.cuda.synchronize()
        code, peer, where = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        exp, seen = ctypes.c_ulonglong(), ctypes.c_ulonglong()
        lib.call("flagcxCommGetDeviceError", comm, ctypes.byref(code), ctypes.byref(peer), ctypes.byref(where), ctypes.byref(exp), ctypes.byref(seen))
        out["code"], out["where"] = code.value, where.value
        out["async"] = lib.flagcxCommGetAsyncError(comm)
        out["still_works"] = float(torch.ones(4, device="cuda").sum().item())
        lib.call("flagcxCommClearError", comm)
        out["async_after_clear"] = lib.flagcxCommGetAsyncError(comm)
        lib.call("flagcxCommSetTimeoutMs", comm, 20000)
    x = torch.ones(1000, device="cuda")
    lib.flagcxAllReduce(x.data_ptr(), x.data_ptr(), 1000, 7, 0, comm, st)
    torch.cuda.synchronize()
    out["sum"] = float(x[0].item())
    lib.flagcxCommDestroy(comm)
    return out


def test_bounded_wait_reports_and_recovers(native_lib):
    world = min(_world(), 2)
    res, _ = run_ranks(_timeout_path, world, timeout=300, env={"NCCL_NVLS_ENABLE": "0", "FLAGCX_NVLS_ENABLE": "0"})
    out0 = res[0][1]
    assert out0["code"] == 1 and out0["where"] == 7 and out0["async"] == 6
    assert out0["still_works"] == 4.0 and out0["async_after_clear"] == 0
    for r in range(world):
        assert res[r][1]["sum"] == world


def _torch_ddp(lib, uid, rank, world, port):
    import torch.distributed as dist
    import torch.nn as nn
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    import flagcx  # noqa: F401
    dist.init_process_group("cpu:gloo,cuda:flagcx", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = nn.Sequential(nn.Linear(512, 2048), nn.GELU(), nn.Linear(2048, 512)).cuda()
    ddp = nn.parallel.DistributedDataParallel(model, device_ids=[rank], bucket_cap_mb=1)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
    torch.manual_seed(10 + rank)
    for _ in range(3):
        x = torch.randn(64, 512, device="cuda")
        ddp(x).square().mean().backward()
        opt.step()
        opt.zero_grad()
    # all ranks must hold identical weights
    w = model[0].weight.detach().clone()
    ws = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(ws, w)
    same = all(bool(torch.equal(ws[0], t)) for t in ws)
    # uneven all_to_all_single and batched p2p on device tensors
    inp = torch.full(((rank + 1) * world, 3), float(rank), device="cuda")
    outp = torch.zeros(sum(p + 1 for p in range(world)), 3, device="cuda")
    dist.all_to_all_single(outp, inp, output_split_sizes=[p + 1 for p in range(world)], input_split_sizes=[rank + 1] * world)
    exp = torch.cat([torch.full((p + 1, 3), float(p)) for p in range(world)]).cuda()
    a2a = bool(torch.equal(outp, exp))
    rcv = torch.zeros(1 << 16, device="cuda")
    ops = [dist.P2POp(dist.isend, torch.full((1 << 16,), float(rank), device="cuda"), (rank + 1) % world),
           dist.P2POp(dist.irecv, rcv, (rank - 1) % world)]
    for wk in dist.batch_isend_irecv(ops):
        wk.wait()
    torch.cuda.synchronize()
    p2p = bool((rcv == (rank - 1) % world).all())
    dist.barrier(device_ids=[rank])
    dist.destroy_process_group()
    return {"same": same, "a2a": a2a, "p2p": p2p}


def test_c10d_backend_ddp(native_lib):
    import socket
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    world = _world()
    res, _ = run_ranks(_torch_ddp, world, args=(port,), timeout=600)
    for r in range(world):
        assert res[r][1] == {"same": True, "a2a": True, "p2p": True}, res[r][1]
