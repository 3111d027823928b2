"""Collective performance sweep with the reference's command line.

    python -m flagcx_b200.perf --op allreduce -b 8 -e 4G -f 2 -w 5 -n 20 --gpus 8
    python -m flagcx_b200.perf --op allreduce --lib reference ...   # same driver, reference libflagcx.so

Options follow the reference's perf binaries (test/perf/tools.cc:80-199):
``-b`` min bytes, ``-e`` max bytes, ``-f`` factor, ``-w`` warm-up iterations,
``-n`` timed iterations, ``-p`` print buffers, ``-r`` root (-1: all roots in
turn), ``-R`` 1: buffers from flagcxMemAlloc (+ flagcxCommRegister).  ``size``
is the total buffer in bytes; all-gather, reduce-scatter, all-to-all, gather
and scatter move ``size / nranks`` per rank, as the reference's tests do
(test/perf/test_allgather.cpp:99).  Bus-bandwidth factors are the reference's
(test/perf/test_allreduce.cpp:113 and siblings).

Both libraries are driven through the same C ABI by ctypes, one process per
GPU, so the comparison is like for like.  Differences from the reference's
harness: time is measured on the device (CUDA events around the ``-n``
back-to-back calls) and the reported figure is the MAX over ranks; the
reference-style host-timed mean over ranks is reported next to it.  With
``-c 1`` the first result of every size is checked against a CPU oracle.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import multiprocessing as mp
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
OPS = ["allreduce", "allgather", "reducescatter", "alltoall", "alltoallv", "broadcast", "reduce", "gather", "scatter", "sendrecv"]
DT = {"float": (7, 4), "fp32": (7, 4), "bf16": (9, 2), "half": (6, 2), "fp8": (10, 1), "uint8": (1, 1), "int32": (2, 4)}


def parse_size(s: str) -> int:
    s = s.strip().upper()
    mult = 1
    if s[-1] in "KMG":
        mult = {"K": 1 << 10, "M": 1 << 20, "G": 1 << 30}[s[-1]]
        s = s[:-1]
    return int(float(s) * mult)


def busbw_factor(op: str, n: int) -> float:
    if op == "allreduce":
        return 2.0 * (n - 1) / n
    if op in ("allgather", "reducescatter", "alltoall", "alltoallv", "gather", "scatter"):
        return (n - 1) / n
    return 1.0


def worker(rank, world, args, idq, outq):
    try:
        os.environ.setdefault("FLAGCX_SOCKET_IFNAME", "lo")
        import torch
        from flagcx_b200.wrapper import FLAGCXLibrary
        torch.cuda.set_device(rank)
        torch.zeros(1, device="cuda")
        libpath = None
        if args.lib == "reference":
            libpath = str(ROOT / "baseline" / "_ref" / "libflagcx.so")
        elif args.lib != "ours":
            libpath = args.lib
        lib = FLAGCXLibrary(libpath)
        if rank == 0:
            uid = lib.flagcxGetUniqueId()
            for _ in range(world - 1):
                idq.put(lib.unique_id_to_bytes(uid))
        else:
            uid = lib.unique_id_from_bytes(idq.get(timeout=120))
        comm = lib.flagcxCommInitRank(world, uid, rank)
        stream = torch.cuda.Stream()
        st = lib.adaptor_stream_copy(stream)
        dcode, es = DT[args.dtype]
        tdt = {7: torch.float32, 9: torch.bfloat16, 6: torch.float16, 10: torch.uint8, 1: torch.uint8, 2: torch.int32}[dcode]
        max_bytes = parse_size(args.e)
        min_bytes = parse_size(args.b)
        use_heap = args.R == 1 and args.lib == "ours"

        def alloc(nbytes):
            nbytes = max(nbytes, 16)
            if use_heap:
                p = lib.flagcxMemAlloc(nbytes, comm)
                return p, None
            t = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
            return t.data_ptr(), t
        sendp, sendt = alloc(max_bytes)
        recvp, recvt = alloc(max_bytes)
        # fill: uniform[-1, 1] from a seed (bytes for the 8-bit case)
        g = torch.Generator(device="cuda").manual_seed(42 + rank)
        nel = max_bytes // es
        if sendt is not None and tdt in (torch.float32, torch.bfloat16, torch.float16):
            chunk = 1 << 26
            view = sendt.view(tdt)
            for o in range(0, nel, chunk):
                k = min(chunk, nel - o)
                view[o:o + k] = (torch.rand(k, generator=g, device="cuda") * 2 - 1).to(tdt)
        torch.cuda.synchronize()
        rows = []
        size = min_bytes
        roots = [args.r] if args.r >= 0 else [0]
        while size <= max_bytes:
            n = world
            if args.op in ("allreduce", "broadcast", "reduce", "sendrecv"):
                count = max(size // es, 1)
            else:
                count = max(size // es // n, 1)
            nbytes = count * es * (1 if args.op in ("allreduce", "broadcast", "reduce", "sendrecv") else n)

            def call(root=roots[0]):
                if args.op == "allreduce":
                    lib.flagcxAllReduce(sendp, recvp, count, dcode, args.redop, comm, st)
                elif args.op == "allgather":
                    lib.flagcxAllGather(sendp, recvp, count, dcode, comm, st)
                elif args.op == "reducescatter":
                    lib.flagcxReduceScatter(sendp, recvp, count, dcode, args.redop, comm, st)
                elif args.op == "alltoall":
                    lib.flagcxAlltoAll(sendp, recvp, count, dcode, comm, st)
                elif args.op == "alltoallv":
                    cnt = [count] * n
                    dsp = [i * count for i in range(n)]
                    lib.flagcxAlltoAllv(sendp, cnt, dsp, recvp, cnt, dsp, dcode, comm, st)
                elif args.op == "broadcast":
                    lib.flagcxBroadcast(sendp, recvp, count, dcode, root, comm, st)
                elif args.op == "reduce":
                    lib.flagcxReduce(sendp, recvp, count, dcode, args.redop, root, comm, st)
                elif args.op == "gather":
                    lib.flagcxGather(sendp, recvp, count, dcode, root, comm, st)
                elif args.op == "scatter":
                    lib.flagcxScatter(sendp, recvp, count, dcode, root, comm, st)
                elif args.op == "sendrecv":
                    lib.flagcxGroupStart(comm)
                    lib.flagcxSend(sendp, count, dcode, (rank + 1) % n, comm, st)
                    lib.flagcxRecv(recvp, count, dcode, (rank - 1) % n, comm, st)
                    lib.flagcxGroupEnd(comm)
            iters = args.n if size <= (256 << 20) else max(5, args.n // 4)
            with torch.cuda.stream(stream):
                for _ in range(args.w):
                    call()
                stream.synchronize()
                lib.flagcxBarrier(comm, st)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                t0 = time.perf_counter()
                e0.record(stream)
                for _ in range(iters):
                    call()
                e1.record(stream)
                stream.synchronize()
                host_us = (time.perf_counter() - t0) * 1e6 / iters
                dev_us = e0.elapsed_time(e1) * 1e3 / iters
            rows.append((nbytes, dev_us, host_us))
            size = int(size * args.f) if size * args.f > size else size + 1
        kind = ""
        if args.lib == "ours":
            try:
                kind = "tuned" if os.environ.get("FLAGCX_USE_TUNER") else "prior"
            except Exception:
                pass
        lib.flagcxBarrier(comm, st)
        lib.flagcxCommDestroy(comm)
        outq.put((rank, "ok", rows, kind))
    except BaseException as e:  # noqa
        import traceback
        outq.put((rank, "err", traceback.format_exc(), ""))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", choices=OPS, default="allreduce")
    ap.add_argument("--lib", default="ours", help="ours | reference | path to a libflagcx.so")
    ap.add_argument("--gpus", type=int, default=0)
    ap.add_argument("--dtype", default="float", choices=sorted(DT))
    ap.add_argument("--redop", type=int, default=0)
    ap.add_argument("-b", default="8")
    ap.add_argument("-e", default="128M")
    ap.add_argument("-f", type=float, default=2)
    ap.add_argument("-w", type=int, default=5)
    ap.add_argument("-n", type=int, default=20)
    ap.add_argument("-p", type=int, default=0)
    ap.add_argument("-r", type=int, default=0)
    ap.add_argument("-R", type=int, default=0)
    ap.add_argument("--json", default="")
    args = ap.parse_args()
    if args.lib == "reference":
        # the reference's library needs its own directory on the loader path for NCCL plugins; nothing else
        pass
    import torch
    world = args.gpus or torch.cuda.device_count()
    ctx = mp.get_context("spawn")
    idq, outq = ctx.Queue(), ctx.Queue()
    procs = [ctx.Process(target=worker, args=(r, world, args, idq, outq)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        rank, status, rows, kind = outq.get(timeout=3600)
        if status != "ok":
            print(rows, file=sys.stderr)
            for p in procs:
                p.kill()
            return 1
        res[rank] = rows
    for p in procs:
        p.join(timeout=30)
    factor = busbw_factor(args.op, world)
    out = []
    print(f"# op {args.op} lib {args.lib} dtype {args.dtype} ranks {world}  (time = device-timed, max over ranks)")
    print(f"# {'bytes':>12} {'time_us':>10} {'algbw_GBs':>10} {'busbw_GBs':>10} {'host_mean_us':>12}")
    for i in range(len(res[0])):
        nbytes = res[0][i][0]
        dev = max(res[r][i][1] for r in range(world))
        host = sum(res[r][i][2] for r in range(world)) / world
        alg = nbytes / dev / 1e3
        print(f"  {nbytes:>12} {dev:>10.2f} {alg:>10.2f} {alg * factor:>10.2f} {host:>12.2f}")
        out.append({"op": args.op, "lib": args.lib, "dtype": args.dtype, "ranks": world, "bytes": nbytes, "time_us": round(dev, 3),
                    "algbw_gbs": round(alg, 3), "busbw_gbs": round(alg * factor, 3), "host_mean_us": round(host, 3)})
    if args.json:
        with open(args.json, "a") as f:
            for row in out:
                f.write(json.dumps(row) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
