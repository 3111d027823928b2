"""Tensor-parallel layer benchmark: Llama-3-8B-shaped transformer layer,
8192 tokens x hidden 4096, FFN 14336 and 32/8 heads sharded over the ranks,
sequence-parallel (all-gather on entry, reduce-scatter on exit of each block).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m flagcx_b200.bench_tp --impl fused

``--impl fused``   this library's one-kernel all-gather->GEMM and GEMM->reduce-scatter;
``--impl unfused`` this library's collectives followed by cuBLAS GEMMs;
``--impl reference`` the reference plugin's collectives (NCCL) followed by cuBLAS GEMMs.
Times the four projection GEMMs with their collectives (QKV, attention output, FFN up+gate, FFN down),
device-timed, max over ranks, and reports each against its roofline: the slower of FLOPs at the measured
GEMM peak and NVLink bytes at 770 GB/s per direction."""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--impl", choices=["fused", "unfused", "reference"], default="fused")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--ffn", type=int, default=14336)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--comm-ctas", type=int, default=0, help="0: sized per call")
    args = ap.parse_args()
    rank, world, lr = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("FLAGCX_SOCKET_IFNAME", "lo")
    if args.impl == "reference" and os.environ.get("FLAGCX_REF_REEXEC") != "1":
        env = dict(os.environ)
        env["LD_LIBRARY_PATH"] = str(ROOT / "baseline" / "_ref") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
        env["FLAGCX_REF_REEXEC"] = "1"
        os.execve(sys.executable, [sys.executable, "-m", "flagcx_b200.bench_tp"] + sys.argv[1:], env)
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
        import flagcx  # noqa: F401  (reference plugin)
    else:
        import flagcx  # noqa: F401
    dist.init_process_group("cpu:gloo,cuda:flagcx", rank=rank, world_size=world)
    T, H = args.tokens, args.hidden
    hd = H // args.heads
    qkv_n = (args.heads + 2 * args.kv_heads) * hd // world
    ffn_n = args.ffn // world
    torch.manual_seed(1 + rank)
    x_local = (torch.randn(T // world, H, device=dev) * 0.02).bfloat16()
    w_qkv = (torch.randn(qkv_n, H, device=dev) * 0.02).bfloat16()
    w_o = (torch.randn(H, args.heads * hd // world, device=dev) * 0.02).bfloat16()
    w_up = (torch.randn(2 * ffn_n, H, device=dev) * 0.02).bfloat16()
    w_down = (torch.randn(H, ffn_n, device=dev) * 0.02).bfloat16()
    attn_out = (torch.randn(T, args.heads * hd // world, device=dev) * 0.02).bfloat16()
    ffn_act = (torch.randn(T, ffn_n, device=dev) * 0.02).bfloat16()
    if args.impl in ("fused", "unfused"):
        import flagcx_b200
        from flagcx_b200.parallel.tp import TensorParallelContext
        comm = flagcx_b200.get_comm_handle(None, dev)
        tp = TensorParallelContext(comm, world, rank, max_rows=T, max_k=H, max_n=H, comm_ctas=args.comm_ctas or None, device=dev)
        if args.impl == "fused":
            ag = lambda x, w: tp.ag_gemm(x, w)  # noqa: E731
            rs = lambda a, w: tp.gemm_rs(a, w)  # noqa: E731
        else:
            ag, rs = tp.unfused_ag_gemm, tp.unfused_gemm_rs
    else:
        def ag(x, w):
            full = torch.empty(x.shape[0] * world, x.shape[1], dtype=x.dtype, device=x.device)
            dist.all_gather_into_tensor(full, x)
            return full @ w.t()

        def rs(a, w):
            part = a @ w.t()
            out = torch.empty(a.shape[0] // world, w.shape[0], dtype=a.dtype, device=a.device)
            dist.reduce_scatter_tensor(out, part)
            return out
    ops = [("qkv: AG+GEMM", lambda: ag(x_local, w_qkv), 2.0 * T * H * qkv_n, (world - 1) * (T // world) * H * 2),
           ("attn_out: GEMM+RS", lambda: rs(attn_out, w_o), 2.0 * T * (args.heads * hd // world) * H, (world - 1) * (T // world) * H * 2),
           ("ffn_up_gate: AG+GEMM", lambda: ag(x_local, w_up), 2.0 * T * H * 2 * ffn_n, (world - 1) * (T // world) * H * 2),
           ("ffn_down: GEMM+RS", lambda: rs(ffn_act, w_down), 2.0 * T * ffn_n * H, (world - 1) * (T // world) * H * 2)]
    peaks = ROOT / "MEASURED_PEAKS.json"
    gemm_peak = json.loads(peaks.read_text())["bf16_tflops"] * 1e12 if peaks.exists() else 1.59e15
    rows = []
    total = 0.0
    for name, fn, flops, link_bytes in ops:
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        dist.barrier(device_ids=[lr]) if args.impl != "reference" else dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / args.iters], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item()) * 1e3
        roof = max(flops / gemm_peak, link_bytes / 770e9) * 1e6
        rows.append({"op": name, "us": round(us, 1), "roofline_us": round(roof, 1), "fraction_of_roofline": round(roof / us, 3),
                     "tflops": round(flops / us / 1e6, 1)})
        total += us
    if args.impl in ("fused", "unfused"):
        torch.cuda.synchronize()
        tp.check()
    if rank == 0:
        print(json.dumps({"bench": "tp_layer_projections", "impl": args.impl, "n_gpus": world, "tokens": T, "hidden": H, "ffn": args.ffn,
                          "total_us": round(total, 1), "ops": rows, "peak": "of measured" if peaks.exists() else "of fallback"}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
