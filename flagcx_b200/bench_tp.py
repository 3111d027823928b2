"""Tensor-parallel layer benchmark: Llama-3-8B-shaped transformer layer,
8192 tokens x hidden 4096, FFN 14336 and 32/8 heads sharded over the ranks,
sequence-parallel (all-gather on entry, reduce-scatter on exit of each block).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m flagcx_b200.bench_tp --impl fused

``--impl fused``   this library's one-kernel all-gather->GEMM and GEMM->reduce-scatter;
``--impl unfused`` this library's collectives followed by cuBLAS GEMMs;
``--impl reference`` the reference plugin's collectives (NCCL) followed by cuBLAS GEMMs.
``--mode layer`` times a whole layer forward + backward (attention included) in the same three arms.
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


def _unfused_linears(all_gather, reduce_scatter, world):
    """Differentiable column- and row-parallel linears made of a collective and a library GEMM, forward and
    backward: what a user of the reference runs (its all-gather / reduce-scatter, then torch.matmul)."""

    class Col(torch.autograd.Function):
        @staticmethod
        def forward(ctx, x_local, w):
            full = torch.empty(x_local.shape[0] * world, x_local.shape[1], dtype=x_local.dtype, device=x_local.device)
            all_gather(full, x_local)
            ctx.save_for_backward(full, w)
            return full @ w.t()

        @staticmethod
        def backward(ctx, dy):
            full, w = ctx.saved_tensors
            dy = dy.contiguous()
            dfull = dy @ w
            dx = torch.empty(dfull.shape[0] // world, dfull.shape[1], dtype=dfull.dtype, device=dfull.device)
            reduce_scatter(dx, dfull)
            return dx, dy.t() @ full

    class Row(torch.autograd.Function):
        @staticmethod
        def forward(ctx, a, w):
            ctx.save_for_backward(a, w)
            part = a @ w.t()
            out = torch.empty(a.shape[0] // world, w.shape[0], dtype=a.dtype, device=a.device)
            reduce_scatter(out, part)
            return out

        @staticmethod
        def backward(ctx, dz):
            a, w = ctx.saved_tensors
            dz = dz.contiguous()
            dfull = torch.empty(dz.shape[0] * world, dz.shape[1], dtype=dz.dtype, device=dz.device)
            all_gather(dfull, dz)
            return dfull @ w, dfull.t() @ a

    return Col.apply, Row.apply


def layer_bench(args, rank, world, lr, dev):
    """One Llama-3-8B-shaped layer, forward + backward, tensor parallel with sequence parallelism: RMSNorm,
    all-gather -> QKV GEMM, causal grouped-query attention on the local heads (PyTorch's library flash attention in
    every arm), output GEMM -> reduce-scatter, residual, RMSNorm, all-gather -> up/gate GEMM, SiLU x gate, down GEMM ->
    reduce-scatter, residual; the backward pass runs the mirrored collectives and the weight-gradient GEMMs."""
    import torch.nn.functional as F
    T, H = args.tokens, args.hidden
    hd = H // args.heads
    nq, nkv = args.heads // world, max(1, args.kv_heads // world)
    ffn_n = args.ffn // world
    torch.manual_seed(1 + rank)
    mk = lambda *sh: (torch.randn(*sh, device=dev) * 0.02).bfloat16().requires_grad_(True)  # noqa: E731
    w_qkv, w_o, w_ug, w_down = mk((nq + 2 * nkv) * hd, H), mk(H, nq * hd), mk(2 * ffn_n, H), mk(H, ffn_n)
    g1, g2 = torch.ones(H, device=dev, dtype=torch.bfloat16, requires_grad=True), torch.ones(H, device=dev, dtype=torch.bfloat16, requires_grad=True)
    x_local = (torch.randn(T // world, H, device=dev)).bfloat16().requires_grad_(True)
    grad_out = (torch.randn(T // world, H, device=dev) * 0.01).bfloat16()
    tp = None
    if args.impl == "fused":
        import flagcx_b200
        from flagcx_b200.parallel.tp import TensorParallelContext, column_parallel_linear, row_parallel_linear
        comm = flagcx_b200.get_comm_handle(None, dev)
        tp = TensorParallelContext(comm, world, rank, max_rows=T, max_k=H, max_n=H, comm_ctas=args.comm_ctas or None, device=dev, buffers=4)
        col = lambda x, w: column_parallel_linear(x, w, tp)  # noqa: E731
        row = lambda a, w: row_parallel_linear(a, w, tp)  # noqa: E731
    elif args.impl == "unfused":
        import flagcx_b200
        nat = flagcx_b200.native()
        comm = flagcx_b200.get_comm_handle(None, dev)
        col, row = _unfused_linears(lambda out, x: nat.comm_all_gather(comm, x, out), lambda out, x: nat.comm_reduce_scatter(comm, x, out, 0), world)
    else:
        col, row = _unfused_linears(lambda out, x: dist.all_gather_into_tensor(out, x), lambda out, x: dist.reduce_scatter_tensor(out, x), world)

    def step():
        h = F.rms_norm(x_local, (H,), g1)
        qkv = col(h, w_qkv).view(1, T, nq + 2 * nkv, hd)
        q, k, v = qkv[:, :, :nq], qkv[:, :, nq:nq + nkv], qkv[:, :, nq + nkv:]
        att = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True, enable_gqa=True)
        x1 = x_local + row(att.transpose(1, 2).reshape(T, nq * hd), w_o)
        ug = col(F.rms_norm(x1, (H,), g2), w_ug)
        out = x1 + row(F.silu(ug[:, :ffn_n]) * ug[:, ffn_n:], w_down)
        out.backward(grad_out)
        for t in (w_qkv, w_o, w_ug, w_down, g1, g2, x_local):
            t.grad = None
        return out

    for _ in range(3):
        out = step()
    torch.cuda.synchronize()
    dist.barrier(device_ids=[lr]) if args.impl != "reference" else dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        out = step()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.iters], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    us = float(t.item()) * 1e3
    if tp is not None:
        tp.check()
    chk = torch.tensor([float(out.float().abs().mean())], dtype=torch.float64)
    dist.all_reduce(chk)
    peaks = ROOT / "MEASURED_PEAKS.json"
    gemm_peak = json.loads(peaks.read_text())["bf16_tflops"] * 1e12 if peaks.exists() else 1.59e15
    gemm_flops = 3 * 2.0 * T * H * ((nq + 2 * nkv) * hd + nq * hd + 2 * ffn_n + ffn_n)
    attn_flops = 3.5 * 2.0 * 2 * nq * T * T * hd / 2
    link_bytes = 8 * (world - 1) * (T // world) * H * 2
    roof = max((gemm_flops + attn_flops) / gemm_peak, link_bytes / 770e9) * 1e6
    if rank == 0:
        print(json.dumps({"bench": "tp_layer_fwd_bwd", "impl": args.impl, "n_gpus": world, "tokens": T, "hidden": H, "ffn": args.ffn,
                          "heads_per_rank": nq, "kv_heads_per_rank": nkv, "us": round(us, 1), "roofline_us": round(roof, 1),
                          "fraction_of_roofline": round(roof / us, 3), "checksum": float(chk.item()) / world,
                          "peak": "of measured" if peaks.exists() else "of fallback"}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=["projections", "layer"], default="projections",
                    help="projections: the four fused forward ops one by one; layer: a whole layer forward + backward")
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
    if args.mode == "layer":
        layer_bench(args, rank, world, lr, dev)
        dist.destroy_process_group()
        return
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
