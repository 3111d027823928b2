"""Expert-parallel MoE layer benchmark: Mixtral-shaped (hidden 4096, expert FFN
14336, top-2), one expert per rank, 8192 bf16 tokens per rank, router logits
drawn from N(0,1) so the all-to-all-v splits vary from rank to rank.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m flagcx_b200.bench_ep --impl fused

``--impl fused``     dispatch kernel -> tcgen05 GEMMs with device-side row counts -> combine fused into the down GEMM;
``--impl unfused``   this library's all-to-all-v with host counts + cuBLAS GEMMs;
``--impl reference`` the reference plugin's all-to-all-v (NCCL) + cuBLAS GEMMs.
Device-timed, max over ranks.  The roofline is the slower of the expert FLOPs at the measured GEMM peak and the
bytes each GPU must send over NVLink (dispatch + combine) at 770 GB/s per direction."""
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
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--dispatch-ctas", type=int, default=64)
    ap.add_argument("--save-dir", default="", help="leave rank 0's output here and compare with the reference arm's, if it is there")
    args = ap.parse_args()
    rank, world, lr = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    os.environ.setdefault("FLAGCX_SOCKET_IFNAME", "lo")
    os.environ.setdefault("FLAGCX_HEAP_USER_BYTES", "2G")
    if args.impl == "reference" and os.environ.get("FLAGCX_REF_REEXEC") != "1":
        env = dict(os.environ)
        env["LD_LIBRARY_PATH"] = str(ROOT / "baseline" / "_ref") + os.pathsep + env.get("LD_LIBRARY_PATH", "")
        env["FLAGCX_REF_REEXEC"] = "1"
        os.execve(sys.executable, [sys.executable, "-m", "flagcx_b200.bench_ep"] + sys.argv[1:], env)
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline" / "_ref"))
    import flagcx  # noqa: F401  (this library's shim, or the reference plugin)
    dist.init_process_group("cpu:gloo,cuda:flagcx", rank=rank, world_size=world)
    T, H, F, K = args.tokens, args.hidden, args.ffn, min(args.topk, max(world, 1))
    torch.manual_seed(11 + rank)
    x = torch.randn(T, H, device=dev).bfloat16()
    logits = torch.randn(T, world, device=dev)
    topk_w, topk_idx = torch.topk(torch.softmax(logits, -1), K, dim=-1)
    topk_idx = topk_idx.int().contiguous()
    topk_w = topk_w.float().contiguous()
    w1 = (torch.randn(2 * F, H, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(H, F, device=dev) * 0.02).bfloat16()

    if args.impl in ("fused", "unfused"):
        import flagcx_b200
        from flagcx_b200.parallel.ep import ExpertParallelContext
        comm = flagcx_b200.get_comm_handle(None, dev)
        ep = ExpertParallelContext(comm, world, rank, T, H, F, K, dispatch_ctas=args.dispatch_ctas, device=dev)
        step = (lambda: ep.forward(x, topk_idx, topk_w, w1, w2)) if args.impl == "fused" else (lambda: ep.unfused_forward(x, topk_idx, topk_w, w1, w2))
    else:
        def step():
            flat = topk_idx.flatten().long()
            order = torch.argsort(flat, stable=True)
            send = x[order // K]
            sc = torch.bincount(flat, minlength=world)
            rc = torch.empty_like(sc)
            dist.all_to_all_single(rc, sc)
            scl, rcl = sc.cpu().tolist(), rc.cpu().tolist()
            recv = torch.empty(sum(rcl), H, dtype=x.dtype, device=dev)
            dist.all_to_all_single(recv, send, rcl, scl)
            gu = recv @ w1.t()
            h = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
            y = h @ w2.t()
            back = torch.empty_like(send)
            dist.all_to_all_single(back, y, scl, rcl)
            ret = torch.empty_like(back)
            ret[order] = back
            return (ret.view(T, K, H).float() * topk_w.unsqueeze(2)).sum(1).to(x.dtype)

    for _ in range(3):
        out = step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.iters):
        out = step()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.iters], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    agree = None
    if args.impl in ("fused", "unfused"):
        ep.check()
        # the two paths of this library must agree element by element (a mean over random data would hide a misrouted row)
        other = ep.unfused_forward(x, topk_idx, topk_w, w1, w2) if args.impl == "fused" else ep.forward(x, topk_idx, topk_w, w1, w2)
        torch.cuda.synchronize()
        agree = float(((out.float() - other.float()).abs().max() / other.float().abs().max()).item())
    # Across arms: every arm leaves rank 0's output next to the others (same seeds, same inputs), and compares it
    # element by element with what the reference arm left there, when that arm ran before on this machine.
    vs_ref = None
    if rank == 0 and args.save_dir:
        os.makedirs(args.save_dir, exist_ok=True)
        torch.save(out.float().cpu(), os.path.join(args.save_dir, f"ep_out_{args.impl}_{world}.pt"))
        ref_file = os.path.join(args.save_dir, f"ep_out_reference_{world}.pt")
        if args.impl != "reference" and os.path.exists(ref_file):
            ref = torch.load(ref_file)
            vs_ref = float(((out.float().cpu() - ref).abs().max() / ref.abs().max()).item())
    # rows this rank's expert processed, and bytes this rank had to send to other ranks (there and back)
    rows = torch.tensor([float((topk_idx == r).sum().item()) for r in range(world)], dtype=torch.float64)
    remote = float(rows.sum() - rows[rank]) * H * 2
    dist.all_reduce(rows)
    my_rows = float(rows[rank])
    flops = 2.0 * my_rows * H * 3 * F
    worst = torch.tensor([flops, remote], dtype=torch.float64)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    peaks = ROOT / "MEASURED_PEAKS.json"
    gemm_peak = json.loads(peaks.read_text())["bf16_tflops"] * 1e12 if peaks.exists() else 1.59e15
    roof_ms = max(float(worst[0]) / gemm_peak, 2 * float(worst[1]) / 770e9) * 1e3
    if rank == 0:
        print(json.dumps({"bench": "ep_moe_layer", "impl": args.impl, "n_gpus": world, "tokens_per_rank": T, "hidden": H, "ffn": F,
                          "topk": K, "ms": round(ms, 3), "tokens_per_s": round(world * T / ms * 1e3, 1), "roofline_ms": round(roof_ms, 3),
                          "fraction_of_roofline": round(roof_ms / ms, 3), "checksum": float(out.float().abs().mean().item()), "max_rel_diff_vs_other_path": agree, "max_rel_diff_vs_reference_arm": vs_ref,
                          "peak": "of measured" if peaks.exists() else "of fallback"}))
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
