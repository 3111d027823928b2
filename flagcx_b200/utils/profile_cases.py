"""Small, self-contained workloads for profiling one kernel at a time.

    python -m flagcx_b200.utils.profile_cases --case adamw

Each case touches more than the 126 MB L2 but holds at most a few GB, runs a
couple of warm-up launches and three measured ones, and prints the
CUDA-event time with the achieved fraction of the measured HBM copy rate
(MEASURED_PEAKS.json, else 6.65 TB/s).  Cases: adamw, cross_entropy,
layernorm_fwd, layernorm_bwd, bias_gelu, emu_allreduce (8 emulated ranks,
two-shot kernel, one cooperative launch on this GPU), emu_allgather, gemm / gemm_one_cta
(tcgen05 GEMM, against the measured cuBLAS rate), gemm_fp8 (block-scaled e4m3 GEMM), moe_dispatch and moe_layer
(expert-parallel kernels on a one-rank communicator), emu_allreduce_zc / emu_allreduce_ll / emu_sendrecv (zero-copy,
LL and grouped send/recv kernels on emulated ranks), gemm_dgrad / gemm_wgrad (transposed-operand GEMMs), gemm_ag /
gemm_rs (fused all-gather / reduce-scatter GEMMs on a one-rank communicator)."""
from __future__ import annotations

import argparse
import ctypes
import json
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent.parent


def hbm_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return json.loads(p.read_text())["hbm_gbs"] * 1e9, "of measured"
    return 6.65e12, "of fallback"


def timed(fn, reps=3, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    best = 1e9
    for _ in range(reps):
        flush.zero_()  # evict L2 between measurements
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", required=True)
    args = ap.parse_args()
    import flagcx_b200
    nat = flagcx_b200.native()
    peak, label = hbm_peak()
    torch.manual_seed(0)
    if args.case == "adamw":
        n = 64 << 20
        master = torch.randn(n, device="cuda")
        param, grad = master.bfloat16(), torch.randn(n, device="cuda").bfloat16()
        m, v = torch.zeros_like(master), torch.zeros_like(master)
        ms = timed(lambda: nat.adamw_(master, param, grad, m, v, 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, 1.0, True))
        nbytes = n * (4 * 3 * 2 + 2 + 2 + 2)  # master/m/v read+write, grad read+clear, param write
    elif args.case == "cross_entropy":
        M, V, Vp = 2048, 50257, 50304
        logits = torch.randn(M, Vp, device="cuda").bfloat16()
        tgt = torch.randint(0, V, (M,), device="cuda")
        ms = timed(lambda: nat.cross_entropy_(logits, tgt, V, 1.0 / M))
        nbytes = M * Vp * 2 * 2  # algorithmic: read once, write once (the two extra read passes should hit L2)
    elif args.case in ("layernorm_fwd", "layernorm_bwd"):
        M, C = 65536, 1024
        x, d = torch.randn(M, C, device="cuda").bfloat16(), torch.randn(M, C, device="cuda").bfloat16()
        g, b = torch.ones(C, device="cuda").bfloat16(), torch.zeros(C, device="cuda").bfloat16()
        if args.case == "layernorm_fwd":
            ms = timed(lambda: nat.layernorm_fwd(x, d, g, b, 1e-5))
            nbytes = M * C * 2 * 4
        else:
            res, y, mean, rstd = nat.layernorm_fwd(x, d, g, b, 1e-5)
            dy = torch.randn_like(y)
            ms = timed(lambda: nat.layernorm_bwd(dy, res, g, mean, rstd, d))
            nbytes = M * C * 2 * 4
    elif args.case == "bias_gelu":
        M, C = 32768, 4096
        x, b = torch.randn(M, C, device="cuda").bfloat16(), torch.randn(C, device="cuda").bfloat16()
        ms = timed(lambda: nat.bias_gelu_fwd(x, b))
        nbytes = M * C * 2 * 2
    elif args.case in ("emu_allreduce", "emu_allgather"):
        from flagcx_b200.wrapper import FLAGCXLibrary
        lib = FLAGCXLibrary()
        n = 8
        emu = ctypes.c_void_p()
        lib.call("flagcxEmuCreate", ctypes.byref(emu), n, 64 << 20)
        arr = ctypes.c_void_p * n
        if args.case == "emu_allreduce":
            count = 8 << 20  # 32 MiB of fp32 per rank
            xs = [torch.randn(count, device="cuda") for _ in range(n)]
            ys = [torch.empty_like(x) for x in xs]
            op, kind = 6, b"ar_twoshot"
            nbytes = n * count * 4 * (1 + 1 + 2.0 * (n - 1) / n * 2)  # read+write own, slices pushed and read back twice
        else:
            count = 1 << 20
            xs = [torch.randn(count, device="cuda") for _ in range(n)]
            ys = [torch.empty(count * n, device="cuda") for _ in range(n)]
            op, kind = 7, b"ag"
            nbytes = n * count * 4 * (1 + 2 * (n - 1) + n)
        s = arr(*[x.data_ptr() for x in xs])
        r = arr(*[y.data_ptr() for y in ys])
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        ms = timed(lambda: lib.call("flagcxEmuCollective", emu, op, kind, 16, s, r, count, 7, 7, ctypes.c_float(1.0), 0, 0, None, st))
        lib.call("flagcxEmuDestroy", emu)
    elif args.case in ("emu_allreduce_zc", "emu_allreduce_ll", "emu_sendrecv"):
        # the zero-copy all-reduce (plain peer loads, 16 in flight per thread: one GPU has no switch to reduce in),
        # the LL all-reduce at 4 KiB, and the grouped send/recv kernel, each as 8 (2) emulated ranks in one launch
        from flagcx_b200.wrapper import FLAGCXLibrary
        lib = FLAGCXLibrary()
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        if args.case == "emu_sendrecv":
            n, nbytes_each = 2, 64 << 20
            emu = ctypes.c_void_p()
            lib.call("flagcxEmuCreate", ctypes.byref(emu), n, 1 << 20)
            sb = [torch.randint(0, 255, (nbytes_each,), device="cuda", dtype=torch.uint8) for _ in range(n)]
            rb = [torch.empty_like(t) for t in sb]
            k = n
            args_ = (emu, k, (ctypes.c_int * k)(*range(n)), (ctypes.c_int * k)(*[(r + 1) % n for r in range(n)]),
                     (ctypes.c_void_p * k)(*[t.data_ptr() for t in sb]), (ctypes.c_void_p * k)(*[t.data_ptr() for t in rb]),
                     (ctypes.c_size_t * k)(*[nbytes_each] * k), 16, st)
            ms = timed(lambda: lib.call("flagcxEmuSendRecv", *args_))
            nbytes = n * nbytes_each * 4  # staged: read + write into the slot, read + write out of it
        else:
            n = 8
            emu = ctypes.c_void_p()
            lib.call("flagcxEmuCreate", ctypes.byref(emu), n, 1 << 20)
            arr = ctypes.c_void_p * n
            zc = args.case == "emu_allreduce_zc"
            count = (8 << 20) if zc else 1024
            xs = [torch.randn(count, device="cuda") for _ in range(n)]
            ys = [torch.empty_like(x) for x in xs]
            s, r = arr(*[x.data_ptr() for x in xs]), arr(*[y.data_ptr() for y in ys])
            kind, ctas = (b"ar_zc", 16) if zc else (b"ar_ll", 1)
            ms = timed(lambda: lib.call("flagcxEmuCollective", emu, 6, kind, ctas, s, r, count, 7, 7, ctypes.c_float(1.0), 0, 0, None, st))
            nbytes = n * count * 4 * 2 if zc else n * count * 4 * (1 + 2 * (n - 1) * 2 + 1)  # zc: every element read once and written once per rank
        lib.call("flagcxEmuDestroy", emu)
    elif args.case in ("gemm_dgrad", "gemm_wgrad", "gemm_ag", "gemm_rs"):
        # the backward GEMMs of a linear layer (operands read transposed in place; the weight gradient splits K) and
        # the fused all-gather / reduce-scatter forms on a one-rank communicator (comm CTAs, flags, staging and tail
        # reduction all run, with this GPU as its own peer)
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        pk = ROOT / "MEASURED_PEAKS.json"
        tf_peak = json.loads(pk.read_text())["bf16_tflops"] if pk.exists() else 1590.0
        if args.case in ("gemm_dgrad", "gemm_wgrad"):
            T, O, I = 8192, 4096, 4096
            dy = (torch.randn(T, O, device="cuda") * 0.1).bfloat16()
            w = (torch.randn(O, I, device="cuda") * 0.1).bfloat16()
            x = (torch.randn(T, I, device="cuda") * 0.1).bfloat16()
            if args.case == "gemm_dgrad":
                ms = timed(lambda: nat.gemm(dy, w, False, True, None, 0, err))
            else:
                ms = timed(lambda: nat.gemm(dy, x, True, True, None, 0, err))
            flops = 2.0 * T * O * I
        else:
            import os
            os.environ.setdefault("FLAGCX_HEAP_USER_BYTES", "1G")
            from flagcx_b200.parallel.tp import TensorParallelContext
            from flagcx_b200.wrapper import FLAGCXLibrary
            lib = FLAGCXLibrary()
            comm = lib.flagcxCommInitRank(1, lib.flagcxGetUniqueId(), 0)
            M, N, K = 8192, 4096, 4096
            tp = TensorParallelContext(comm.value, 1, 0, max_rows=M, max_k=K, max_n=N, comm_ctas=4)
            a = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
            b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
            ms = timed((lambda: tp.ag_gemm(a, b)) if args.case == "gemm_ag" else (lambda: tp.gemm_rs(a, b)))
            torch.cuda.synchronize()
            tp.check()
            del tp
            lib.flagcxCommDestroy(comm)
            flops = 2.0 * M * N * K
        tf = flops / (ms * 1e-3) / 1e12
        print(json.dumps({"case": args.case, "ms": round(ms, 4), "tflops": round(tf, 1), "fraction_of_gemm_peak": round(tf / tf_peak, 3),
                          "peak": label, "err": int(err.item())}))
        return
    elif args.case == "gemm_fp8":
        M, N, K = 8192, 4096, 4096
        a = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
        b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
        q, sa = nat.quant_fp8_act(a)
        qw, sb = nat.quant_fp8_weight(b)
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        ms = timed(lambda: nat.gemm_fp8_nt(q, sa, qw, sb, err))
        tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
        print(json.dumps({"case": "gemm_fp8", "shape": [M, N, K], "ms": round(ms, 4), "tflops": round(tf, 1),
                          "fraction_of_nominal_fp8_peak": round(tf / 4500.0, 3), "err": int(err.item())}))
        return
    elif args.case in ("gemm", "gemm_one_cta"):
        # tensor-core bound: reported against the measured cuBLAS bf16 rate instead of the copy rate.
        # "gemm": the kernel the launcher picks for this shape (CTA pairs); "gemm_one_cta": the 128 x 256 kernel
        M, N, K = 8192, 4096, 4096
        a = (torch.randn(M, K, device="cuda") * 0.1).bfloat16()
        b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
        err = torch.zeros(1, dtype=torch.int32, device="cuda")
        ms = timed(lambda: nat.gemm(a, b, False, False, None, 0, err, 0 if args.case == "gemm_one_cta" else -1))
        pk = ROOT / "MEASURED_PEAKS.json"
        tf_peak = json.loads(pk.read_text())["bf16_tflops"] if pk.exists() else 1590.0
        tf = 2.0 * M * N * K / (ms * 1e-3) / 1e12
        print(json.dumps({"case": args.case, "shape": [M, N, K], "ms": round(ms, 4), "tflops": round(tf, 1),
                          "fraction_of_gemm_peak": round(tf / tf_peak, 3), "peak": label, "err": int(err.item())}))
        return
    elif args.case in ("moe_dispatch", "moe_layer"):
        # one-rank communicator: the dispatch kernel (count, exchange, push), the device-row-count GEMMs,
        # the ROWMAP epilogue and the combine kernel all run, with this GPU as its own peer
        import os
        os.environ.setdefault("FLAGCX_HEAP_USER_BYTES", "1G")
        from flagcx_b200.parallel.ep import ExpertParallelContext
        from flagcx_b200.wrapper import FLAGCXLibrary
        lib = FLAGCXLibrary()
        comm = lib.flagcxCommInitRank(1, lib.flagcxGetUniqueId(), 0)
        T, H, F, K = 8192, 4096, 2048, 2
        ep = ExpertParallelContext(comm.value, 1, 0, T, H, F, K)
        x = torch.randn(T, H, device="cuda").bfloat16()
        idx = torch.zeros(T, K, dtype=torch.int32, device="cuda")
        wts = torch.rand(T, K, device="cuda")
        w1 = (torch.randn(2 * F, H, device="cuda") * 0.02).bfloat16()
        w2 = (torch.randn(H, F, device="cuda") * 0.02).bfloat16()
        if args.case == "moe_dispatch":
            state = {"calls": 0}

            def disp():
                par, epoch = state["calls"] & 1, (state["calls"] >> 1) + 1
                state["calls"] += 1
                nat.moe_dispatch(comm.value, x, idx, ep.count_mat[par], ep.count_flags[par], ep.recv[par], ep.info[par], ep.disp_done[par],
                                 epoch, ep.slot, ep.local_counts, ep.recv_total, ep.err, ep.dispatch_ctas)
            ms = timed(disp)
            nbytes = T * K * H * 2 * 2  # every (token, choice) row read once and written once
        else:
            ms = timed(lambda: ep.forward(x, idx, wts, w1, w2))
            nbytes = T * K * H * 2 * 2
        torch.cuda.synchronize()
        ep.check()
        del ep
        lib.flagcxCommDestroy(comm)
    else:
        raise SystemExit(f"unknown case {args.case}")
    gbs = nbytes / (ms * 1e-3)
    print(json.dumps({"case": args.case, "ms": round(ms, 4), "algorithmic_GBs": round(gbs / 1e9, 1), "fraction_of_hbm": round(gbs / peak, 3),
                      "peak": label}))


if __name__ == "__main__":
    main()
