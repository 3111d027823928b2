"""Offline tuning: measure every kernel variant of every collective on this machine and write the table the
library loads with ``FLAGCX_TUNER_CACHE``.

    python -m flagcx_b200.tools.tune --gpus 8 --out tuner_8gpu.json
    FLAGCX_TUNER_CACHE=tuner_8gpu.json <any program using the library>

For each (operation, message size) every legal candidate (kernel kind x CTA count, and the pipeline sub-chunk
size of the staged kinds at large sizes) is pinned and timed on the device, the slowest rank's time counts, and
the fastest candidate of each size bucket goes into the table: by default inside one set of rank processes
(the perf binary's ``-T 1`` mode, seconds for a whole sweep), with ``--per-process`` one process per candidate.
A table named ``<gpu model>_<n>gpu.json`` under ``flagcx_b200/lib/tuned`` is loaded by default on such a machine.  The reference tunes online only and forgets the result at exit
(flagcx/core/flagcx_tuner.cc:330-341); the online search exists here too (``FLAGCX_USE_TUNER=1``).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent.parent

# flagcxCommOp_t values and the perf binary's operation names
OPS = {"broadcast": 2, "gather": 3, "scatter": 4, "reduce": 5, "allreduce": 6, "allgather": 7, "reducescatter": 8, "alltoall": 9}
# operations whose tuner key is the per-rank piece, while the perf binary reports the whole buffer
PER_RANK = {"gather", "scatter", "allgather", "reducescatter", "alltoall"}
LL_MAX = 32768

# kind -> (smallest, largest) payload in bytes of the tuner key for which the kind may run
CANDIDATES = {
    "allreduce": {"ar_ll": (1, LL_MAX), "ar_oneshot": (1, 8 << 20), "ar_twoshot": (2049, None), "ar_nvls": (4096, None)},
    "allgather": {"move_ll": (1, LL_MAX), "ag": (1, None), "ag_nvls": (4096, None)},
    "reducescatter": {"rs_ll": (1, LL_MAX), "rs": (1, None), "rs_nvls": (4096, None)},
    "broadcast": {"move_ll": (1, LL_MAX), "bcast": (1, None)},
    "reduce": {"reduce_ll": (1, LL_MAX), "reduce": (1, None)},
    "gather": {"move_ll": (1, LL_MAX), "gather": (1, None)},
    "scatter": {"move_ll": (1, LL_MAX), "scatter": (1, None)},
    "alltoall": {"move_ll": (1, LL_MAX), "a2a": (1, None)},
}
LL_KINDS = {"ar_ll", "move_ll", "rs_ll", "reduce_ll"}


def bucket(nbytes: int) -> int:
    """The library's size bucket: smallest l with 2**l >= bytes."""
    l = 0
    while (1 << l) < nbytes and l < 62:
        l += 1
    return l


def key_bytes(op: str, total_bytes: int, nranks: int) -> int:
    return total_bytes // nranks if op in PER_RANK else total_bytes


def legal(op: str, kind: str, kbytes: int, multicast: bool) -> bool:
    lo, hi = CANDIDATES[op][kind]
    if "nvls" in kind and not multicast:
        return False
    return kbytes >= lo and (hi is None or kbytes <= hi)


def cta_choices(kind: str):
    return (1, 2, 4) if kind in LL_KINDS else (8, 32, 64, 128)


def build_cache(rows, nranks: int):
    """rows: dicts with op, kind, nctas, bytes (perf binary's total), time_us.  Returns the table entries."""
    best = {}
    for r in rows:
        if r.get("wrong"):
            continue  # a variant that produced a wrong result never enters the table
        kb = key_bytes(r["op"], int(r["bytes"]), nranks)
        k = (OPS[r["op"]], bucket(max(kb, 1)))
        if k not in best or r["time_us"] < best[k]["time_us"]:
            best[k] = r
    out = []
    for (op, l2), r in sorted(best.items()):
        out.append({"op": op, "log2_bytes": l2, "nranks": nranks, "kind": r["kind"], "nctas": int(r["nctas"]), "us": round(float(r["time_us"]), 3)})
    return out


def write_cache(entries, path):
    """One entry per line, in the exact form the library's loader scans for."""
    with open(path, "w") as f:
        f.write("[\n")
        for i, e in enumerate(entries):
            f.write(' {"op": %d, "log2_bytes": %d, "nranks": %d, "kind": "%s", "nctas": %d, "us": %.3f}%s\n'
                    % (e["op"], e["log2_bytes"], e["nranks"], e["kind"], e["nctas"], e["us"], "" if i == len(entries) - 1 else ","))
        f.write("]\n")


def sweep(nranks: int, ops, sizes, multicast: bool, perf_bin: Path, iters: int = 20, warm: int = 5, verbose: bool = True):
    rows = []
    for op in ops:
        for kind in CANDIDATES[op]:
            wanted = [s for s in sizes if legal(op, kind, key_bytes(op, s, nranks), multicast)]
            if not wanted:
                continue
            for nctas in cta_choices(kind):
                with tempfile.NamedTemporaryFile(suffix=".jsonl", delete=False) as tf:
                    out = tf.name
                env = dict(os.environ, FLAGCX_USE_COMM_TAG=f"{kind}:{nctas}")
                for s in wanted:  # one process per size keeps a failing size from hiding the others
                    cmd = [str(perf_bin), "-o", op, "-g", str(nranks), "-d", "float", "-b", str(s), "-e", str(s), "-w", str(warm),
                           "-n", str(iters), "-c", "1", "-J", out]
                    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
                    if res.returncode != 0 and verbose:
                        print(f"  {op} {kind}:{nctas} {s} B failed", file=sys.stderr)
                for line in Path(out).read_text().splitlines():
                    r = json.loads(line)
                    r.update(kind=kind, nctas=nctas)
                    rows.append(r)
                os.unlink(out)
                if verbose:
                    print(f"{op:14s} {kind:11s} x{nctas:<3d} measured at {len(wanted)} sizes", flush=True)
    return rows


def tune_in_process(nranks: int, ops, min_bytes: int, max_bytes: int, factor: int, out: str, perf_bin: Path, dtype: str = "float",
                    iters: int = 10, log=None):
    """The fast way: the perf binary's tune mode (-T 1) times every legal variant of every (operation, size)
    inside ONE set of rank processes, first on ordinary buffers, then on buffers from flagcxMemAlloc (which adds
    the zero-copy kinds), and the library writes the merged table.  Returns the tool's output."""
    env = dict(os.environ, FLAGCX_TUNER_CACHE=out, FLAGCX_TUNER_DEFAULTS="0")
    env.setdefault("FLAGCX_HEAP_USER_BYTES", str(2 * max_bytes + (256 << 20)))
    text = ""
    for reg in (0, 1):
        cmd = [str(perf_bin), "-o", ",".join(ops), "-g", str(nranks), "-d", dtype, "-b", str(min_bytes), "-e", str(max_bytes), "-f", str(factor),
               "-w", "2", "-n", str(iters), "-T", "1", "-R", str(reg), "-S", out]
        res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1800)
        text += res.stdout + res.stderr
        if log:
            Path(log).write_text(text)
        if res.returncode != 0:
            raise RuntimeError(f"tune run failed (registered={reg}): {res.stderr[-2000:]}")
    return text


def main():
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--gpus", type=int, required=True)
    ap.add_argument("--out", required=True)
    ap.add_argument("--ops", default=",".join(OPS))
    ap.add_argument("--min-bytes", type=int, default=64)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--factor", type=int, default=4)
    ap.add_argument("--no-multicast", action="store_true", help="skip the NVLS kinds")
    ap.add_argument("--rows", help="also keep every measured row in this JSON-lines file")
    ap.add_argument("--per-process", action="store_true", help="one perf process per variant and size (slow; isolates failures)")
    ap.add_argument("--log", help="keep the tune run's output in this file")
    args = ap.parse_args()
    from flagcx_b200 import _build
    perf = _build.build_tools()
    if not args.per_process:
        ops = [o for o in args.ops.split(",") if o in OPS]
        text = tune_in_process(args.gpus, ops, args.min_bytes, args.max_bytes, args.factor, args.out, perf, log=args.log)
        n = sum(1 for line in text.splitlines() if line.startswith("tune "))
        print(f"{n} (operation, size) pairs tuned; table written to {args.out}")
        return
    sizes, s = [], args.min_bytes
    while s <= args.max_bytes:
        sizes.append(s)
        s *= args.factor
    rows = sweep(args.gpus, [o for o in args.ops.split(",") if o in OPS], sizes, not args.no_multicast, perf)
    if args.rows:
        Path(args.rows).write_text("".join(json.dumps(r) + "\n" for r in rows))
    entries = build_cache(rows, args.gpus)
    write_cache(entries, args.out)
    print(f"{len(entries)} decisions from {len(rows)} measurements written to {args.out}")


if __name__ == "__main__":
    main()
