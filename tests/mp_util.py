"""Run a function as several cooperating processes (one per rank) and collect
the results.  Rank 0 creates the unique id; it travels through a queue."""
import multiprocessing as mp
import os
import traceback


def _child(fn, rank, world, idq, resq, env, args):
    try:
        os.environ.update(env or {})
        os.environ.setdefault("FLAGCX_SOCKET_IFNAME", "lo")
        from flagcx_b200.wrapper import FLAGCXLibrary
        lib = FLAGCXLibrary()
        if rank == 0:
            uid = lib.flagcxGetUniqueId()
            raw = lib.unique_id_to_bytes(uid)
            for _ in range(world - 1):
                idq.put(raw)
        else:
            raw = idq.get(timeout=60)
            uid = lib.unique_id_from_bytes(raw)
        out = fn(lib, uid, rank, world, *args)
        resq.put((rank, "ok", out))
    except BaseException as e:  # noqa
        resq.put((rank, "err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))


def run_ranks(fn, world, args=(), env=None, timeout=120, per_rank_env=None, expect_fail=False):
    ctx = mp.get_context("spawn")
    idq, resq = ctx.Queue(), ctx.Queue()
    procs = []
    for r in range(world):
        e = dict(env or {})
        if per_rank_env:
            e.update(per_rank_env.get(r, {}))
        p = ctx.Process(target=_child, args=(fn, r, world, idq, resq, e, args))
        p.start()
        procs.append(p)
    results = {}
    try:
        for _ in range(world):
            try:
                rank, status, out = resq.get(timeout=timeout)
            except Exception:
                break
            results[rank] = (status, out)
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    if not expect_fail:
        for r in range(world):
            assert r in results, f"rank {r} produced no result (exit codes {[p.exitcode for p in procs]})"
            assert results[r][0] == "ok", f"rank {r} failed: {results[r][1]}"
    return results, [p.exitcode for p in procs]
