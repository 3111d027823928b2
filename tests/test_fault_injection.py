"""Failure detection and recovery, exercised on CPU ranks only.

Failures are made on the host: a rank that corrupts its handshake, a rank
that exits in the middle of a collective, a rank that never joins.  The
survivors must get an error code within the configured deadline instead of
hanging, and must be able to build a smaller communicator afterwards.  No GPU
is involved, nothing is faulted or hung on purpose on a device."""
import ctypes
import time

import numpy as np

from flagcx_b200.wrapper import FLAGCXError
from tests.mp_util import run_ranks


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _init_only(lib, uid, rank, world):
    t0 = time.time()
    try:
        comm = lib.flagcxCommInitRank(world, uid, rank)
    except FLAGCXError as e:
        return {"error": e.code, "secs": time.time() - t0}
    x = np.ones(16, np.float32)
    lib.flagcxAllReduce(_p(x), _p(x), 16, 7, 0, comm)
    lib.flagcxCommDestroy(comm)
    return {"error": 0, "sum": float(x[0]), "secs": time.time() - t0}


def test_corrupted_handshake_is_rejected_and_others_time_out(native_lib):
    res, _ = run_ranks(_init_only, 2, env={"FLAGCX_FAULT_INJECT": "bad_magic", "FLAGCX_FAULT_RANK": "1", "FLAGCX_BOOTSTRAP_TIMEOUT_MS": "2500"},
                       timeout=60)
    for r in range(2):
        out = res[r][1]
        assert out["error"] != 0, out       # nobody gets a communicator
        assert out["secs"] < 30, out        # and nobody hangs


def _exchange_then_maybe_die(lib, uid, rank, world):
    comm = lib.flagcxCommInitRank(world, uid, rank)
    x = np.full(1 << 16, float(rank), np.float32)
    codes = []
    t0 = time.time()
    for it in range(50):
        try:
            lib.flagcxAllReduce(_p(x), _p(x), x.size, 7, 2, comm)  # max: stays finite
            codes.append(0)
        except FLAGCXError as e:
            codes.append(e.code)
            break
    return {"codes": codes, "secs": time.time() - t0, "async": 0}


def test_rank_exit_mid_run_surfaces_as_remote_error(native_lib):
    # rank 1 leaves the process after 40 bootstrap messages (host-side injection); rank 0 must see an error, quickly
    res, codes = run_ranks(_exchange_then_maybe_die, 2, env={"FLAGCX_FAULT_INJECT": "exit_after:40", "FLAGCX_FAULT_RANK": "1",
                                                             "FLAGCX_BOOTSTRAP_TIMEOUT_MS": "3000"}, timeout=60, expect_fail=True)
    assert codes[1] == 17                      # the injected exit
    assert 0 in res and res[0][0] == "ok"
    out = res[0][1]
    assert out["codes"][-1] == 6, out          # flagcxRemoteError
    assert out["secs"] < 30


def _shrink(lib, uid, rank, world):
    """World of 3; rank 2 never takes part in the work.  Ranks 0 and 1 notice the missing peer through the
    deadline, drop the communicator and continue on a 2-rank communicator split off beforehand."""
    comm = lib.flagcxCommInitRank(world, uid, rank)
    pair = lib.flagcxCommSplit(comm, 0 if rank < 2 else -1, rank)  # survivors' communicator, made while all are alive
    if rank == 2:
        lib.flagcxCommDestroy(comm)
        return {"left": True}
    x = np.ones(8, np.float32)
    err = 0
    try:
        lib.flagcxAllReduce(_p(x), _p(x), 8, 7, 0, comm)  # rank 2 is gone: must fail, not hang
    except FLAGCXError as e:
        err = e.code
    y = np.full(8, float(rank + 1), np.float32)
    lib.flagcxAllReduce(_p(y), _p(y), 8, 7, 0, pair)
    return {"err": err, "sum": float(y[0])}


def test_survivors_continue_on_smaller_communicator(native_lib):
    res, _ = run_ranks(_shrink, 3, env={"FLAGCX_BOOTSTRAP_TIMEOUT_MS": "2500"}, timeout=90, expect_fail=True)
    assert res[2][1] == {"left": True}
    for r in (0, 1):
        assert res[r][0] == "ok", res[r]
        assert res[r][1]["err"] == 6 and res[r][1]["sum"] == 3.0, res[r][1]
