"""Zero-copy collective kernels on ONE GPU (emulated ranks, see test_emu_collectives.py).

The zero-copy kinds read and write the peers' user buffers in place; here every emulated rank's buffers live
on the same device, so a buffer's address serves as its peer-visible location and the plain peer load/store
path of each kind runs (the switch-reduction path needs real NVSwitch hardware and is covered by the
multi-GPU tests).  Results are compared with a PyTorch fp32 reference.
"""
import ctypes

import pytest
import torch

from flagcx_b200.wrapper import FLAGCXLibrary
from tests.test_emu_collectives import DT, OPS, Emu, _rand, _reduce_ref, _tol

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib(native_lib):
    return FLAGCXLibrary(native_lib)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
@pytest.mark.parametrize("count,nctas", [(1, 1), (7, 2), (4099, 3), (262147, 8), (1 << 20, 16)])
def test_allreduce_zero_copy(lib, n, count, nctas):
    emu = Emu(lib, n, stage=16 << 20)  # the staged kind interleaved below needs (n + n) slices of staging
    try:
        for dtype in (torch.float32, torch.bfloat16):
            for rep in range(3):
                xs = _rand(n, count, dtype, seed=rep)
                ys = [torch.empty_like(x) for x in xs]
                emu.coll("allreduce", "ar_zc", nctas, xs, ys, count, dtype)
                ref = _reduce_ref(xs, 0)
                for y in ys:
                    torch.testing.assert_close(y.float(), ref, atol=_tol(dtype) * n, rtol=_tol(dtype))
                for y in ys[1:]:
                    assert torch.equal(y, ys[0])  # one owner computes each slice: all ranks hold the same bits
            # in place, and interleaved with a staged kind so that both share flags, parities and mailboxes
            zs = [x.clone() for x in xs]
            emu.coll("allreduce", "ar_zc", nctas, zs, zs, count, dtype, red=4)
            for z in zs:
                torch.testing.assert_close(z.float(), ref / n, atol=_tol(dtype), rtol=_tol(dtype))
            ws = [torch.empty_like(x) for x in xs]
            emu.coll("allreduce", "ar_twoshot", min(nctas, 4), xs, ws, count, dtype)
            for w in ws:
                torch.testing.assert_close(w.float(), ref, atol=_tol(dtype) * n, rtol=_tol(dtype))
    finally:
        emu.close()


@pytest.mark.parametrize("dtype", [torch.int8, torch.uint8, torch.int32, torch.int64, torch.float16, torch.float64,
                                   torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("red", [0, 2, 3, 4])
def test_allreduce_zero_copy_types_and_ops(lib, dtype, red):
    n, count = 4, 4099
    emu = Emu(lib, n)
    try:
        xs = _rand(n, count, dtype, seed=7)
        ys = [torch.empty_like(x) for x in xs]
        emu.coll("allreduce", "ar_zc", 3, xs, ys, count, dtype, red=red)
        ref = _reduce_ref(xs, red)
        for y in ys:
            if dtype.is_floating_point:
                torch.testing.assert_close(y.float(), ref.float(), atol=_tol(dtype) * n, rtol=_tol(dtype))
            else:
                exp = ref if red != 4 else torch.div(_reduce_ref(xs, 0), n, rounding_mode="trunc")
                assert torch.equal(y.double(), exp.double())
    finally:
        emu.close()


def test_allreduce_zero_copy_unaligned_and_cast(lib):
    n, count = 4, 10007
    emu = Emu(lib, n)
    try:
        base = _rand(n, count + 3, torch.float32, seed=3)
        xs = [b[3:] for b in base]  # 12-byte offset: the scalar path
        ref = _reduce_ref(xs, 0)
        emu.coll("allreduce", "ar_zc", 3, xs, xs, count, torch.float32)
        for x in xs:
            torch.testing.assert_close(x, ref, atol=1e-5, rtol=1e-5)
        for in_dt, out_dt in ((torch.float32, torch.bfloat16), (torch.bfloat16, torch.float8_e4m3fn), (torch.bfloat16, torch.float32)):
            xs = _rand(n, count, in_dt, seed=11)
            ys = [torch.empty(count, dtype=out_dt, device="cuda") for _ in range(n)]
            emu.coll("allreduce", "ar_zc", 4, xs, ys, count, in_dt, out_dt=out_dt, scale=0.5)
            ref = (_reduce_ref(xs, 0) * 0.5).to(out_dt).float()
            for y in ys:
                torch.testing.assert_close(y.float(), ref, atol=_tol(out_dt) * 2, rtol=_tol(out_dt) * 2)
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("count", [1, 777, 150001])
def test_reducescatter_allgather_reduce_zero_copy(lib, n, count):
    emu = Emu(lib, n)
    try:
        for dtype in (torch.float32, torch.bfloat16):
            xs = _rand(n, count * n, dtype, seed=5)
            ref = _reduce_ref(xs, 0)
            ys = [torch.empty(count, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("reducescatter", "rs_zc", 4, xs, ys, count, dtype)
            for r, y in enumerate(ys):
                torch.testing.assert_close(y.float(), ref[r * count:(r + 1) * count], atol=_tol(dtype) * n, rtol=_tol(dtype))
            zs = [torch.empty(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("allgather", "move_zc", 4, ys, zs, count, dtype)
            exp = torch.cat(ys)
            for z in zs:
                assert torch.equal(z, exp)
            ws = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]  # in place
            for r in range(n):
                ws[r][r * count:(r + 1) * count] = ys[r]
            emu.coll("allgather", "move_zc", 2, [ws[r][r * count:(r + 1) * count] for r in range(n)], ws, count, dtype)
            for w in ws:
                assert torch.equal(w, exp)
            root = n - 1
            rd = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("reduce", "reduce_zc", 3, xs, rd, count * n, dtype, root=root)
            torch.testing.assert_close(rd[root].float(), ref, atol=_tol(dtype) * n, rtol=_tol(dtype))
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 5, 8])
def test_movers_zero_copy(lib, n):
    emu = Emu(lib, n)
    try:
        for dtype, count in ((torch.float32, 12345), (torch.uint8, 13), (torch.bfloat16, 70001)):
            xs = _rand(n, count * n, dtype, seed=9)
            pieces = [x[:count].clone() for x in xs]
            for root in (0, n - 1):
                bs = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
                emu.coll("bcast", "move_zc", 3, pieces, bs, count, dtype, root=root)
                for b in bs:
                    assert torch.equal(b, pieces[root])
                gg = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
                emu.coll("gather", "move_zc", 3, pieces, gg, count, dtype, root=root)
                assert torch.equal(gg[root], torch.cat(pieces))
                ss = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
                emu.coll("scatter", "move_zc", 3, xs, ss, count, dtype, root=root)
                for r in range(n):
                    assert torch.equal(ss[r], xs[root][r * count:(r + 1) * count])
            outs = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("a2a", "move_zc", 4, xs, outs, count, dtype)
            for r in range(n):
                assert torch.equal(outs[r], torch.cat([xs[p][r * count:(r + 1) * count] for p in range(n)]))
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 4, 8])
def test_alltoallv_zero_copy(lib, n):
    emu = Emu(lib, n)
    try:
        sc = [[40000 * ((r + p) % 3) + 17 * p for p in range(n)] for r in range(n)]
        tables, sends, recvs, exps = [], [], [], []
        for r in range(n):
            sd = [sum(sc[r][:p]) for p in range(n)]
            rc = [sc[p][r] for p in range(n)]
            rd = [sum(rc[:p]) for p in range(n)]
            tables += sc[r] + sd + rc + rd
            sends.append(torch.rand(max(1, sum(sc[r])), device="cuda") * 2 - 1)
            recvs.append(torch.zeros(max(1, sum(rc)), device="cuda"))
        for r in range(n):
            parts = [sends[p][sum(sc[p][:r]):sum(sc[p][:r]) + sc[p][r]] for p in range(n)]
            exps.append(torch.cat(parts))
        emu.coll("a2av", "move_zc", 4, sends, recvs, 0, torch.float32, tables=tables)
        for r in range(n):
            assert torch.equal(recvs[r][:exps[r].numel()], exps[r])
    finally:
        emu.close()


def test_zero_copy_rejects_a_buffer_the_peers_cannot_see(lib):
    """A rank whose buffer is not peer-visible makes every rank record a bad-argument error and skip the data
    phase; nothing is read or written through a bad address and the emulated communicator's GPU stays usable."""
    n, count = 4, 1000
    emu = Emu(lib, n)
    try:
        xs = _rand(n, count, torch.float32, seed=1)
        ys = [torch.full((count,), -7.0, device="cuda") for _ in range(n)]
        arr = ctypes.c_void_p * n
        recv = [y.data_ptr() for y in ys]
        recv[1] = None  # rank 1 offers no receive buffer
        lib.call("flagcxEmuCollective", emu.h, OPS["allreduce"], b"ar_zc", 2, arr(*[x.data_ptr() for x in xs]), arr(*recv), count,
                 DT[torch.float32], DT[torch.float32], ctypes.c_float(1.0), 0, 0, None,
                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        code = ctypes.c_int()
        lib.call("flagcxEmuGetError", emu.h, ctypes.byref(code))
        assert code.value == 3  # FCX_ERR_BADARG
        for y in ys:
            assert bool((y == -7.0).all())
    finally:
        emu.close()


def test_a_launch_that_does_not_fit_the_staging_area_is_refused(lib):
    """The emulator launches a message as one piece (the library proper cuts it to the staging size first); a
    staged kind whose slots would overrun the staging half records a bad-argument error and moves nothing."""
    n, count = 2, 1 << 20
    emu = Emu(lib, n, stage=4 << 20)  # all-reduce needs 2 x (2 + 2) MiB here
    try:
        xs = _rand(n, count, torch.float32, seed=1)
        ys = [torch.full((count,), -7.0, device="cuda") for _ in range(n)]
        arr = ctypes.c_void_p * n
        lib.call("flagcxEmuCollective", emu.h, OPS["allreduce"], b"ar_twoshot", 4, arr(*[x.data_ptr() for x in xs]),
                 arr(*[y.data_ptr() for y in ys]), count, DT[torch.float32], DT[torch.float32], ctypes.c_float(1.0), 0, 0, None,
                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        code = ctypes.c_int()
        lib.call("flagcxEmuGetError", emu.h, ctypes.byref(code))
        assert code.value == 3
        for y in ys:
            assert bool((y == -7.0).all())
    finally:
        emu.close()
