"""Protocol tests of the collective kernels on ONE GPU.

`flagcxEmu*` runs n emulated ranks inside a single cooperative launch (each
rank with its own heap on the same device), so flags, parities, unit
ownership and chunk counters of the real multi-GPU kernels are exercised
without NVLink.  Results are compared with a plain PyTorch fp32 reference of
the same operation.  Small and odd sizes, unaligned tails and every rank count
from 2 to 8 are covered; the reference library's own tests only print
(test/perf/test_allreduce.cpp) or compare empty strings (test/unittest/main.cpp:61-63).
"""
import ctypes

import pytest
import torch

from flagcx_b200.wrapper import FLAGCXLibrary

pytestmark = pytest.mark.gpu

OPS = dict(send=0, recv=1, bcast=2, gather=3, scatter=4, reduce=5, allreduce=6, allgather=7, reducescatter=8, a2a=9, a2av=10)
DT = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7, torch.float64: 8,
      torch.bfloat16: 9, torch.float8_e4m3fn: 10, torch.float8_e5m2: 11}


@pytest.fixture(scope="module")
def lib(native_lib):
    return FLAGCXLibrary(native_lib)


class Emu:
    def __init__(self, lib, n, stage=4 << 20):
        self.lib, self.n = lib, n
        self.h = ctypes.c_void_p()
        lib.call("flagcxEmuCreate", ctypes.byref(self.h), n, stage)

    def close(self):
        self.lib.call("flagcxEmuDestroy", self.h)

    def coll(self, op, kind, nctas, send, recv, count, dt, out_dt=None, scale=1.0, red=0, root=0, tables=None):
        n = self.n
        arr = ctypes.c_void_p * n
        s = arr(*[(t.data_ptr() if t is not None else None) for t in send]) if send else None
        r = arr(*[(t.data_ptr() if t is not None else None) for t in recv]) if recv else None
        tb = None
        if tables is not None:
            flat = [int(v) for v in tables]
            tb = (ctypes.c_size_t * len(flat))(*flat)
        self.lib.call("flagcxEmuCollective", self.h, OPS[op], kind.encode(), nctas, s, r, count, DT[dt],
                      DT[out_dt if out_dt is not None else dt], ctypes.c_float(scale), red, root, tb,
                      ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        torch.cuda.synchronize()
        code = ctypes.c_int()
        self.lib.call("flagcxEmuGetError", self.h, ctypes.byref(code))
        assert code.value == 0, f"device wait gave up, code {code.value}"


def _rand(n, count, dtype, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    out = []
    for r in range(n):
        if dtype in (torch.int8, torch.uint8, torch.int32, torch.int64):
            out.append(torch.randint(0, 5, (count,), generator=g, device="cuda").to(dtype))
        else:
            out.append((torch.rand(count, generator=g, device="cuda") * 2 - 1).to(dtype))
    return out


def _reduce_ref(xs, red):
    st = torch.stack([x.float() if x.dtype.is_floating_point else x.double() for x in xs])
    if red == 0:
        return st.sum(0)
    if red == 1:
        return st.prod(0)
    if red == 2:
        return st.max(0).values
    if red == 3:
        return st.min(0).values
    return st.sum(0) / len(xs)


def _tol(dtype):
    return {torch.float32: 1e-5, torch.float64: 1e-5, torch.bfloat16: 2e-2, torch.float16: 3e-3,
            torch.float8_e4m3fn: 0.13, torch.float8_e5m2: 0.26}.get(dtype, 0)


@pytest.mark.parametrize("n", [2, 3, 4, 8])
@pytest.mark.parametrize("kind,count,nctas", [("ar_ll", 1, 1), ("ar_ll", 1000, 2), ("ar_ll", 8192, 4), ("ar_oneshot", 5, 1),
                                              ("ar_oneshot", 70001, 4), ("ar_twoshot", 3, 2), ("ar_twoshot", 65536, 8),
                                              ("ar_twoshot", 262147, 16)])
def test_allreduce_variants(lib, n, kind, count, nctas):
    emu = Emu(lib, n)
    try:
        for dtype in (torch.float32, torch.bfloat16):
            if kind == "ar_ll" and count * dtype.itemsize > 32768:
                continue
            for rep in range(3):  # consecutive launches exercise both parities and the done counters
                xs = _rand(n, count, dtype, seed=rep)
                ys = [torch.empty_like(x) for x in xs]
                emu.coll("allreduce", kind, nctas, xs, ys, count, dtype)
                ref = _reduce_ref(xs, 0)
                for y in ys:
                    torch.testing.assert_close(y.float(), ref, atol=_tol(dtype) * n, rtol=_tol(dtype))
                # every rank must hold bit-identical results
                for y in ys[1:]:
                    assert torch.equal(y, ys[0])
    finally:
        emu.close()


@pytest.mark.parametrize("dtype", [torch.int8, torch.uint8, torch.int32, torch.int64, torch.float16, torch.float64,
                                   torch.float8_e4m3fn, torch.float8_e5m2])
@pytest.mark.parametrize("red", [0, 2, 3, 4])
def test_allreduce_types_and_ops(lib, dtype, red):
    n, count = 4, 4099
    emu = Emu(lib, n)
    try:
        xs = _rand(n, count, dtype, seed=7)
        for kind, nctas in (("ar_oneshot", 2), ("ar_twoshot", 4)):
            ys = [torch.empty_like(x) for x in xs]
            emu.coll("allreduce", kind, nctas, xs, ys, count, dtype, red=red)
            ref = _reduce_ref(xs, red)
            for y in ys:
                if dtype.is_floating_point:
                    torch.testing.assert_close(y.float(), ref.float(), atol=_tol(dtype) * n, rtol=_tol(dtype))
                else:
                    exp = ref if red != 4 else torch.div(_reduce_ref(xs, 0), n, rounding_mode="trunc")
                    assert torch.equal(y.double(), exp.double())
    finally:
        emu.close()


def test_allreduce_in_place_and_unaligned(lib):
    n, count = 4, 10007
    emu = Emu(lib, n)
    try:
        for kind, nctas in (("ar_oneshot", 2), ("ar_twoshot", 3), ("ar_ll", 2)):
            base = _rand(n, count + 3, torch.float32, seed=3)
            xs = [b[3:] for b in base]  # 12-byte offset: not 16-byte aligned
            if kind == "ar_ll":
                xs = [x[:2000] for x in xs]
            ref = _reduce_ref(xs, 0)
            emu.coll("allreduce", kind, nctas, xs, xs, xs[0].numel(), torch.float32)
            for x in xs:
                torch.testing.assert_close(x, ref, atol=1e-5, rtol=1e-5)
    finally:
        emu.close()


@pytest.mark.parametrize("in_dt,out_dt", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float8_e4m3fn),
                                           (torch.float32, torch.float8_e4m3fn), (torch.bfloat16, torch.float32)])
def test_allreduce_fused_cast_and_scale(lib, in_dt, out_dt):
    n, count = 4, 33333
    emu = Emu(lib, n)
    try:
        xs = _rand(n, count, in_dt, seed=11)
        for kind, nctas in (("ar_oneshot", 2), ("ar_twoshot", 4)):
            ys = [torch.empty(count, dtype=out_dt, device="cuda") for _ in range(n)]
            emu.coll("allreduce", kind, nctas, xs, ys, count, in_dt, out_dt=out_dt, scale=0.5)
            ref = (_reduce_ref(xs, 0) * 0.5).to(out_dt).float()
            for y in ys:
                torch.testing.assert_close(y.float(), ref, atol=_tol(out_dt) * 2, rtol=_tol(out_dt) * 2)
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("count", [1, 777, 40000])
def test_reducescatter_allgather(lib, n, count):
    emu = Emu(lib, n)
    try:
        for dtype in (torch.float32, torch.bfloat16):
            xs = _rand(n, count * n, dtype, seed=5)
            ys = [torch.empty(count, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("reducescatter", "rs", 4, xs, ys, count, dtype)
            ref = _reduce_ref(xs, 0)
            for r, y in enumerate(ys):
                torch.testing.assert_close(y.float(), ref[r * count:(r + 1) * count], atol=_tol(dtype) * n, rtol=_tol(dtype))
            # all-gather the scattered pieces back
            zs = [torch.empty(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("allgather", "ag", 4, ys, zs, count, dtype)
            exp = torch.cat(ys)
            for z in zs:
                assert torch.equal(z, exp)
            # in-place all-gather: send is recv + rank*count
            ws = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            for r in range(n):
                ws[r][r * count:(r + 1) * count] = ys[r]
            emu.coll("allgather", "ag", 2, [ws[r][r * count:(r + 1) * count] for r in range(n)], ws, count, dtype)
            for w in ws:
                assert torch.equal(w, exp)
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 3, 8])
@pytest.mark.parametrize("nctas", [1, 3])
def test_ll_forms_of_small_collectives(lib, n, nctas):
    """The barrier-free forms used for small messages: flags travel inside the data lines."""
    emu = Emu(lib, n)
    try:
        for dtype, count in ((torch.float32, 1), (torch.float32, 1000), (torch.bfloat16, 4093), (torch.int8, 13), (torch.uint8, 8190)):
            xs = _rand(n, count * n, dtype, seed=21)
            pieces = [x[:count].clone() for x in xs]
            gs = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("allgather", "move_ll", nctas, pieces, gs, count, dtype)
            for g in gs:
                assert torch.equal(g, torch.cat(pieces))
            outs = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("a2a", "move_ll", nctas, xs, outs, count, dtype)
            for r in range(n):
                assert torch.equal(outs[r], torch.cat([xs[p][r * count:(r + 1) * count] for p in range(n)]))
            for root in (0, n - 1):
                bs = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
                emu.coll("bcast", "move_ll", nctas, pieces, bs, count, dtype, root=root)
                for b in bs:
                    assert torch.equal(b, pieces[root])
                gg = [torch.zeros(count * n, dtype=dtype, device="cuda") for _ in range(n)]
                emu.coll("gather", "move_ll", nctas, pieces, gg, count, dtype, root=root)
                assert torch.equal(gg[root], torch.cat(pieces))
                ss = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
                emu.coll("scatter", "move_ll", nctas, xs, ss, count, dtype, root=root)
                for r in range(n):
                    assert torch.equal(ss[r], xs[root][r * count:(r + 1) * count])
            if dtype in (torch.float32, torch.bfloat16):
                ref = _reduce_ref(xs, 0)
                ys = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
                emu.coll("reducescatter", "rs_ll", nctas, xs, ys, count, dtype)
                for r, y in enumerate(ys):
                    torch.testing.assert_close(y.float(), ref[r * count:(r + 1) * count], atol=_tol(dtype) * n, rtol=_tol(dtype))
                root = n // 2
                rd = [torch.zeros(count, dtype=dtype, device="cuda") for _ in range(n)]
                emu.coll("reduce", "reduce_ll", nctas, pieces, rd, count, dtype, root=root)
                torch.testing.assert_close(rd[root].float(), _reduce_ref(pieces, 0), atol=_tol(dtype) * n, rtol=_tol(dtype))
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 3, 8])
def test_pipelined_sub_chunks(lib, n, monkeypatch):
    """With a tiny sub-chunk size every large-message kind runs many pipeline iterations (push of chunk i
    overlapping the reduction / copy-out of chunks i-1 and i-2), in place and out of place."""
    monkeypatch.setenv("FLAGCX_PIPE_BYTES", "65536")
    emu = Emu(lib, n, stage=16 << 20)
    try:
        count = 150001  # per-rank piece: odd, not a multiple of the unit, ~10-40 sub-chunks
        for dtype in (torch.float32, torch.bfloat16):
            xs = _rand(n, count * n, dtype, seed=11)
            ref = _reduce_ref(xs, 0)
            for kind, ctas in (("ar_twoshot", 5), ("ar_twoshot", 8)):
                ys = [torch.empty_like(x) for x in xs]
                emu.coll("allreduce", kind, ctas, xs, ys, count * n, dtype)
                for y in ys:
                    torch.testing.assert_close(y.float(), ref, atol=_tol(dtype) * n, rtol=_tol(dtype))
            zs = [x.clone() for x in xs]  # in place
            emu.coll("allreduce", "ar_twoshot", 6, zs, zs, count * n, dtype)
            for z in zs:
                torch.testing.assert_close(z.float(), ref, atol=_tol(dtype) * n, rtol=_tol(dtype))
            ys = [torch.empty(count, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("reducescatter", "rs", 7, xs, ys, count, dtype)
            for r, y in enumerate(ys):
                torch.testing.assert_close(y.float(), ref[r * count:(r + 1) * count], atol=_tol(dtype) * n, rtol=_tol(dtype))
            gs = [torch.empty(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("allgather", "ag", 5, ys, gs, count, dtype)
            for g in gs:
                assert torch.equal(g, torch.cat(ys))
            outs = [torch.empty(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("a2a", "a2a", 6, xs, outs, count, dtype)
            for r in range(n):
                exp = torch.cat([xs[p][r * count:(r + 1) * count] for p in range(n)])
                assert torch.equal(outs[r], exp)
            root = n - 1
            bs = [torch.empty(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("bcast", "bcast", 4, xs, bs, count * n, dtype, root=root)
            for b in bs:
                assert torch.equal(b, xs[root])
            rd = [torch.empty(count * n, dtype=dtype, device="cuda") for _ in range(n)]
            emu.coll("reduce", "reduce", 5, xs, rd, count * n, dtype, root=root)
            torch.testing.assert_close(rd[root].float(), ref, atol=_tol(dtype) * n, rtol=_tol(dtype))
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 5, 8])
def test_rooted_ops(lib, n):
    emu = Emu(lib, n)
    count = 12345
    try:
        for root in (0, n - 1):
            xs = _rand(n, count, torch.float32, seed=root)
            ys = [torch.zeros(count, device="cuda") for _ in range(n)]
            emu.coll("bcast", "bcast", 4, xs, ys, count, torch.float32, root=root)
            for y in ys:
                assert torch.equal(y, xs[root])
            ys = [torch.zeros(count, device="cuda") for _ in range(n)]
            emu.coll("reduce", "reduce", 4, xs, ys, count, torch.float32, root=root)
            torch.testing.assert_close(ys[root], _reduce_ref(xs, 0), atol=1e-5, rtol=1e-5)
            gs = [torch.zeros(count * n, device="cuda") for _ in range(n)]
            emu.coll("gather", "gather", 4, xs, gs, count, torch.float32, root=root)
            assert torch.equal(gs[root], torch.cat(xs))
            big = _rand(n, count * n, torch.float32, seed=9)
            ss = [torch.zeros(count, device="cuda") for _ in range(n)]
            emu.coll("scatter", "scatter", 4, big, ss, count, torch.float32, root=root)
            for r in range(n):
                assert torch.equal(ss[r], big[root][r * count:(r + 1) * count])
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 4, 8])
def test_alltoall_and_alltoallv(lib, n):
    emu = Emu(lib, n, stage=1 << 20)
    try:
        count = 5001
        xs = _rand(n, count * n, torch.bfloat16, seed=1)
        ys = [torch.zeros(count * n, dtype=torch.bfloat16, device="cuda") for _ in range(n)]
        emu.coll("a2a", "a2a", 4, xs, ys, count, torch.bfloat16)
        for r in range(n):
            exp = torch.cat([xs[p][r * count:(r + 1) * count] for p in range(n)])
            assert torch.equal(ys[r], exp)
        # variable: rank r sends 1000*((r+p)%3) + 17*p elements to p; some blocks are empty and
        # some exceed one staging round (stage/n/2 bytes), which forces several rounds
        sc = [[40000 * ((r + p) % 3) + 17 * p for p in range(n)] for r in range(n)]
        tables = []
        sends, recvs, exps = [], [], []
        for r in range(n):
            sd = [sum(sc[r][:p]) for p in range(n)]
            rc = [sc[p][r] for p in range(n)]
            rd = [sum(rc[:p]) for p in range(n)]
            tables += sc[r] + sd + rc + rd
            sends.append((torch.rand(max(1, sum(sc[r])), device="cuda") * 2 - 1))
            recvs.append(torch.zeros(max(1, sum(rc)), device="cuda"))
        for r in range(n):
            parts = []
            for p in range(n):
                sd = sum(sc[p][:r])
                parts.append(sends[p][sd:sd + sc[p][r]])
            exps.append(torch.cat(parts) if parts else torch.zeros(0, device="cuda"))
        emu.coll("a2av", "a2av", 4, sends, recvs, 0, torch.float32, tables=tables)
        for r in range(n):
            assert torch.equal(recvs[r][:exps[r].numel()], exps[r])
    finally:
        emu.close()


@pytest.mark.parametrize("n", [2, 4])
@pytest.mark.parametrize("zero_copy", [False, True])
def test_grouped_sendrecv(lib, n, zero_copy, monkeypatch):
    # zero_copy: the sender publishes where its buffer lies and the receiver reads it in place (the form used
    # for buffers in the symmetric heap or in a registered segment); otherwise data travels through staging slots
    monkeypatch.setenv("FLAGCX_EMU_P2P_ZEROCOPY", "1" if zero_copy else "0")
    emu = Emu(lib, n)
    try:
        # a ring exchange plus a self copy per rank, two rounds, message larger than two staging chunks
        for nbytes in (0, 100, 300000):
            for rnd in range(2):
                srcs, dsts, sb, rb, sizes, keep = [], [], [], [], [], []
                for r in range(n):
                    s = torch.randint(0, 255, (max(nbytes, 1),), device="cuda", dtype=torch.uint8)
                    d = torch.zeros(max(nbytes, 1), device="cuda", dtype=torch.uint8)
                    keep.append((s, d, r, (r + 1) % n))
                    srcs.append(r); dsts.append((r + 1) % n); sb.append(s.data_ptr()); rb.append(d.data_ptr()); sizes.append(nbytes)
                    s2 = torch.randint(0, 255, (max(nbytes, 1),), device="cuda", dtype=torch.uint8)
                    d2 = torch.zeros(max(nbytes, 1), device="cuda", dtype=torch.uint8)
                    keep.append((s2, d2, r, r))
                    srcs.append(r); dsts.append(r); sb.append(s2.data_ptr()); rb.append(d2.data_ptr()); sizes.append(nbytes)
                k = len(srcs)
                lib.call("flagcxEmuSendRecv", emu.h, k, (ctypes.c_int * k)(*srcs), (ctypes.c_int * k)(*dsts),
                         (ctypes.c_void_p * k)(*sb), (ctypes.c_void_p * k)(*rb), (ctypes.c_size_t * k)(*sizes), 2,
                         ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                torch.cuda.synchronize()
                code = ctypes.c_int()
                lib.call("flagcxEmuGetError", emu.h, ctypes.byref(code))
                assert code.value == 0
                for s, d, _, _ in keep:
                    assert torch.equal(s[:nbytes], d[:nbytes])
    finally:
        emu.close()


def test_barrier_kernel(lib):
    emu = Emu(lib, 8)
    try:
        for _ in range(4):
            emu.coll("allreduce", "barrier", 1, None, None, 0, torch.int8)
    finally:
        emu.close()
