"""fcxColSumNoAlloc, the column-sum entry point that allocates nothing.

Some users of the fused kernels cannot allocate device memory when they need a
bias gradient: a server whose own pool owns the whole GPU, a loop that must
not pay for the synchronisation inside cudaMalloc/cudaFree, a caller without
PyTorch's caching allocator.  For them the library carries a fixed 1 MiB
scratch array and exposes one C symbol that uses it.  This test calls that
symbol the way such a user would (ctypes, raw pointers, the current stream),
twice in a row, and checks both results against the regular entry point
(`col_sum`, which takes its scratch from the caller).  The file name sorts
last so that it runs after every other test; it also passes on its own.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    import flagcx_b200
    flagcx_b200.native()  # makes sure the extension is built and its dependencies are loaded
    lib = ctypes.CDLL(flagcx_b200.lib_path("_flagcx_torch.so"))
    lib.fcxColSumNoAlloc.restype = ctypes.c_int
    lib.fcxColSumNoAlloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.fcxNoAllocErrorString.restype = ctypes.c_char_p
    lib.fcxNoAllocErrorString.argtypes = [ctypes.c_int]
    return lib


def test_no_alloc_column_sum_matches_regular_entry_point_twice():
    import flagcx_b200
    nat = flagcx_b200.native()
    lib = _lib()
    torch.manual_seed(0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    first = True
    for M, C in ((4096, 1024), (8192, 4096)):  # second call reuses (and overwrites) the same scratch
        a = torch.randn(M, C, device="cuda").bfloat16()
        out = torch.empty(C, dtype=torch.bfloat16, device="cuda")
        # Free device memory as the driver reports it (cudaMemGetInfo): unlike PyTorch's own counters it
        # would show a cudaMalloc made behind PyTorch's back.  The first call on a device also looks up the
        # scratch address, so the comparison brackets a call that comes after one has already been made.
        if first:
            rc = lib.fcxColSumNoAlloc(a.data_ptr(), out.data_ptr(), M, C, 0, stream)
            assert rc == 0, lib.fcxNoAllocErrorString(rc).decode()
            first = False
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        rc = lib.fcxColSumNoAlloc(a.data_ptr(), out.data_ptr(), M, C, 0, stream)
        assert rc == 0, lib.fcxNoAllocErrorString(rc).decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, (free_before, free_after)
        ref = nat.col_sum(a)
        torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
        exact = a.float().sum(0)
        err = (out.float() - exact).abs().max() / (exact.abs().max() + 1e-6)
        assert err < 3e-2, err


def test_no_alloc_refuses_shapes_beyond_its_scratch():
    lib = _lib()
    a = torch.zeros(64, 64, device="cuda", dtype=torch.bfloat16)
    out = torch.zeros(64, device="cuda", dtype=torch.bfloat16)
    # 32 row slices x 16384 columns = 524288 floats > 262144
    rc = lib.fcxColSumNoAlloc(a.data_ptr(), out.data_ptr(), 1 << 20, 16384, 0, None)
    assert rc == -1 and b"scratch" in lib.fcxNoAllocErrorString(rc)
    assert lib.fcxColSumNoAlloc(a.data_ptr(), out.data_ptr(), 64, 100, 0, None) == -2
    assert lib.fcxColSumNoAlloc(None, out.data_ptr(), 64, 64, 0, None) == -3
    # an odd byte offset into the matrix: refused, nothing launched
    assert lib.fcxColSumNoAlloc(a.data_ptr() + 2, out.data_ptr(), 32, 64, 0, None) == -4
    assert b"aligned" in lib.fcxNoAllocErrorString(-4)
