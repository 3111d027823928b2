"""Host-side decisions of the tcgen05 GEMM launchers, checked without a GPU: the K split never leaves a piece empty,
and the CTA-pair kernel is chosen for shapes that fill its 256-row tiles."""
import ctypes

import pytest


@pytest.fixture(scope="module")
def ext():
    import flagcx_b200
    mod = flagcx_b200.native()  # imports torch first, then the extension (needs no GPU to load)
    lib = ctypes.CDLL(mod.__file__)
    lib.fcxGemmPickSplitK.restype = ctypes.c_int
    lib.fcxGemmPickSplitK.argtypes = [ctypes.c_int] * 5
    lib.fcxGemmPairSuits.restype = ctypes.c_int
    lib.fcxGemmPairSuits.argtypes = [ctypes.c_int] * 3
    return lib


def test_split_k_never_leaves_a_piece_empty(ext):
    for n_k in range(1, 200):
        for requested in (0, 1, 2, 3, 5, 7, 8, 12, 64, 1000):
            for units in (1, 4, 16, 48, 54, 64, 100, 148, 300):
                s = ext.fcxGemmPickSplitK(requested, units, 74, n_k, 1024)
                assert 1 <= s <= n_k
                per = -(-n_k // s)
                assert (s - 1) * per < n_k, (n_k, requested, units, s)  # the last piece starts inside the K range
                if requested > 0:
                    assert s <= requested
    assert ext.fcxGemmPickSplitK(4, 16, 74, 128, 1023) == 1  # partial results are added two columns at a time


def test_split_k_fills_the_machine_for_weight_gradients(ext):
    # 16 tiles, K = 8192 tokens (128 K blocks), 74 CTA pairs: the launcher must cut K
    assert ext.fcxGemmPickSplitK(0, 16, 74, 128, 1024) >= 4
    # plenty of tiles: no split
    assert ext.fcxGemmPickSplitK(0, 384, 74, 16, 3072) == 1
    # a short K is never split by the launcher's own choice
    assert ext.fcxGemmPickSplitK(0, 16, 74, 16, 1024) == 1
    # 128 tiles on 74 pairs (1.73 waves): cut only when K is very long (the LM head's input gradient, K = 50304)
    assert ext.fcxGemmPickSplitK(0, 128, 74, 786, 1024) == 4
    assert ext.fcxGemmPickSplitK(0, 128, 74, 48, 1024) == 1


def test_pair_kernel_choice_by_shape(ext):
    assert ext.fcxGemmPairSuits(8192, 3072, 1024) == 1
    assert ext.fcxGemmPairSuits(1024, 1024, 8192) == 1
    assert ext.fcxGemmPairSuits(128, 4096, 4096) == 0      # one row block: the second CTA of a pair would idle
    assert ext.fcxGemmPairSuits(384, 4096, 4096) == 0      # 1.5 row blocks: a third of the pair tiles' rows are padding
    assert ext.fcxGemmPairSuits(8192, 128, 4096) == 0      # half a column block
