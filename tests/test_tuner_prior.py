"""The tuner's cost-model prior, queried without a GPU: small messages take the barrier-free LL forms, nothing is ever
planned beyond what a kind can hold, large messages get the whole grid, and estimates grow with the message."""
import pytest

from flagcx_b200.wrapper import FLAGCXLibrary

OPS = {"bcast": 2, "gather": 3, "scatter": 4, "reduce": 5, "allreduce": 6, "allgather": 7, "reducescatter": 8, "a2a": 9}
LL_KINDS = {"ar_ll", "move_ll", "rs_ll", "reduce_ll"}
FP32 = 7


@pytest.fixture(scope="module")
def lib(native_lib):
    return FLAGCXLibrary(native_lib)


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("mc", [False, True])
def test_prior_plans_are_sane(lib, n, mc):
    for name, op in OPS.items():
        last = 0.0
        for nbytes in (8, 64, 1024, 32768, 32772, 1 << 20, 16 << 20, 256 << 20, 1 << 30):
            kind, ctas, us = lib.tuner_prior_plan(op, nbytes, FP32, n, mc)
            assert 1 <= ctas <= 128, (name, nbytes, kind, ctas)
            assert us > 0
            if nbytes <= 64:
                assert kind in LL_KINDS, (name, nbytes, kind)
            if nbytes > 32768:
                assert kind not in LL_KINDS, (name, nbytes, kind)  # an LL slot holds 32 KiB of payload
            if not mc:
                assert "nvls" not in kind
            if nbytes >= (256 << 20):
                assert ctas >= 64, (name, nbytes, kind, ctas)
            assert us >= last * 0.9, (name, nbytes, us, last)  # a change of kind may dip a little
            last = us


def test_prior_rejects_bad_world():
    lib = FLAGCXLibrary()
    with pytest.raises(Exception):
        lib.tuner_prior_plan(6, 1024, FP32, 9, True)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_prior_sends_peer_visible_buffers_to_zero_copy_kinds(n):
    """What the multi-GPU tests rely on: for buffers every rank can see, the cost model picks the zero-copy kinds from a
    megabyte up, with and without the switch, and respects a CTA budget."""
    lib = FLAGCXLibrary()
    for mc in (True, False):
        for op, want in ((OPS["allreduce"], "ar_zc"), (OPS["reducescatter"], "rs_zc"), (OPS["allgather"], "move_zc")):
            kind, ctas, us = lib.tuner_prior_plan_ex(op, 300007 * 4, FP32, n, mc, True, 8)
            assert kind == want and 1 <= ctas <= 8 and us > 0, (n, mc, op, kind, ctas)
        kind, ctas, _ = lib.tuner_prior_plan_ex(OPS["allreduce"], 64, FP32, n, mc, True, 8)
        assert kind in LL_KINDS, kind


def test_copy_engine_kind_is_offered_on_two_ranks_only():
    """The copy-engine movers passed their multi-GPU test on two GPUs only: beyond that the prior must not pick them
    (FLAGCX_COPY_ENGINE=1 lifts the restriction; it is read once per process and is not set here)."""
    import os
    assert os.environ.get("FLAGCX_COPY_ENGINE") in (None, "0")
    lib = FLAGCXLibrary()
    seen = {n: set() for n in (2, 3, 4, 8)}
    for n in seen:
        for op in (OPS["bcast"], OPS["scatter"], OPS["allgather"], OPS["a2a"]):
            for lg in range(10, 33):
                for budget in (0, 8, 16):
                    seen[n].add(lib.tuner_prior_plan_ex(op, 1 << lg, FP32, n, True, True, budget)[0])
    assert "move_ce" in seen[2]
    for n in (3, 4, 8):
        assert "move_ce" not in seen[n], n
