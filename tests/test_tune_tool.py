"""Offline tuning tool: candidate legality, selection of the fastest variant per size bucket, and the file format
that the library's loader scans (csrc/core/tuner.cc, Tuner::load)."""
import re

from flagcx_b200.tools import tune

LINE = re.compile(r'^ \{"op": (\d+), "log2_bytes": (\d+), "nranks": (\d+), "kind": "([a-z_0-9]+)", "nctas": (\d+), "us": ([0-9.]+)\},?$')


def test_buckets_and_legality():
    assert tune.bucket(1) == 0 and tune.bucket(2) == 1 and tune.bucket(3) == 2 and tune.bucket(32768) == 15 and tune.bucket(32769) == 16
    assert tune.key_bytes("allgather", 1 << 20, 8) == 1 << 17 and tune.key_bytes("allreduce", 1 << 20, 8) == 1 << 20
    assert tune.legal("allreduce", "ar_ll", 32768, True) and not tune.legal("allreduce", "ar_ll", 32769, True)
    assert not tune.legal("allreduce", "ar_nvls", 1 << 20, False) and tune.legal("allreduce", "ar_nvls", 1 << 20, True)
    assert not tune.legal("allreduce", "ar_oneshot", (8 << 20) + 4, True)
    assert tune.cta_choices("move_ll") == (1, 2, 4) and 128 in tune.cta_choices("ag")


def test_fastest_variant_per_bucket_and_file_format(tmp_path):
    rows = [
        {"op": "allreduce", "kind": "ar_ll", "nctas": 2, "bytes": 1024, "time_us": 10.0, "wrong": 0},
        {"op": "allreduce", "kind": "ar_oneshot", "nctas": 8, "bytes": 1024, "time_us": 12.0, "wrong": 0},
        {"op": "allreduce", "kind": "ar_twoshot", "nctas": 128, "bytes": 1 << 28, "time_us": 700.0, "wrong": 0},
        {"op": "allreduce", "kind": "ar_nvls", "nctas": 128, "bytes": 1 << 28, "time_us": 650.0, "wrong": 0},
        {"op": "allreduce", "kind": "ar_nvls", "nctas": 64, "bytes": 1 << 28, "time_us": 600.0, "wrong": 3},  # wrong result: ignored
        {"op": "allgather", "kind": "ag", "nctas": 128, "bytes": 8 << 20, "time_us": 40.0, "wrong": 0},
    ]
    entries = tune.build_cache(rows, 8)
    by = {(e["op"], e["log2_bytes"]): e for e in entries}
    assert by[(6, 10)]["kind"] == "ar_ll" and by[(6, 10)]["nctas"] == 2
    assert by[(6, 28)]["kind"] == "ar_nvls" and by[(6, 28)]["nctas"] == 128
    assert by[(7, 20)]["kind"] == "ag"  # 8 MiB over 8 ranks: keyed by the 1 MiB piece
    path = tmp_path / "cache.json"
    tune.write_cache(entries, path)
    lines = path.read_text().splitlines()
    assert lines[0] == "[" and lines[-1] == "]"
    for ln in lines[1:-1]:
        assert LINE.match(ln), ln
    assert not lines[-2].endswith(",")
