"""Host-side pieces of bench.py that run without a GPU: workload lengths, the CPU sample,
the clock sampler's life cycle and the reference arm's JSON line."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_lengths_and_sample():
    sys.path.insert(0, ROOT)
    import bench

    lens = bench.make_lengths(1234)
    assert lens[:3] == [1, 7, 32768] and len(lens) == 16 and all(1 <= l <= 32768 for l in lens)
    assert bench.make_lengths(1234) == lens and bench.make_lengths(1235) != lens
    # the seeded sample: deterministic per (workload, sequence, head), lengths of the batch
    assert bench.sample_indices("ragged") == [0, 1, 2, 5]
    q, k, v = bench.sample_sequence("ragged", 5)
    assert q.shape == (32, 128) and k.shape == (8, lens[5], 128) == v.shape
    q2, k2, _ = bench.sample_sequence("ragged", 5, heads=[3])
    assert torch.equal(q2, q[12:16]) and torch.equal(k2[0], k[3])
    # the same description on both arms; shards divide the bytes, replicas do not
    assert bench.static_config("headshard", 8) == bench.static_config("headshard", 8)
    assert bench.rank_bytes("headshard", 8) * 8 == bench.rank_bytes("headshard", 1) == 2 ** 31
    assert bench.rank_bytes("single", 8) == 67108864 and bench.kv_sets("single", 1) == 8
    assert bench.kv_sets("headshard", 1) == 1 and bench.kv_sets("seqshard", 8) == 8


def test_clock_sampler_lifecycle():
    sys.path.insert(0, ROOT)
    import bench

    s = bench.ClockSampler(0)  # no NVML device here: must start and stop cleanly anyway
    s.start()
    out = s.stop()
    assert set(out) >= {"sm_mhz", "sm_max_mhz", "reasons"}


def test_reference_arm_json_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                        "--steps", "1", "--warmup", "1", "--workload", "single"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads([l for l in r.stdout.splitlines() if l.startswith("{")][-1])
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] in ("reference", "port")
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0
    sys.path.insert(0, ROOT)
    import bench

    assert line["config"] == bench.static_config("single", 1)
