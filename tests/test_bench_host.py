"""Host-side pieces of bench.py that run without a GPU: workload lengths, the CPU sample,
the clock sampler's life cycle and the reference arm's JSON line."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_lengths_and_sample():
    sys.path.insert(0, ROOT)
    import bench

    lens = bench.make_lengths(1234)
    assert lens[:3] == [1, 7, 32768] and len(lens) == 16 and all(1 <= l <= 32768 for l in lens)
    assert bench.make_lengths(1234) == lens and bench.make_lengths(1235) != lens
    sample, nbytes, what = bench.make_cpu_sample("ragged", 3000)
    assert nbytes == 2 * 8 * sum(k.shape[1] for _, k, _ in sample) * 128 * 2
    assert sum(k.shape[1] for _, k, _ in sample) <= 3000 + 8


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
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] == "port"
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0
