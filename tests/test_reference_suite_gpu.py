"""The reference project's own test files, run unmodified against this package.

``import gqa_decode`` resolves to the alias package at the repository root, so the reference's
assertions (its tolerances: tests/test_correctness.py:30-31, test_edge_cases.py:17,29,
test_fp8.py:49-56,87, test_persistent.py:38-39 of the reference) grade the sm_100a kernels.
The files are looked for in the reference checkout next to this repository's reference
install (``baseline/_ref/tests``; ``__graft_entry__.build()`` places an unmodified copy there
when a reference checkout is present) and are never part of this repository.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CANDIDATES = [os.path.join(ROOT, "baseline", "_ref", "tests")] + (
    [os.path.join(os.environ["GQA_REFERENCE_ROOT"], "tests")] if "GQA_REFERENCE_ROOT" in os.environ else [])
FILES = ["test_correctness.py", "test_edge_cases.py", "test_fp8.py", "test_persistent.py"]


def test_reference_test_files_pass_in_place():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    where = next((c for c in CANDIDATES if all(os.path.exists(os.path.join(c, f)) for f in FILES)), None)
    if where is None:
        pytest.skip("the reference's test files are not present on this machine")
    env = dict(os.environ, PYTHONPATH=ROOT, PYTHONDONTWRITEBYTECODE="1")
    r = subprocess.run(
        [sys.executable, "-m", "pytest", "-p", "no:cacheprovider", "-q", "-x", "--rootdir", where,
         *[os.path.join(where, f) for f in FILES]],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=1500)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert " passed" in r.stdout and "skipped" not in r.stdout.splitlines()[-1], tail
