"""Build recipe for the native library: one nvcc call, sm_100a only, output in-tree.

    python -m gqa_decode_b200.build            # build if sources are newer than the .so
    python -m gqa_decode_b200.build --force
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libgqa_decode_b200.so")
INCLUDE = os.path.join(os.path.dirname(PKG_DIR), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
]


def _sources():
    out = [os.path.join(INCLUDE, "gqa_decode_b200.h")]
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cu", ".cuh", ".h")):
            out.append(os.path.join(CSRC, name))
    return out


def needs_build() -> bool:
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    return any(os.path.getmtime(s) > built for s in _sources())


def build(force: bool = False, verbose: bool = False, defines=(), output: str = "") -> str:
    """Compile csrc/*.cu into lib/libgqa_decode_b200.so and return its path.  `defines`
    (macro definitions) together with `output` build a differently configured library
    elsewhere, e.g. -DGQA_PROFILE_WAITS for the diagnostics counters; such a library is
    selected at run time through the environment variable GQA_DECODE_B200_LIB."""
    if output:
        return _compile(output, verbose, defines)
    if not force and not needs_build():
        return LIB_PATH
    return _compile(LIB_PATH, verbose, defines)


def _compile(LIB_PATH: str, verbose: bool, defines) -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: cannot build libgqa_decode_b200.so")
    os.makedirs(os.path.dirname(os.path.abspath(LIB_PATH)), exist_ok=True)
    cus = [s for s in _sources() if s.endswith(".cu")]
    tmp = LIB_PATH + ".tmp"
    cmd = [nvcc, *NVCC_FLAGS, *(["-Xptxas", "-v"] if verbose else []), *[f"-D{d}" for d in defines],
           *cus, "-o", tmp]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("nvcc failed:\n" + proc.stdout + proc.stderr)
    if verbose:
        sys.stderr.write(proc.stderr)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    defs = [a[2:] for a in sys.argv[1:] if a.startswith("-D")]
    outs = [a[6:] for a in sys.argv[1:] if a.startswith("--out=")]
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, defines=defs,
                output=outs[0] if outs else ""))
