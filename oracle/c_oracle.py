"""ctypes wrapper of oracle/gqa_oracle.c (TEST INFRASTRUCTURE ONLY; see that file)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(HERE, "_build", "libgqa_oracle.so")
_lib = None


def load():
    global _lib
    if _lib is None:
        src = os.path.join(HERE, "gqa_oracle.c")
        if not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(src):
            subprocess.run(["make", "-s", "-C", HERE], check=True)
        _lib = ctypes.CDLL(_LIB)
        _lib.gqa_oracle_attend.restype = ctypes.c_int
    return _lib


def _kind(t: torch.Tensor) -> int:
    return {torch.bfloat16: 0, torch.float16: 1, torch.float8_e4m3fn: 2}[t.dtype]


def attend(q, k, v, k_scale=None, v_scale=None, threads=None):
    """q [Hq, D]; k, v [Hkv, S, D] (bf16 / fp16 / e4m3 + per-head scales), CPU tensors.
    Returns (out float64 [Hq, D], lse float64 [Hq]) accumulated in float64."""
    lib = load()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    hq, d = q.shape
    hkv, s, _ = k.shape
    out = np.zeros((hq, d), dtype=np.float64)
    lse = np.zeros(hq, dtype=np.float64)
    ks = None if k_scale is None else k_scale.float().contiguous()
    vs = None if v_scale is None else v_scale.float().contiguous()
    rc = lib.gqa_oracle_attend(
        ctypes.c_void_p(q.data_ptr()), _kind(q), ctypes.c_void_p(k.data_ptr()),
        ctypes.c_void_p(v.data_ptr()), _kind(k),
        ctypes.c_void_p(ks.data_ptr() if ks is not None else None),
        ctypes.c_void_p(vs.data_ptr() if vs is not None else None),
        hq, hkv, ctypes.c_long(s), d, ctypes.c_long(s * d),
        ctypes.c_void_p(out.ctypes.data), ctypes.c_void_p(lse.ctypes.data),
        int(threads or os.cpu_count() or 1))
    if rc:
        raise RuntimeError(f"gqa_oracle_attend failed ({rc})")
    return torch.from_numpy(out), torch.from_numpy(lse)
