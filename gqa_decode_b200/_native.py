"""ctypes binding of libgqa_decode_b200.so (the C ABI in include/gqa_decode_b200.h).

There is no fallback: if the library is missing or a symbol is absent, importing a
kernel entry raises, and every compute call goes through the CUDA kernels.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_float, c_int32, c_int64, c_size_t, c_void_p

from . import build as _build

DTYPE_BF16, DTYPE_FP16, DTYPE_E4M3 = 0, 1, 2
LAYOUT_PADDED, LAYOUT_PACKED, LAYOUT_PAGED_HND, LAYOUT_PAGED_NHD = 0, 1, 2, 3
GATHER_HEADS, GATHER_SEQUENCE = 0, 1
FLAG_SEPARATE_MERGE = 1
FLAG_NO_MERGE = 2
FLAG_FP8_EXACT_V = 4
FLAG_WORK_STEALING = 8
FLAG_CLEAR_WORKSPACE = 16
FLAG_DEPENDENT_LAUNCH = 32
FLAG_TICKET_MERGE = 64
TIMESTAMP_WORDS = 12  # uint64 words per CTA in DecodeArgs.debug_timestamps
STATIC_SCRATCH_BYTES = 16 << 20  # GQA_STATIC_SCRATCH_BYTES

ERRORS = {
    -1: "bad argument (null/misaligned pointer or non-positive size)",
    -2: "unsupported head_dim / group size / dtype combination",
    -3: "workspace too small",
    -4: "cuTensorMapEncodeTiled unavailable or failed",
    -5: "size beyond a documented maximum",
    -6: "internal self-check failed",
}


class DecodeArgs(ctypes.Structure):
    """Mirror of gqa_decode_args_t."""

    _fields_ = [
        ("q", c_void_p), ("k", c_void_p), ("v", c_void_p), ("out", c_void_p),
        ("out_f32", c_void_p), ("out_lse", c_void_p), ("seq_lens", c_void_p),
        ("k_scale", c_void_p), ("v_scale", c_void_p),
        ("batch", c_int32), ("num_q_heads", c_int32), ("num_kv_heads", c_int32),
        ("head_dim", c_int32), ("max_seq_len", c_int32), ("total_rows", c_int64),
        ("q_dtype", c_int32), ("kv_dtype", c_int32), ("kv_layout", c_int32),
        ("num_splits", c_int32), ("num_ctas", c_int32), ("flags", c_int32),
        ("softmax_scale", c_float), ("workspace", c_void_p), ("workspace_bytes", c_size_t),
        ("stream", c_void_p),
        ("block_table", c_void_p), ("page_size", c_int32), ("block_table_stride", c_int32),
        ("wait_limit_ns", ctypes.c_uint64), ("debug_timestamps", c_void_p),
    ]


class GatherArgs(ctypes.Structure):
    """Mirror of gqa_gather_args_t."""

    _fields_ = [
        ("peer_out", POINTER(c_void_p)), ("peer_flags", POINTER(c_void_p)),
        ("world", c_int32), ("rank", c_int32), ("epoch", ctypes.c_uint32), ("mode", c_int32),
    ]


class AppendArgs(ctypes.Structure):
    """Mirror of gqa_append_args_t."""

    _fields_ = [
        ("k_new", c_void_p), ("v_new", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
        ("k_scale", c_void_p), ("v_scale", c_void_p), ("positions", c_void_p),
        ("block_table", c_void_p), ("saturated", c_void_p),
        ("batch", c_int32), ("num_kv_heads", c_int32), ("head_dim", c_int32),
        ("max_seq_len", c_int32), ("src_dtype", c_int32), ("kv_layout", c_int32),
        ("page_size", c_int32), ("block_table_stride", c_int32), ("stream", c_void_p),
    ]


# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "gqa_decode_version": (c_char_p, []),
    "gqa_decode_tile_rows": (ctypes.c_int, [c_int32, c_int32]),
    "gqa_decode_workspace_bytes": (
        ctypes.c_int, [c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, POINTER(c_size_t)]),
    "gqa_decode_workspace_layout": (
        ctypes.c_int, [c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, POINTER(c_size_t)]),
    "gqa_decode_workspace_reset": (ctypes.c_int, [c_void_p, c_size_t, c_void_p]),
    "gqa_decode_read_status": (ctypes.c_int, [c_void_p, c_void_p, POINTER(c_int32)]),
    "gqa_decode_attention": (ctypes.c_int, [POINTER(DecodeArgs)]),
    "gqa_decode_attention_persistent": (ctypes.c_int, [POINTER(DecodeArgs)]),
    "gqa_decode_attention_fp8": (ctypes.c_int, [POINTER(DecodeArgs)]),
    "gqa_decode_attention_static_scratch": (ctypes.c_int, [POINTER(DecodeArgs)]),
    "gqa_merge_partials": (
        ctypes.c_int,
        [c_void_p, c_void_p, c_int32, c_int64, c_int32, c_void_p, c_int32, c_void_p, c_void_p,
         c_void_p]),
    "gqa_quantize_kv_fp8": (
        ctypes.c_int, [c_void_p, c_int32, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "gqa_decode_attention_gather": (ctypes.c_int, [POINTER(DecodeArgs), POINTER(GatherArgs)]),
    "gqa_quantize_append_fp8": (ctypes.c_int, [POINTER(AppendArgs)]),
    "gqa_exchange_buffer_bytes": (c_size_t, [c_int32, c_int64, c_int32]),
    "gqa_sequence_exchange_bytes": (c_size_t, [c_int32, c_int64, c_int32]),
    "gqa_exchange_merge": (
        ctypes.c_int,
        [c_void_p, c_void_p, c_void_p, c_int32, c_int32, ctypes.c_uint32, c_int64, c_int32,
         c_void_p, c_int32, c_void_p, c_void_p, c_void_p, ctypes.c_uint64, c_void_p]),
    "gqa_select_num_splits": (ctypes.c_int, [c_int32, c_int32, c_int32, c_int32, c_int32]),
    "gqa_schedule_dump": (
        c_int64,
        [c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p,
         c_int64]),
    "gqa_schedule_dump_device": (
        ctypes.c_int,
        [c_void_p, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_int32, c_void_p,
         c_int64, c_void_p, c_void_p]),
}

_lib = None


class _NoRange:
    def __enter__(self):
        return None

    def __exit__(self, *exc):
        return False


class _NvtxRange:
    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        import torch

        torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        import torch

        torch.cuda.nvtx.range_pop()
        return False


_NO_RANGE = _NoRange()
TRACE_RANGES = os.environ.get("GQA_DECODE_B200_NVTX", "0") == "1"


def trace_range(name: str):
    """``with trace_range("gqa_decode:launch"): ...`` - an NVTX range around a host-side phase
    (launch of the decode kernel, the exchange, the collective + merge) when the environment
    variable GQA_DECODE_B200_NVTX=1 was set at import; a shared no-op object otherwise.  The
    pre-bound ``DecodePlan.run`` carries none: it is one C call."""
    return _NvtxRange(name) if TRACE_RANGES else _NO_RANGE


def lib_path() -> str:
    """Path of the shared library: the in-tree build, or the file named by the environment
    variable GQA_DECODE_B200_LIB (a differently configured build of the same sources)."""
    return os.environ.get("GQA_DECODE_B200_LIB") or _build.LIB_PATH


def load() -> ctypes.CDLL:
    """Load the shared library (once) and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not os.path.exists(path):
        raise RuntimeError(
            f"{path} is missing: build it with `python -m gqa_decode_b200.build` "
            "(needs nvcc). There is no non-CUDA fallback.")
    lib = ctypes.CDLL(path)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the .so is stale
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(code: int, what: str) -> None:
    """Turn a C-ABI return code into an exception."""
    if code == 0:
        return
    if code < 0:
        raise RuntimeError(f"{what}: {ERRORS.get(code, 'error')} (code {code})")
    raise RuntimeError(f"{what}: CUDA error {code}")
