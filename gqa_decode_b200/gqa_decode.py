"""Host API of the B200 GQA decode-attention library.

Mirrors the public surface of alityb/gqa-decode's ``gqa_decode/gqa_decode.py`` (same
function names, keyword arguments and ``ValueError`` messages) and adds a batched /
ragged entry point.  All attention math runs in the sm_100a kernels behind the C ABI
(``include/gqa_decode_b200.h``); this module validates arguments, owns a reusable
device workspace and fills in the argument struct.  PyTorch is used for device
memory and streams only.
"""
from __future__ import annotations

import ctypes
import functools
import threading
import weakref
from dataclasses import dataclass
from typing import Optional

import torch

from . import _native

DEFAULT_BLOCK_SEQ = 16
DEFAULT_TARGET_BLOCKS_PER_SM = 16
NUM_SMS_H100_SXM = 132
SMEM_PAD = 8


@dataclass(frozen=True)
class GQADecodeConfig:
    """Tuning knobs of the reference (gqa_decode/gqa_decode.py:29-33), kept for signature
    compatibility.  The B200 kernels choose their own tile size and CTA count; the
    fields only influence :func:`select_num_splits`, exactly as in the reference."""

    block_seq: int = DEFAULT_BLOCK_SEQ
    smem_pad: int = SMEM_PAD
    target_blocks_per_sm: int = DEFAULT_TARGET_BLOCKS_PER_SM


# ---------------------------------------------------------------------------
# Functions of the reference API that are plain tensor algebra
# ---------------------------------------------------------------------------

def reference_gqa_decode(q, k_cache, v_cache, num_kv_heads=None):
    """Exact float32 attention in PyTorch ops, on whatever device the tensors live on.

    Part of the reference's public API (gqa_decode/gqa_decode.py:36-66) and what
    ``backend="torch"`` selects.  It is never chosen automatically: the CUDA kernels
    have no fallback.
    """
    if q.dim() != 2 or k_cache.dim() != 3 or v_cache.dim() != 3:
        raise ValueError(
            "Expected q=(num_q_heads, head_dim), k/v=(num_kv_heads, seq_len, head_dim)"
        )
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have identical shapes")
    num_q_heads, head_dim = q.shape
    kv_heads, _, kv_head_dim = k_cache.shape
    if kv_head_dim != head_dim:
        raise ValueError("Q/K/V head_dim mismatch")
    if num_kv_heads is None:
        num_kv_heads = kv_heads
    if num_kv_heads != kv_heads:
        raise ValueError("num_kv_heads must match k_cache.shape[0]")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    owner = torch.arange(num_q_heads, device=q.device) // (num_q_heads // num_kv_heads)
    logits = torch.einsum("hd,hsd->hs", q.float(), k_cache.float()[owner]) * head_dim ** -0.5
    weights = torch.softmax(logits, dim=-1)
    return torch.einsum("hs,hsd->hd", weights, v_cache.float()[owner]).to(dtype=q.dtype)


def select_num_splits(
    num_kv_heads: int,
    seq_len: int,
    block_seq: int = DEFAULT_BLOCK_SEQ,
    target_blocks_per_sm: int = DEFAULT_TARGET_BLOCKS_PER_SM,
    num_sms: int = NUM_SMS_H100_SXM,
) -> int:
    """The reference's one-wave split heuristic (gqa_decode/gqa_decode.py:80-102),
    evaluated by the native library.  The B200 kernels do not need it (their default is
    the balanced persistent schedule); it is kept because callers use it to pick an
    explicit ``num_splits``."""
    if num_kv_heads <= 0:
        raise ValueError("num_kv_heads must be positive")
    r = _native.load().gqa_select_num_splits(
        num_kv_heads, seq_len, block_seq, target_blocks_per_sm, num_sms)
    if r < 0:
        _native.check(r, "gqa_select_num_splits")
    return r


def reduce_partials(partial_out, partial_max, partial_sum, num_q_heads, num_splits, head_dim):
    """Combine split-K partials given in the reference's three-tensor format
    (gqa_decode/gqa_decode.py:647-669): un-normalised accumulators ``[Hq*splits, D]`` and
    running max / sum broadcast over ``D`` (column 0 is read).  Tensor ops on the
    tensors' own device; this is what ``reduction="python"`` runs."""
    out_dtype = partial_out.dtype
    m = partial_max[:, 0].reshape(num_q_heads, num_splits)
    l = partial_sum[:, 0].reshape(num_q_heads, num_splits)
    top = m.max(dim=1, keepdim=True).values
    w = torch.exp(m - top)
    denom = (l * w).sum(dim=1, keepdim=True)
    acc = partial_out.reshape(num_q_heads, num_splits, head_dim).float()
    return (torch.einsum("qsd,qs->qd", acc, w) / denom).to(out_dtype)


# ---------------------------------------------------------------------------
# Workspace
# ---------------------------------------------------------------------------

_DTYPE_CODE = {torch.bfloat16: _native.DTYPE_BF16, torch.float16: _native.DTYPE_FP16}

# The C library keeps no record of workspaces; this layer owns them and knows what they last
# held.  What a launch uses of its workspace must be zero at launch and kernels leave it
# zero, but where control words and partials lie depends on the launch geometry (sizes, CTA
# count, split count, merge mode): the "geometry key" below.  A launch whose key differs from
# the workspace's previous one, or whose workspace has unknown contents, carries
# GQA_FLAG_CLEAR_WORKSPACE.
_workspaces: dict = {}                       # (device type, index) -> [tensor, geometry key]
_caller_workspaces: dict = {}  # id(caller-owned tensor) -> (weak reference to it, geometry key)


@functools.lru_cache(maxsize=256)
def _workspace_need(batch, num_q_heads, num_kv_heads, head_dim, num_splits, num_ctas, device_index):
    """Bytes of workspace a launch geometry needs on a device (cached: the drop-in entry
    would otherwise ask the library on every call)."""
    need = ctypes.c_size_t(0)
    _native.check(
        _native.load().gqa_decode_workspace_bytes(
            batch, num_q_heads, num_kv_heads, head_dim, num_splits, num_ctas, ctypes.byref(need)),
        "gqa_decode_workspace_bytes")
    return need.value


def workspace_bytes(batch, num_q_heads, num_kv_heads, head_dim, num_splits=0, num_ctas=0) -> int:
    n = ctypes.c_size_t(0)
    _native.check(
        _native.load().gqa_decode_workspace_bytes(
            batch, num_q_heads, num_kv_heads, head_dim, num_splits, num_ctas, ctypes.byref(n)),
        "gqa_decode_workspace_bytes")
    return n.value


def _device_key(device: torch.device):
    return (device.type, device.index if device.index is not None else torch.cuda.current_device())


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """A zero-initialised scratch tensor per device, grown on demand and reused by
    every eager call on that device (calls that overlap on different streams must pass
    their own ``workspace=``)."""
    key = _device_key(device)
    entry = _workspaces.get(key)
    if entry is None or entry[0].numel() < nbytes:
        entry = [torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device), None]
        _workspaces[key] = entry
    return entry[0]


def _needs_clear(ws: torch.Tensor, device: torch.device, geometry) -> bool:
    """Record that `ws` is about to serve a launch of `geometry`; True if its control words
    must be cleared first (another geometry used it last, or its contents are unknown)."""
    entry = _workspaces.get(_device_key(device))
    if entry is not None and entry[0] is ws:
        clear = entry[1] is not None and entry[1] != geometry  # None: still all zeros
        entry[1] = geometry
        return clear
    # (keyed by identity: tensors compare element-wise, so they cannot key a weak dictionary)
    known = _caller_workspaces.get(id(ws))
    clear = known is None or known[0]() is not ws or known[1] != geometry
    if known is None or known[0]() is not ws:
        key = id(ws)
        _caller_workspaces[key] = (weakref.ref(ws, lambda _, key=key: _caller_workspaces.pop(key, None)), geometry)
    else:
        _caller_workspaces[id(ws)] = (known[0], geometry)
    return clear


def reset_workspace(workspace: Optional[torch.Tensor] = None, device=None) -> None:
    """Zero a workspace (default: the shared one of the device) on the current stream.  Needed
    after a launch that reported a non-zero status, whose tickets may be left half counted."""
    if workspace is None:
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        entry = _workspaces.get(_device_key(dev))
        if entry is None:
            return
        workspace, entry[1] = entry[0], None
    else:
        _caller_workspaces.pop(id(workspace), None)
    with torch.cuda.device(workspace.device):
        _native.check(
            _native.load().gqa_decode_workspace_reset(
                workspace.data_ptr(), workspace.numel() * workspace.element_size(),
                torch.cuda.current_stream(workspace.device).cuda_stream),
            "gqa_decode_workspace_reset")


def read_status(workspace: Optional[torch.Tensor] = None, device=None, reset_on_error: bool = True) -> int:
    """Synchronise and return the kernels' status word (0 = ok; non-zero = a bounded
    wait inside a kernel expired and the result of that call is invalid).  A workspace that
    reports an error is zeroed again (``reset_on_error``) so that the next launch on it starts
    from clean tickets."""
    if workspace is None:
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        workspace = _workspace(dev, 512)
        shared = True
    else:
        shared = False
    st = ctypes.c_int32(0)
    with torch.cuda.device(workspace.device):
        _native.check(
            _native.load().gqa_decode_read_status(
                workspace.data_ptr(), torch.cuda.current_stream(workspace.device).cuda_stream,
                ctypes.byref(st)),
            "gqa_decode_read_status")
    if st.value and reset_on_error:
        reset_workspace(None if shared else workspace, workspace.device)
    return st.value


# ---------------------------------------------------------------------------
# Batched entry (new) — everything else is a thin wrapper over it
# ---------------------------------------------------------------------------

def gqa_decode_attention_batched(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    seq_lens: Optional[torch.Tensor] = None,
    *,
    layout: str = "padded",
    k_scale: Optional[torch.Tensor] = None,
    v_scale: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
    num_ctas: int = 0,
    separate_merge: bool = False,
    softmax_scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    return_lse: bool = False,
    return_f32: bool = False,
    workspace: Optional[torch.Tensor] = None,
    max_seq_len: Optional[int] = None,
    num_kv_heads: Optional[int] = None,
    fp8_exact_v: bool = False,
    work_stealing: bool = False,
    block_table: Optional[torch.Tensor] = None,
    dependent_launch: bool = False,
    ticket_merge: bool = False,
    wait_limit_ns: int = 0,
    _timestamps: Optional[torch.Tensor] = None,
    _entry: str = "auto",
    _no_merge: bool = False,
    _plan_only: bool = False,
    _bind_shared_workspace: bool = False,
    _gather=None,
):
    """One decode step for a batch of sequences with individual KV lengths.

    q: ``[B, Hq, D]`` bf16/fp16.
    layout="padded": k/v ``[B, Hkv, Smax, D]``; ``seq_lens`` int32 ``[B]`` on the device
      (``None`` = all ``Smax``).
    layout="packed": k/v ``[Hkv * sum(len), D]`` where sequence ``b`` stores its
      ``[Hkv, len_b, D]`` slab after all earlier sequences; ``seq_lens``, ``num_kv_heads``
      and ``max_seq_len`` (a bound on every length) are required.
    layout="paged_hnd": k/v ``[num_pages, Hkv, page_size, D]``; layout="paged_nhd": k/v
      ``[num_pages, page_size, Hkv, D]``.  ``block_table`` int32 ``[B, max_pages]`` on the
      device names the page of every ``page_size`` consecutive keys of a sequence; entries
      past a sequence's last page are never read.  ``seq_lens`` is required;
      ``max_seq_len`` defaults to ``max_pages * page_size``.  ``page_size`` is a multiple of
      16 that divides the kernel's tile or is a multiple of it (any power of two >= 16 works).
    k/v dtype is q's dtype, or ``float8_e4m3fn`` with ``k_scale``/``v_scale`` fp32
    ``[B, Hkv]`` (per sequence and KV head, the reference's fp8_utils scheme).
    num_splits: ``None`` = balanced persistent schedule; ``K`` = K partials per
      (sequence, KV head).
    work_stealing: let CTAs that finish their static share steal work chunks from others
      (helps when SMs are shared with other work; makes the float32 summation order, hence
      the last bits of the result, depend on timing).  Default: static shares, results are
      bit-reproducible.
    fp8_exact_v: round every dequantised V element to the 16-bit type as
      ``dequantize_kv_fp8`` does (K always is); default applies the V scale to the fp32
      output instead, which is faster and differs only in that rounding.
    dependent_launch: launch with programmatic stream serialization, so that the kernel's
      prologue overlaps the end of the previous kernel on the stream (it waits for that kernel
      before reading inputs); for back-to-back decode steps.
    ticket_merge: detect complete groups with atomic tickets instead of letting the partials
      announce themselves (the default, which keeps atomics and fences off the critical path
      but needs the workspace's partial area to be zero at launch; this module sees to that).
    wait_limit_ns: bound on every wait inside the kernel (0 = two seconds); on expiry the
      status word (:func:`read_status`) is non-zero and the outputs are invalid.
    workspace: a caller-owned uint8 CUDA tensor of :func:`workspace_bytes` bytes instead of
      the shared per-device one; this module remembers what it last held and clears its
      control words when the launch geometry changes.
    Returns out ``[B, Hq, D]`` (q dtype), plus float32 output and/or natural-log LSE
    ``[B, Hq]`` when asked.  A sequence of length 0 yields zeros and LSE = -inf.
    """
    lib = _native.load()
    if q.dim() != 3:
        raise ValueError("Expected q=(batch, num_q_heads, head_dim)")
    if q.device.type != "cuda" or k_cache.device.type != "cuda" or v_cache.device.type != "cuda":
        raise ValueError("All tensors must be CUDA tensors")
    if q.dtype not in _DTYPE_CODE:
        raise ValueError("Only fp16 and bf16 are supported")
    fp8 = k_cache.dtype == torch.float8_e4m3fn
    if fp8:
        if v_cache.dtype != torch.float8_e4m3fn:
            raise ValueError("K/V must be float8_e4m3fn")
    elif k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("Q/K/V dtypes must match")
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    if not (q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("Q/K/V must be contiguous")
    batch, num_q_heads, head_dim = q.shape
    if layout == "padded":
        if k_cache.dim() != 4:
            raise ValueError("padded layout expects k/v=(batch, num_kv_heads, max_seq, head_dim)")
        kb, num_kv_heads, smax, kv_head_dim = k_cache.shape
        if kb != batch:
            raise ValueError("Q and K/V batch sizes differ")
        total_rows = batch * num_kv_heads * smax
        code_layout = _native.LAYOUT_PADDED
    elif layout == "packed":
        if k_cache.dim() != 2 or seq_lens is None or max_seq_len is None or num_kv_heads is None:
            raise ValueError(
                "packed layout expects k/v=(num_kv_heads*sum(len), head_dim), seq_lens, "
                "max_seq_len and num_kv_heads")
        total_rows, kv_head_dim = k_cache.shape
        smax = int(max_seq_len)
        code_layout = _native.LAYOUT_PACKED
    elif layout in ("paged_hnd", "paged_nhd"):
        if k_cache.dim() != 4 or block_table is None or seq_lens is None:
            raise ValueError(
                "paged layouts expect k/v=(num_pages, num_kv_heads, page_size, head_dim) or "
                "(num_pages, page_size, num_kv_heads, head_dim), block_table and seq_lens")
        if layout == "paged_hnd":
            num_pages, num_kv_heads, page_size, kv_head_dim = k_cache.shape
            code_layout = _native.LAYOUT_PAGED_HND
        else:
            num_pages, page_size, num_kv_heads, kv_head_dim = k_cache.shape
            code_layout = _native.LAYOUT_PAGED_NHD
        if (block_table.dtype != torch.int32 or block_table.device != q.device
                or block_table.dim() != 2 or block_table.shape[0] != batch):
            raise ValueError("block_table must be an int32 CUDA tensor of shape [batch, max_pages]")
        block_table = block_table.contiguous()
        tile = lib.gqa_decode_tile_rows(
            head_dim, _native.DTYPE_E4M3 if fp8 else _DTYPE_CODE[q.dtype])
        if page_size < 16 or page_size % 16 or (tile > 0 and page_size % tile and tile % page_size):
            raise ValueError(
                f"page_size must be a multiple of 16 that divides or is a multiple of {tile}")
        total_rows = num_pages * num_kv_heads * page_size
        smax = block_table.shape[1] * page_size if max_seq_len is None else int(max_seq_len)
        if smax > block_table.shape[1] * page_size:
            raise ValueError("max_seq_len exceeds what the block table can address")
    else:
        raise ValueError("layout must be 'padded', 'packed', 'paged_hnd' or 'paged_nhd'")
    if kv_head_dim != head_dim:
        raise ValueError("Q/K/V head_dim mismatch")
    if fp8:
        if k_scale is None or v_scale is None:
            raise ValueError("Scales must be [num_kv_heads]")
        if k_scale.numel() != batch * num_kv_heads or v_scale.numel() != batch * num_kv_heads:
            raise ValueError("Scales must be [num_kv_heads]")
        if k_scale.dtype != torch.float32 or v_scale.dtype != torch.float32:
            raise ValueError("Scales must be float32")
        k_scale = k_scale.contiguous()
        v_scale = v_scale.contiguous()
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    if num_q_heads // num_kv_heads > 16:
        raise ValueError("group size must be in [1, 16]")
    if head_dim not in ((64, 128) if fp8 else (64, 128, 256)):
        raise ValueError("head_dim must be 64, 128 or 256 (64 or 128 for FP8)")
    if seq_lens is not None:
        if seq_lens.dtype != torch.int32 or seq_lens.device != q.device or seq_lens.numel() != batch:
            raise ValueError("seq_lens must be an int32 CUDA tensor of shape [batch]")
        seq_lens = seq_lens.contiguous()
    splits = 0 if num_splits is None else int(num_splits)
    if splits < 0:
        raise ValueError("num_splits must be positive")

    dev = q.device
    need = _workspace_need(batch, num_q_heads, num_kv_heads, head_dim, splits, num_ctas,
                           _device_key(dev)[1])
    if workspace is not None:
        ws = workspace
    elif _plan_only and not _bind_shared_workspace:
        # a plan owns its workspace: fixed geometry, zero from the start, never needs clearing,
        # and nothing another launch does can disturb a captured graph that replays it
        ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    else:
        ws = _workspace(dev, need)
    ws_bytes = ws.numel() * ws.element_size()
    if ws_bytes < need:
        raise ValueError(f"workspace too small: need {need} bytes")
    mode = (bool(separate_merge), bool(_no_merge), bool(work_stealing), bool(ticket_merge))
    geometry = (batch, num_q_heads, num_kv_heads, head_dim, splits, num_ctas, mode, ws_bytes)
    clear = (workspace is not None or not _plan_only) and _needs_clear(ws, dev, geometry)
    if _bind_shared_workspace:
        clear = False  # decided call by call (see _single_sequence_call)
    if _gather is not None and _gather.mode == _native.GATHER_HEADS:
        out = None  # final rows go to the gathered buffers of every rank (distributed.HeadGather)
    elif out is None:
        out = torch.empty_like(q)
    out_f32 = torch.empty(q.shape, dtype=torch.float32, device=dev) if return_f32 else None
    out_lse = torch.empty(q.shape[:2], dtype=torch.float32, device=dev) if return_lse else None

    a = _native.DecodeArgs()
    a.q, a.k, a.v = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    a.out = out.data_ptr() if out is not None else None
    a.out_f32 = out_f32.data_ptr() if out_f32 is not None else None
    a.out_lse = out_lse.data_ptr() if out_lse is not None else None
    a.seq_lens = seq_lens.data_ptr() if seq_lens is not None else None
    a.k_scale = k_scale.data_ptr() if fp8 else None
    a.v_scale = v_scale.data_ptr() if fp8 else None
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = batch, num_q_heads, num_kv_heads, head_dim
    a.max_seq_len, a.total_rows = smax, total_rows
    a.q_dtype = _DTYPE_CODE[q.dtype]
    a.kv_dtype = _native.DTYPE_E4M3 if fp8 else a.q_dtype
    a.kv_layout = code_layout
    a.num_splits, a.num_ctas = splits, num_ctas
    a.flags = (_native.FLAG_SEPARATE_MERGE if separate_merge else 0) | (
        _native.FLAG_NO_MERGE if _no_merge else 0) | (
        _native.FLAG_FP8_EXACT_V if fp8_exact_v else 0) | (
        _native.FLAG_WORK_STEALING if work_stealing else 0) | (
        _native.FLAG_CLEAR_WORKSPACE if clear else 0) | (
        _native.FLAG_TICKET_MERGE if ticket_merge else 0) | (
        _native.FLAG_DEPENDENT_LAUNCH if dependent_launch else 0)
    a.wait_limit_ns = int(wait_limit_ns)
    a.debug_timestamps = _timestamps.data_ptr() if _timestamps is not None else None
    a.softmax_scale = 0.0 if softmax_scale is None else float(softmax_scale)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws_bytes
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    if code_layout >= _native.LAYOUT_PAGED_HND:
        a.block_table = block_table.data_ptr()
        a.page_size, a.block_table_stride = page_size, block_table.shape[1]
    if _gather is not None:
        gather_ref = ctypes.byref(_gather)
        entry = lib.gqa_decode_attention_gather
        fn = lambda ref: entry(ref, gather_ref)  # noqa: E731
    elif fp8:
        fn = lib.gqa_decode_attention_fp8
    elif _entry == "persistent":
        fn = lib.gqa_decode_attention_persistent
    else:
        fn = lib.gqa_decode_attention
    extras = tuple(t for t in (out_f32, out_lse) if t is not None)
    result = (out, *extras) if extras else out
    if _plan_only:
        keep = (q, k_cache, v_cache, seq_lens, k_scale, v_scale, ws, out, out_f32, out_lse, block_table,
                _gather, _timestamps)
        plan = DecodePlan(fn, a, dev, result, keep, ws)
        plan._geometry = geometry
        return plan
    with torch.cuda.device(dev), _native.trace_range("gqa_decode:launch"):
        _native.check(fn(ctypes.byref(a)), "gqa_decode_attention")
    return result


class DecodePlan:
    """A validated, fully bound decode step: ``run()`` is one C call (two tensor-map
    encodes and one kernel launch) on the current stream of the plan's device, with no
    Python-side checks or allocations.  The tensors given to :func:`plan_decode` are
    read and written in place on every run, so a serving loop updates K/V/``seq_lens``
    storage and calls ``run()`` again.  The stream is re-read on each run.  Unless the caller
    passed ``workspace=``, the plan has a workspace of its own (``plan.workspace``), so plans
    may be captured in CUDA graphs and replayed in any order with other launches in between;
    ``status()`` reads its status word."""

    def __init__(self, fn, args, device, result, keep, workspace):
        self._fn, self._args, self.device, self.result, self._keep = fn, args, device, result, keep
        self._ref = ctypes.byref(args)
        self.workspace = workspace

    def run(self):
        self._args.stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self._fn(self._ref)
        if rc:
            _native.check(rc, "gqa_decode_attention")
        # a caller-owned workspace of unknown contents is cleared by the first run only
        self._args.flags &= ~_native.FLAG_CLEAR_WORKSPACE
        return self.result

    def status(self) -> int:
        """Synchronise and return the status word of the plan's workspace (0 = ok)."""
        st = read_status(self.workspace, reset_on_error=True)
        return st


def plan_decode(q, k_cache, v_cache, seq_lens=None, **kw) -> DecodePlan:
    """Validate once and return a :class:`DecodePlan` (same arguments as
    :func:`gqa_decode_attention_batched`; the output tensors are allocated here and
    reused by every ``run()``).  The caller must have the plan's device current."""
    return gqa_decode_attention_batched(q, k_cache, v_cache, seq_lens, _plan_only=True, **kw)


def _partials_for_python_reduction(q, k, v, k_scale, v_scale, splits):
    """Run the kernel with GQA_FLAG_NO_MERGE and return its partials re-expressed in the
    reference's three-tensor format for :func:`reduce_partials`: acc = normalised O,
    max = LSE, sum = 1 (exp(LSE_i - M) * O_i summed over i, divided by the sum of
    exp(LSE_i - M), is the same merge)."""
    num_q_heads, head_dim = q.shape
    num_kv_heads = k.shape[0]
    g = num_q_heads // num_kv_heads
    need = workspace_bytes(1, num_q_heads, num_kv_heads, head_dim, splits, 0)
    ws = _workspace(q.device, need)
    gqa_decode_attention_batched(
        q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), None,
        k_scale=None if k_scale is None else k_scale.view(1, -1),
        v_scale=None if v_scale is None else v_scale.view(1, -1),
        num_splits=splits, workspace=ws, _no_merge=True)
    off = (ctypes.c_size_t * 6)()
    _native.check(
        _native.load().gqa_decode_workspace_layout(
            1, num_q_heads, num_kv_heads, head_dim, splits, 0, off),
        "gqa_decode_workspace_layout")
    slots = num_kv_heads * splits
    lse = ws[off[3]: off[3] + slots * g * 4].view(torch.float32).view(num_kv_heads, splits, g)
    o = ws[off[4]: off[4] + slots * g * head_dim * 4].view(torch.float32).view(
        num_kv_heads, splits, g, head_dim)
    # reference row index = q_head * splits + split (gqa_decode/gqa_decode.py:392-393)
    acc = o.permute(0, 2, 1, 3).reshape(num_q_heads * splits, head_dim).to(q.dtype)
    mx = lse.permute(0, 2, 1).reshape(num_q_heads * splits, 1).expand(-1, head_dim)
    one = torch.ones_like(mx)
    return acc, mx, one


# ---------------------------------------------------------------------------
# Reference-compatible single-sequence entries
# ---------------------------------------------------------------------------

def gqa_decode_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    num_splits: Optional[int] = None,
    config: Optional[GQADecodeConfig] = None,
    backend: str = "cute",
    reduction: str = "fused",
) -> torch.Tensor:
    """Drop-in for gqa_decode/gqa_decode.py:672-762.

    ``backend``: "cute" (the reference's name for its kernel path) and "cuda" both run
    the sm_100a kernels; "torch" is the caller's explicit request for
    :func:`reference_gqa_decode`.  ``num_splits=None`` uses the balanced persistent
    schedule; an integer forces that many partials per KV head.  ``reduction="fused"``
    merges inside the launch, ``"python"`` merges the partials with tensor ops
    (:func:`reduce_partials`).
    """
    if q.dim() != 2 or k_cache.dim() != 3 or v_cache.dim() != 3:
        raise ValueError(
            "Expected q=(num_q_heads, head_dim), k/v=(num_kv_heads, seq_len, head_dim)"
        )
    if q.device.type != "cuda" or k_cache.device.type != "cuda" or v_cache.device.type != "cuda":
        raise ValueError("All tensors must be CUDA tensors")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("Only fp16 and bf16 are supported")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("Q/K/V dtypes must match")
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    if not (q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("Q/K/V must be contiguous")
    num_q_heads, head_dim = q.shape
    num_kv_heads, _, kv_head_dim = k_cache.shape
    if kv_head_dim != head_dim:
        raise ValueError("Q/K/V head_dim mismatch")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    if backend not in {"cute", "cuda", "torch"}:
        raise ValueError("backend must be one of {'cute', 'torch'}")
    if reduction not in {"fused", "python"}:
        raise ValueError("reduction must be one of {'fused', 'python'}")
    if backend == "torch":
        return reference_gqa_decode(q, k_cache, v_cache, num_kv_heads=num_kv_heads)
    if reduction == "python":
        cfg = config or GQADecodeConfig()
        splits = num_splits if num_splits is not None else select_num_splits(
            num_kv_heads, k_cache.shape[1], cfg.block_seq, cfg.target_blocks_per_sm)
        acc, mx, one = _partials_for_python_reduction(q, k_cache, v_cache, None, None, splits)
        return reduce_partials(acc, mx, one, num_q_heads, splits, head_dim)
    return _single_sequence_call(q, k_cache, v_cache, num_splits)


# Argument blocks of the drop-in entry, one per (device, dtype, shapes, split count): a decode
# loop calls it with the same shapes every step, and a kernel of twenty microseconds leaves
# no room for re-validating and re-filling two dozen struct fields in Python each time.
# (Per thread: the block is patched in place before every call.)
_single_calls_tls = threading.local()


def _single_sequence_call(q, k_cache, v_cache, num_splits):
    dev = q.device
    _single_calls = _single_calls_tls.__dict__.setdefault("blocks", {})
    key = (dev.index, q.dtype, q.shape, k_cache.shape, num_splits)
    entry = _single_calls.get(key)
    if entry is None:
        # first call with this signature: the general path validates what is left to validate
        # and allocates the shared workspace; then bind a block for the calls that follow
        out = gqa_decode_attention_batched(
            q.unsqueeze(0), k_cache.unsqueeze(0), v_cache.unsqueeze(0), None, num_splits=num_splits)
        plan = gqa_decode_attention_batched(
            q.unsqueeze(0), k_cache.unsqueeze(0), v_cache.unsqueeze(0), None, num_splits=num_splits,
            _plan_only=True, _bind_shared_workspace=True)
        if len(_single_calls) > 64:
            _single_calls.clear()
        _single_calls[key] = (plan._args, plan._ref, plan._fn, plan._geometry)
        return out.squeeze(0)
    a, ref, fn, geometry = entry
    # the shared workspace may have grown or served another geometry since
    ws_entry = _workspaces.get((dev.type, dev.index))
    if ws_entry is None or ws_entry[0].data_ptr() != a.workspace:
        del _single_calls[key]
        return _single_sequence_call(q, k_cache, v_cache, num_splits)
    clear = ws_entry[1] is not None and ws_entry[1] != geometry
    ws_entry[1] = geometry
    out = torch.empty_like(q)
    a.q, a.k, a.v, a.out = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr()
    a.flags = _native.FLAG_CLEAR_WORKSPACE if clear else 0
    a.stream = torch.cuda.current_stream(dev).cuda_stream
    if dev.index != torch.cuda.current_device():
        with torch.cuda.device(dev):
            rc = fn(ref)
    else:
        rc = fn(ref)
    if rc:
        _native.check(rc, "gqa_decode_attention")
    return out


def gqa_decode_attention_persistent(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    *,
    config: Optional[GQADecodeConfig] = None,
) -> torch.Tensor:
    """Drop-in for gqa_decode/gqa_decode.py:1365-1446: one persistent CTA per SM, each
    walking an equal contiguous share of the (KV head, tile) list."""
    if q.dim() != 2 or k_cache.dim() != 3 or v_cache.dim() != 3:
        raise ValueError(
            "Expected q=(num_q_heads, head_dim), k/v=(num_kv_heads, seq_len, head_dim)"
        )
    if q.device.type != "cuda":
        raise ValueError("All tensors must be CUDA tensors")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("Only fp16 and bf16 are supported")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise ValueError("Q/K/V dtypes must match")
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    if not (q.is_contiguous() and k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("Q/K/V must be contiguous")
    num_q_heads, head_dim = q.shape
    num_kv_heads, _, kv_head_dim = k_cache.shape
    if kv_head_dim != head_dim:
        raise ValueError("Q/K/V head_dim mismatch")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    out = gqa_decode_attention_batched(
        q.unsqueeze(0), k_cache.unsqueeze(0), v_cache.unsqueeze(0), None, _entry="persistent")
    return out.squeeze(0)


def gqa_decode_attention_fp8(
    q: torch.Tensor,
    k_fp8: torch.Tensor,
    v_fp8: torch.Tensor,
    k_scale: torch.Tensor,
    v_scale: torch.Tensor,
    *,
    num_splits: Optional[int] = None,
    config: Optional[GQADecodeConfig] = None,
    reduction: str = "fused",
) -> torch.Tensor:
    """Drop-in for gqa_decode/gqa_decode.py:1900-2010: E4M3 K/V ``[Hkv, S, D]`` with one
    float32 scale per KV head; K/V are dequantised in registers, with the rounding of
    ``fp8_utils.dequantize_kv_fp8``."""
    if q.dim() != 2 or k_fp8.dim() != 3 or v_fp8.dim() != 3:
        raise ValueError(
            "Expected q=(num_q_heads, head_dim), k/v=(num_kv_heads, seq_len, head_dim)"
        )
    if q.device.type != "cuda":
        raise ValueError("All tensors must be CUDA tensors")
    if q.dtype not in (torch.float16, torch.bfloat16):
        raise ValueError("Q must be fp16 or bf16")
    if k_fp8.dtype != torch.float8_e4m3fn or v_fp8.dtype != torch.float8_e4m3fn:
        raise ValueError("K/V must be float8_e4m3fn")
    if k_fp8.shape != v_fp8.shape:
        raise ValueError("k and v must have the same shape")
    if not (q.is_contiguous() and k_fp8.is_contiguous() and v_fp8.is_contiguous()):
        raise ValueError("Q/K/V must be contiguous")
    num_q_heads, head_dim = q.shape
    num_kv_heads, _, kv_head_dim = k_fp8.shape
    if kv_head_dim != head_dim:
        raise ValueError("Q/K/V head_dim mismatch")
    if num_q_heads % num_kv_heads != 0:
        raise ValueError("num_q_heads must be divisible by num_kv_heads")
    if k_scale.shape != (num_kv_heads,) or v_scale.shape != (num_kv_heads,):
        raise ValueError("Scales must be [num_kv_heads]")
    if reduction not in {"fused", "python"}:
        raise ValueError("reduction must be one of {'fused', 'python'}")
    ks = k_scale.to(device=q.device, dtype=torch.float32)
    vs = v_scale.to(device=q.device, dtype=torch.float32)
    if reduction == "python":
        cfg = config or GQADecodeConfig()
        splits = num_splits if num_splits is not None else select_num_splits(
            num_kv_heads, k_fp8.shape[1], cfg.block_seq, cfg.target_blocks_per_sm)
        acc, mx, one = _partials_for_python_reduction(q, k_fp8, v_fp8, ks, vs, splits)
        return reduce_partials(acc, mx, one, num_q_heads, splits, head_dim)
    out = gqa_decode_attention_batched(
        q.unsqueeze(0), k_fp8.unsqueeze(0), v_fp8.unsqueeze(0), None,
        k_scale=ks.view(1, -1), v_scale=vs.view(1, -1), num_splits=num_splits)
    return out.squeeze(0)


def merge_partials(
    o_parts: torch.Tensor,
    lse_parts: torch.Tensor,
    out_dtype: torch.dtype = torch.bfloat16,
    return_lse: bool = False,
):
    """LSE-weighted merge of normalised partials on the GPU (``gqa_merge_partials``).
    o_parts ``[P, R, D]`` float32, lse_parts ``[P, R]`` float32 (natural log; -inf = empty).
    Used for partials gathered from sequence shards on other GPUs."""
    if o_parts.dim() != 3 or lse_parts.shape != o_parts.shape[:2]:
        raise ValueError("Expected o_parts=(parts, rows, head_dim), lse_parts=(parts, rows)")
    if o_parts.dtype != torch.float32 or lse_parts.dtype != torch.float32:
        raise ValueError("partials must be float32")
    if o_parts.device.type != "cuda":
        raise ValueError("All tensors must be CUDA tensors")
    o_parts, lse_parts = o_parts.contiguous(), lse_parts.contiguous()
    parts, rows, d = o_parts.shape
    f32 = out_dtype == torch.float32
    out = torch.empty(rows, d, dtype=out_dtype, device=o_parts.device)
    lse = torch.empty(rows, dtype=torch.float32, device=o_parts.device) if return_lse else None
    with torch.cuda.device(o_parts.device):
        _native.check(
            _native.load().gqa_merge_partials(
                o_parts.data_ptr(), lse_parts.data_ptr(), parts, rows, d,
                None if f32 else out.data_ptr(), _DTYPE_CODE.get(out_dtype, 0),
                out.data_ptr() if f32 else None, lse.data_ptr() if lse is not None else None,
                torch.cuda.current_stream(o_parts.device).cuda_stream),
            "gqa_merge_partials")
    return (out, lse) if return_lse else out
