"""FP8-E4M3 KV-cache helpers with the data contract of the reference's
``gqa_decode/fp8_utils.py``: one float32 scale per KV head, scale = amax / 448,
codes = clamp(x / amax * 448) as ``float8_e4m3fn``; dequantisation is
``float32(code) * scale`` rounded to bf16.  The decode kernels consume exactly this
format (``gqa_decode_attention_fp8``)."""
from __future__ import annotations

import torch

E4M3_MAX = 448.0


def _quantize_one(x: torch.Tensor):
    x32 = x.float()
    amax = x32.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1e-12)
    scale = (amax / E4M3_MAX).reshape(-1).float()
    code = (x32 / amax * E4M3_MAX).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return code, scale


def _quantize_one_cuda(x: torch.Tensor):
    """Two HBM-bound CUDA kernels (amax, convert) through the C ABI; same bits as the
    tensor-op formulation."""
    from . import _native

    lib = _native.load()
    x = x.contiguous()
    heads = x.shape[0]
    per = x.numel() // heads
    code = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    scale = torch.empty(heads, dtype=torch.float32, device=x.device)
    amax = torch.empty(heads, dtype=torch.float32, device=x.device)
    dt = _native.DTYPE_BF16 if x.dtype == torch.bfloat16 else _native.DTYPE_FP16
    with torch.cuda.device(x.device):
        _native.check(
            lib.gqa_quantize_kv_fp8(x.data_ptr(), dt, heads, per, code.data_ptr(), scale.data_ptr(),
                                    amax.data_ptr(), torch.cuda.current_stream(x.device).cuda_stream),
            "gqa_quantize_kv_fp8")
    return code.view(torch.float8_e4m3fn), scale


def quantize_kv_fp8(k_bf16: torch.Tensor, v_bf16: torch.Tensor):
    """Per-KV-head quantisation of ``[Hkv, S, D]`` caches (gqa_decode/fp8_utils.py:8-43).
    Returns ``(k_fp8, v_fp8, k_scale[Hkv], v_scale[Hkv])``; multiply by the scale to
    dequantise.  CUDA tensors (bf16/fp16, S*D a multiple of 8) go through the fused CUDA
    kernels; tensors on other devices are quantised with the same arithmetic as tensor ops
    (host-side preparation of test data - this is not part of the decode path)."""
    def one(x):
        if x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and (x.numel() // x.shape[0]) % 8 == 0:
            return _quantize_one_cuda(x)
        return _quantize_one(x)

    k8, ks = one(k_bf16)
    v8, vs = one(v_bf16)
    return k8, v8, ks, vs


def dequantize_kv_fp8(k_fp8, v_fp8, k_scale, v_scale):
    """Back to bf16 (gqa_decode/fp8_utils.py:46-56), for comparisons against a 16-bit path."""
    h = k_fp8.shape[0]
    k = (k_fp8.float() * k_scale.view(h, 1, 1)).to(torch.bfloat16)
    v = (v_fp8.float() * v_scale.view(h, 1, 1)).to(torch.bfloat16)
    return k, v


def append_kv_fp8(k_new, v_new, k_cache, v_cache, k_scale, v_scale, positions, *,
                  layout: str = "padded", block_table=None, saturated=None):
    """Quantise one new token per sequence into E4M3 caches in place (the reference has
    only the whole-cache :func:`quantize_kv_fp8`; a decode loop needs this between steps).

    k_new/v_new ``[B, Hkv, D]`` bf16/fp16; caches ``float8_e4m3fn`` in the padded layout
    ``[B, Hkv, Smax, D]`` or paged (``"paged_hnd"`` ``[pages, Hkv, page, D]``, ``"paged_nhd"``
    ``[pages, page, Hkv, D]`` with ``block_table`` int32 ``[B, max_pages]``); scales fp32
    ``[B, Hkv]`` as produced when the prompt was quantised; ``positions`` int32 ``[B]`` = the row
    each token is written to (the sequence length before the append).  Same arithmetic as
    ``quantize_kv_fp8`` with ``amax = scale * 448``; values outside a head's range saturate
    (``saturated``, an optional int32 device scalar, counts them).  CUDA only.
    """
    import ctypes

    from . import _native

    lib = _native.load()
    if not (k_new.is_cuda and k_cache.is_cuda):
        raise ValueError("All tensors must be CUDA tensors")
    if k_new.dtype not in (torch.bfloat16, torch.float16) or v_new.dtype != k_new.dtype:
        raise ValueError("Only fp16 and bf16 are supported")
    if k_cache.dtype != torch.float8_e4m3fn or v_cache.dtype != torch.float8_e4m3fn:
        raise ValueError("K/V must be float8_e4m3fn")
    if k_new.dim() != 3 or k_new.shape != v_new.shape or k_cache.shape != v_cache.shape:
        raise ValueError("Expected k_new/v_new=(batch, num_kv_heads, head_dim) and equal cache shapes")
    batch, hkv, d = k_new.shape
    a = _native.AppendArgs()
    if layout == "padded":
        if k_cache.dim() != 4 or tuple(k_cache.shape[:2]) != (batch, hkv) or k_cache.shape[3] != d:
            raise ValueError("padded layout expects caches=(batch, num_kv_heads, max_seq, head_dim)")
        a.kv_layout, a.max_seq_len = _native.LAYOUT_PADDED, k_cache.shape[2]
    elif layout in ("paged_hnd", "paged_nhd"):
        if k_cache.dim() != 4 or block_table is None or block_table.dtype != torch.int32:
            raise ValueError("paged layouts expect 4-D caches and an int32 block_table")
        hnd = layout == "paged_hnd"
        page = k_cache.shape[2] if hnd else k_cache.shape[1]
        if (k_cache.shape[1] if hnd else k_cache.shape[2]) != hkv or k_cache.shape[3] != d:
            raise ValueError("cache shape does not match k_new")
        block_table = block_table.contiguous()
        a.kv_layout = _native.LAYOUT_PAGED_HND if hnd else _native.LAYOUT_PAGED_NHD
        a.page_size, a.block_table_stride = page, block_table.shape[1]
        a.max_seq_len = block_table.shape[1] * page
        a.block_table = block_table.data_ptr()
    else:
        raise ValueError("layout must be 'padded', 'paged_hnd' or 'paged_nhd'")
    if positions.dtype != torch.int32 or positions.numel() != batch or not positions.is_cuda:
        raise ValueError("positions must be an int32 CUDA tensor of shape [batch]")
    if k_scale.numel() != batch * hkv or v_scale.numel() != batch * hkv or k_scale.dtype != torch.float32:
        raise ValueError("Scales must be float32 [batch, num_kv_heads]")
    if not (k_new.is_contiguous() and v_new.is_contiguous() and k_cache.is_contiguous()
            and v_cache.is_contiguous()):
        raise ValueError("Q/K/V must be contiguous")
    k_scale, v_scale, positions = k_scale.contiguous(), v_scale.contiguous(), positions.contiguous()
    a.k_new, a.v_new = k_new.data_ptr(), v_new.data_ptr()
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.k_scale, a.v_scale = k_scale.data_ptr(), v_scale.data_ptr()
    a.positions = positions.data_ptr()
    a.saturated = saturated.data_ptr() if saturated is not None else None
    a.batch, a.num_kv_heads, a.head_dim = batch, hkv, d
    a.src_dtype = _native.DTYPE_BF16 if k_new.dtype == torch.bfloat16 else _native.DTYPE_FP16
    a.stream = torch.cuda.current_stream(k_new.device).cuda_stream
    with torch.cuda.device(k_new.device):
        _native.check(lib.gqa_quantize_append_fp8(ctypes.byref(a)), "gqa_quantize_append_fp8")
