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
