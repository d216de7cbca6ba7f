"""CPU restatement of the reference's decode-attention arithmetic.

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
benchmark's CPU-baseline leg.  The shipped package never imports this module.

Parity status: PINNED.  `tests/golden/make_golden.py` imports the reference
implementation itself (alityb/gqa-decode, `gqa_decode/gqa_decode.py` and
`gqa_decode/fp8_utils.py`) and stores its outputs on seeded inputs under
`tests/golden/*.npz`; `tests/test_oracle_golden.py` requires every function in
this file to reproduce those outputs bit for bit.

Each function names the reference lines it follows.  All arithmetic is float32
on CPU tensors, exactly as the reference's own PyTorch path does it.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

E4M3_MAX = 448.0  # torch.finfo(torch.float8_e4m3fn).max, gqa_decode/fp8_utils.py:23


def attend_one_sequence(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Exact single-token grouped-query attention for one sequence.

    Follows `reference_gqa_decode`, gqa_decode/gqa_decode.py:36-66:
      * query head h reads KV head h // (Hq // Hkv)            (:58-59)
      * K is widened to float32 and gathered per query head    (:61)
      * scores = q . k * head_dim**-0.5                        (:60, :62)
      * float32 softmax over the key axis                      (:63)
      * out = weights . V (float32), cast back to q's dtype    (:64-66)

    q: [Hq, D]; k, v: [Hkv, S, D]; returns [Hq, D] in q.dtype.
    """
    if q.dim() != 2 or k.dim() != 3 or v.dim() != 3:
        raise ValueError("q must be [Hq, D] and k/v [Hkv, S, D]")
    if k.shape != v.shape:
        raise ValueError("k and v shapes differ")
    n_q, d = q.shape
    n_kv, _, d_kv = k.shape
    if d_kv != d:
        raise ValueError("head_dim mismatch")
    if n_q % n_kv:
        raise ValueError("Hq must be a multiple of Hkv")
    owner = torch.arange(n_q, device=q.device) // (n_q // n_kv)
    k32 = k.float()[owner]
    logits = torch.einsum("hd,hsd->hs", q.float(), k32) * (d ** -0.5)
    probs = torch.softmax(logits, dim=-1)
    v32 = v.float()[owner]
    return torch.einsum("hs,hsd->hd", probs, v32).to(q.dtype)


def attend_batch(
    q: torch.Tensor, k_list: Sequence[torch.Tensor], v_list: Sequence[torch.Tensor]
) -> torch.Tensor:
    """Ragged batch = a Python loop of `attend_one_sequence` (the reference has no
    batch dimension, gqa_decode/gqa_decode.py:682-685, so a batch is B calls)."""
    return torch.stack(
        [attend_one_sequence(q[b], k_list[b], v_list[b]) for b in range(q.shape[0])]
    )


def attend_one_sequence_f64(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Same attention in float64 without the final cast: the yardstick used to
    report how far the float32 oracle and the CUDA path each sit from the
    exact answer.  Not a reference function."""
    n_q, d = q.shape
    n_kv = k.shape[0]
    g = n_q // n_kv
    qg = q.double().view(n_kv, g, d)
    logits = torch.matmul(qg, k.double().transpose(1, 2)) / math.sqrt(d)
    probs = torch.softmax(logits, dim=-1)
    return torch.matmul(probs, v.double()).view(n_q, d)


def lse_one_sequence(q: torch.Tensor, k: torch.Tensor) -> torch.Tensor:
    """Natural-log sum-exp of the scaled scores per query head, float64.
    Checks the (O, LSE) partials that sequence shards exchange."""
    n_q, d = q.shape
    n_kv = k.shape[0]
    g = n_q // n_kv
    qg = q.double().view(n_kv, g, d)
    logits = torch.matmul(qg, k.double().transpose(1, 2)) / math.sqrt(d)
    return torch.logsumexp(logits, dim=-1).view(n_q)


def quantize_kv_e4m3(k: torch.Tensor, v: torch.Tensor):
    """Per-KV-head E4M3 quantisation, gqa_decode/fp8_utils.py:8-43.

    amax over (S, D) per head, floored at 1e-12 (:26-27); scale = amax / 448
    (:29-30); code = clamp(x / amax * 448, +-448) cast to float8_e4m3fn (:32-41).
    Returns (k_fp8, v_fp8, k_scale[Hkv], v_scale[Hkv]).
    """
    def one(x):
        x32 = x.float()
        amax = x32.abs().amax(dim=(1, 2), keepdim=True).clamp(min=1e-12)
        scale = (amax / E4M3_MAX).reshape(-1).float()
        code = (x32 / amax * E4M3_MAX).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
        return code, scale

    k8, ks = one(k)
    v8, vs = one(v)
    return k8, v8, ks, vs


def dequantize_kv_e4m3(k8, v8, k_scale, v_scale):
    """gqa_decode/fp8_utils.py:46-56: float32(code) * scale[head], rounded to bf16."""
    h = k8.shape[0]
    kd = (k8.float() * k_scale.view(h, 1, 1)).to(torch.bfloat16)
    vd = (v8.float() * v_scale.view(h, 1, 1)).to(torch.bfloat16)
    return kd, vd


def append_codes_e4m3(x_new: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """E4M3 codes of new rows under an existing per-head scale: the arithmetic of
    gqa_decode/fp8_utils.py:32-41 with amax = scale * 448 (fp32).  The reference has no
    append step; this restates what a cache that keeps its prompt-time scales must do.
    x_new [..., D] with one scale per leading index (scale.shape == x_new.shape[:-1])."""
    amax = (scale.float() * 448.0).clamp(min=1e-12).unsqueeze(-1)
    return (x_new.float() / amax * 448.0).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)


def attend_one_sequence_e4m3(q, k8, v8, k_scale, v_scale):
    """The FP8 oracle the reference's tests use (tests/test_fp8.py:37-41):
    dequantise to bf16, then run the exact attention."""
    kd, vd = dequantize_kv_e4m3(k8, v8, k_scale, v_scale)
    return attend_one_sequence(q, kd, vd)


def merge_reference_partials(partial_out, partial_max, partial_sum, n_q, n_splits, d):
    """Split-K merge in the reference's own partial format,
    gqa_decode/gqa_decode.py:647-669: column 0 of max/sum holds the scalar
    (:657-659); M = max_i m_i (:661); w_i = exp(m_i - M) (:662);
    out = sum_i w_i acc_i / sum_i w_i l_i (:663-669), in partial_out's dtype."""
    m = partial_max[:, 0].view(n_q, n_splits)
    l = partial_sum[:, 0].view(n_q, n_splits)
    top = m.max(dim=1, keepdim=True).values
    w = torch.exp(m - top)
    denom = (l * w).sum(dim=1, keepdim=True)
    acc = partial_out.view(n_q, n_splits, d).float()
    num = torch.einsum("qsd,qs->qd", acc, w)
    return (num / denom).to(partial_out.dtype)


def merge_lse_partials(o_parts: torch.Tensor, lse_parts: torch.Tensor) -> torch.Tensor:
    """Merge normalised partials: o_parts [P, R, D] float32, lse_parts [P, R]
    (natural log; -inf marks an empty partial).  The same algebra as
    gqa_decode/gqa_decode.py:661-669 with acc_i = l_i * o_i and
    lse_i = m_i + log l_i.  Returns float64 [R, D]."""
    lse = lse_parts.double()
    top = lse.max(dim=0, keepdim=True).values
    top = torch.where(torch.isinf(top), torch.zeros_like(top), top)
    w = torch.exp(lse - top)
    num = (o_parts.double() * w.unsqueeze(-1)).sum(dim=0)
    return num / w.sum(dim=0).unsqueeze(-1)


def split_count(num_kv_heads, seq_len, block_seq=16, target_blocks_per_sm=16, num_sms=132):
    """One-wave split heuristic, gqa_decode/gqa_decode.py:69-102 (H100 constants
    132 SMs / 228 KB; two padded tiles of head_dim 128 at pad 8, 16-byte rounded)."""
    if num_kv_heads <= 0:
        raise ValueError("num_kv_heads must be positive")
    tile = (((block_seq - 1) * (128 + 8) + 128) * 2 + 15) & ~15
    per_block = 2 * tile
    cap = max(1, (228 * 1024) // per_block - 1)
    grid = num_sms * min(target_blocks_per_sm, cap)
    return min(max(1, grid // num_kv_heads), max(1, math.ceil(seq_len / block_seq)))


# ----------------------------------------------------------------------------
# Seeded synthetic inputs with the shapes and value distributions of the five
# benchmark configurations.  Generated on CPU so the oracle and the GPU path
# see the same bits.
# ----------------------------------------------------------------------------

def randn_bf16(shape, gen, dtype=torch.bfloat16):
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)


def ragged_lengths(batch: int, max_len: int, seed: int, fixed=(1, 7, None)) -> list[int]:
    """Lengths for the ragged batch: `fixed` first (None = max_len), the rest
    uniform in [1, max_len] from `seed`."""
    gen = torch.Generator().manual_seed(seed)
    fixed = [max_len if f is None else f for f in fixed][:batch]
    rest = torch.randint(1, max_len + 1, (batch - len(fixed),), generator=gen).tolist()
    return fixed + rest


def outlier_kv(shape, gen, rate=1e-3, gain=20.0):
    """N(0,1) with a Bernoulli(rate) subset multiplied by `gain`, as bf16."""
    x = torch.randn(shape, generator=gen, dtype=torch.float32)
    hit = torch.rand(shape, generator=gen) < rate
    return torch.where(hit, x * gain, x).to(torch.bfloat16)
