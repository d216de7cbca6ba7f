"""Generate the golden fixtures in this directory from the reference implementation.

Run where the reference checkout is importable (it is NOT needed to run the tests):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/gqa-decode

The script imports the reference's own `reference_gqa_decode`, `reduce_partials`,
`select_num_splits`, `quantize_kv_fp8` and `dequantize_kv_fp8`, feeds them seeded CPU
tensors and stores inputs (small cases) or seeds (large cases) together with the
reference's outputs.  bf16/fp16/fp8 tensors are stored as their raw integer bits.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def randn(shape, gen, dtype):
    return torch.randn(shape, generator=gen, dtype=torch.float32).to(dtype)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    import gqa_decode as ref  # the reference package
    from gqa_decode import fp8_utils as ref_fp8

    # ---- attention, inputs stored -------------------------------------------------
    small = [
        ("a", 32, 8, 128, 65, torch.bfloat16),
        ("b", 28, 4, 128, 130, torch.bfloat16),
        ("c", 16, 4, 64, 257, torch.bfloat16),
        ("d", 8, 1, 128, 1, torch.bfloat16),
        ("e", 32, 32, 128, 17, torch.bfloat16),
        ("f", 64, 8, 128, 40, torch.float16),
    ]
    out = {}
    for i, (tag, hq, hkv, d, s, dt) in enumerate(small):
        g = torch.Generator().manual_seed(1000 + i)
        q, k, v = randn((hq, d), g, dt), randn((hkv, s, d), g, dt), randn((hkv, s, d), g, dt)
        o = ref.reference_gqa_decode(q, k, v, num_kv_heads=hkv)
        out[f"{tag}_q"], out[f"{tag}_k"], out[f"{tag}_v"], out[f"{tag}_out"] = (
            bits(q), bits(k), bits(v), bits(o))
        out[f"{tag}_fp16"] = np.array(dt == torch.float16)
    np.savez_compressed(os.path.join(HERE, "attention_small.npz"), **out)

    # ---- attention, seeds stored (inputs = randn from torch.Generator(seed), q then k then v)
    seeded = [(7, 32, 8, 128, 16384), (8, 64, 8, 128, 4096), (9, 32, 8, 128, 4209)]
    out = {"cases": np.array(seeded, dtype=np.int64)}
    for seed, hq, hkv, d, s in seeded:
        g = torch.Generator().manual_seed(seed)
        q = randn((hq, d), g, torch.bfloat16)
        k = randn((hkv, s, d), g, torch.bfloat16)
        v = randn((hkv, s, d), g, torch.bfloat16)
        out[f"out_{seed}"] = bits(ref.reference_gqa_decode(q, k, v))
        out[f"probe_{seed}"] = bits(k[0, :2])  # detects a change in the RNG stream
    np.savez_compressed(os.path.join(HERE, "attention_seeded.npz"), **out)

    # ---- FP8: quantise / dequantise / attention on outlier data ---------------------
    g = torch.Generator().manual_seed(4242)
    hq, hkv, d, s = 32, 8, 128, 96
    q = randn((hq, d), g, torch.bfloat16)

    def outlier(shape):
        x = torch.randn(shape, generator=g, dtype=torch.float32)
        hit = torch.rand(shape, generator=g) < 1e-2
        return torch.where(hit, x * 20.0, x).to(torch.bfloat16)

    k, v = outlier((hkv, s, d)), outlier((hkv, s, d))
    k8, v8, ks, vs = ref_fp8.quantize_kv_fp8(k, v)
    kd, vd = ref_fp8.dequantize_kv_fp8(k8, v8, ks, vs)
    o = ref.reference_gqa_decode(q, kd, vd, num_kv_heads=hkv)
    np.savez_compressed(
        os.path.join(HERE, "fp8.npz"), q=bits(q), k=bits(k), v=bits(v), k8=bits(k8), v8=bits(v8),
        k_scale=ks.numpy(), v_scale=vs.numpy(), k_deq=bits(kd), v_deq=bits(vd), out=bits(o))

    # ---- reduce_partials in the reference's format ---------------------------------
    g = torch.Generator().manual_seed(77)
    hq, splits, d = 8, 5, 64
    acc = randn((hq * splits, d), g, torch.bfloat16)
    mx = torch.randn((hq * splits, 1), generator=g).expand(-1, d).contiguous()
    mx[3] = float("-inf")  # an empty split: max=-inf, sum=0, acc=0
    sm = (torch.rand((hq * splits, 1), generator=g) + 0.5).expand(-1, d).contiguous()
    sm[3] = 0.0
    acc[3] = 0.0
    red = ref.reduce_partials(acc, mx, sm, hq, splits, d)
    np.savez_compressed(
        os.path.join(HERE, "reduce_partials.npz"), acc=bits(acc), mx=mx.numpy(), sm=sm.numpy(),
        out=bits(red), dims=np.array([hq, splits, d]))

    # ---- select_num_splits table ----------------------------------------------------
    rows = []
    for hkv in (1, 4, 8, 32):
        for s in (1, 7, 64, 4208, 4209, 16384, 32768, 131072):
            for bs, tb in ((16, 16), (32, 16), (16, 4), (64, 8)):
                rows.append((hkv, s, bs, tb, 132, ref.select_num_splits(hkv, s, bs, tb)))
        rows.append((hkv, 8192, 16, 16, 148, ref.select_num_splits(hkv, 8192, 16, 16, 148)))
    np.savez_compressed(os.path.join(HERE, "select_num_splits.npz"),
                        table=np.array(rows, dtype=np.int64))
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <checkout of alityb/gqa-decode>")
    main(sys.argv[1])
