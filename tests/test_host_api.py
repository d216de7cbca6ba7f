"""Host-side mirror of the reference interface: same names, same ValueErrors, same
answers for the helper functions (checked against the golden fixtures)."""
import numpy as np
import pytest
import torch

import gqa_decode
import gqa_decode.fp8_utils
import gqa_decode.gqa_decode
import gqa_decode_b200 as G
from gqa_decode_b200 import fp8_utils
from tests.golden_io import bits_equal, from_bits, load


def test_public_names():
    for n in ["GQADecodeConfig", "gqa_decode_attention", "gqa_decode_attention_fp8",
              "gqa_decode_attention_persistent", "reduce_partials", "reference_gqa_decode",
              "select_num_splits"]:
        assert hasattr(gqa_decode, n) and hasattr(gqa_decode.gqa_decode, n)
    assert hasattr(gqa_decode.fp8_utils, "quantize_kv_fp8")
    assert hasattr(gqa_decode.fp8_utils, "dequantize_kv_fp8")
    cfg = G.GQADecodeConfig()
    assert (cfg.block_seq, cfg.smem_pad, cfg.target_blocks_per_sm) == (16, 8, 16)
    with pytest.raises(Exception):
        cfg.block_seq = 4  # frozen, like the reference's dataclass


def test_select_num_splits_table(native_lib):
    for hkv, s, bs, tb, sms, want in load("select_num_splits.npz")["table"]:
        assert G.select_num_splits(int(hkv), int(s), int(bs), int(tb), int(sms)) == int(want)
    with pytest.raises(ValueError, match="num_kv_heads must be positive"):
        G.select_num_splits(0, 10)


def test_reduce_partials_matches_reference():
    z = load("reduce_partials.npz")
    hq, splits, d = (int(x) for x in z["dims"])
    out = G.reduce_partials(from_bits(z["acc"], torch.bfloat16), torch.from_numpy(z["mx"]),
                            torch.from_numpy(z["sm"]), hq, splits, d)
    assert bits_equal(out, from_bits(z["out"], torch.bfloat16))


def test_fp8_utils_match_reference():
    z = load("fp8.npz")
    bf, f8 = torch.bfloat16, torch.float8_e4m3fn
    k8, v8, ks, vs = fp8_utils.quantize_kv_fp8(from_bits(z["k"], bf), from_bits(z["v"], bf))
    assert bits_equal(k8, from_bits(z["k8"], f8)) and bits_equal(v8, from_bits(z["v8"], f8))
    assert np.array_equal(ks.numpy(), z["k_scale"]) and np.array_equal(vs.numpy(), z["v_scale"])
    kd, vd = fp8_utils.dequantize_kv_fp8(k8, v8, ks, vs)
    assert bits_equal(kd, from_bits(z["k_deq"], bf)) and bits_equal(vd, from_bits(z["v_deq"], bf))


def test_torch_entry_matches_reference_output():
    z = load("attention_small.npz")
    q, k, v, ref = (from_bits(z[f"b_{n}"], torch.bfloat16) for n in ("q", "k", "v", "out"))
    assert bits_equal(G.reference_gqa_decode(q, k, v), ref)


def test_validation_errors_cpu():
    bf = torch.bfloat16
    q, k, v = torch.zeros(8, 64, dtype=bf), torch.zeros(2, 5, 64, dtype=bf), torch.zeros(2, 5, 64, dtype=bf)
    with pytest.raises(ValueError, match="Expected q="):
        G.gqa_decode_attention(q[0], k, v)
    with pytest.raises(ValueError, match="All tensors must be CUDA tensors"):
        G.gqa_decode_attention(q, k, v)  # CPU tensors are refused: there is no CPU path
    with pytest.raises(ValueError, match="All tensors must be CUDA tensors"):
        G.gqa_decode_attention_persistent(q, k, v)
    with pytest.raises(ValueError, match="All tensors must be CUDA tensors"):
        G.gqa_decode_attention_fp8(q, k, v, torch.ones(2), torch.ones(2))
    with pytest.raises(ValueError, match="identical shapes"):
        G.reference_gqa_decode(q, k, v[:, :4])
    with pytest.raises(ValueError, match="head_dim mismatch"):
        G.reference_gqa_decode(q[:, :32], k, v)
    with pytest.raises(ValueError, match="divisible"):
        G.reference_gqa_decode(q[:7], k, v)
    with pytest.raises(ValueError, match="num_kv_heads must match"):
        G.reference_gqa_decode(q, k, v, num_kv_heads=4)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from gqa_decode_b200 import _native

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "lib_path", lambda: str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no non-CUDA fallback"):
        _native.load()


def test_workspace_bookkeeping_is_by_identity():
    """The Python layer decides when a workspace's contents have to be cleared: a tensor it has
    not seen, a tensor last used with another geometry, never the same tensor with the same
    geometry; a tensor that was freed is forgotten (a new tensor at the same address is new)."""
    import gc

    import torch

    from gqa_decode_b200 import gqa_decode as g

    dev = torch.device("cuda", 0)  # only used as a dictionary key here
    a, b = torch.zeros(16, dtype=torch.uint8), torch.zeros(16, dtype=torch.uint8)
    geo1, geo2 = (1, 32, 8, 128, 0, 0, (False,) * 4, 16), (2, 32, 8, 128, 0, 0, (False,) * 4, 16)
    assert g._needs_clear(a, dev, geo1) is True      # unknown contents
    assert g._needs_clear(a, dev, geo1) is False     # same tensor, same geometry
    assert g._needs_clear(b, dev, geo1) is True      # another tensor
    assert g._needs_clear(a, dev, geo2) is True      # geometry changed
    assert g._needs_clear(a, dev, geo2) is False
    known = len(g._caller_workspaces)
    del a
    gc.collect()
    assert len(g._caller_workspaces) == known - 1


def test_epochs_wrap_without_zero_and_keep_alternating():
    from gqa_decode_b200.distributed import next_epoch

    e, seen = 0xFFFFFFFD, []
    for _ in range(6):
        e = next_epoch(e)
        seen.append(e)
    assert seen == [0xFFFFFFFE, 0xFFFFFFFF, 2, 3, 4, 5]
    assert all(x != 0 and x <= 0xFFFFFFFF for x in seen)
    assert all((x & 1) != (y & 1) for x, y in zip(seen, seen[1:]))  # the buffer halves keep alternating
    assert next_epoch(0) == 1


def test_optional_nvtx_ranges(monkeypatch):
    """With GQA_DECODE_B200_NVTX=1 the host-side phases are wrapped in NVTX ranges (pushed and
    popped in pairs, in order); without it trace_range() hands out one shared no-op object."""
    import torch

    from gqa_decode_b200 import _native, distributed

    assert _native.trace_range("a") is _native.trace_range("b")  # disabled: the shared no-op
    seen = []
    monkeypatch.setattr(_native, "TRACE_RANGES", True)
    monkeypatch.setattr(torch.cuda.nvtx, "range_push", lambda name: seen.append(("push", name)))
    monkeypatch.setattr(torch.cuda.nvtx, "range_pop", lambda: seen.append(("pop",)))

    def local_fn(q, k, v, lens, **kw):
        b, hq, d = q.shape
        return torch.zeros(b, hq, d), torch.zeros(b, hq)

    def merge_fn(o, lse, dtype):
        return o[0].to(dtype)

    q = torch.zeros(2, 4, 8, dtype=torch.bfloat16)
    out = distributed.sequence_sharded_decode(q, None, None, None, local_fn=local_fn, merge_fn=merge_fn)
    assert out.shape == (2, 4, 8)
    assert seen == [("push", "gqa_decode:local_partial"), ("pop",)]
    with _native.trace_range("x"):
        pass
    assert seen[-2:] == [("push", "x"), ("pop",)]
