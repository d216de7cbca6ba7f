"""The five benchmark configurations at their full sizes, CUDA path (through the C ABI)
against the C restatement of the reference (oracle/gqa_oracle.c, float64 accumulation).

The reference pins its kernels to its PyTorch oracle at the shapes it benchmarks
(tests/test_correctness.py:19-31 of the reference, S up to 16384); these tests do the same
at the sizes the benchmark of this repository times.  Tolerance as everywhere:
|out - ref| <= 2e-2 + 1e-2 * |ref| per element, plus 5e-3 (about one bf16 output ulp)
against the float64 result for the 16-bit caches.

Inputs are generated on the GPU (gigabytes of N(0,1) take seconds there) and the sequences
that are checked are copied to the host for the oracle.
"""
import pytest
import torch

from oracle import c_oracle
from tests.golden_io import within_tolerance

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gqa_decode_b200 as g
    from gqa_decode_b200 import _native, build

    build.build()
    _native.load()
    return g


def _randn(shape, seed, dtype=torch.bfloat16):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return torch.randn(shape, generator=g, device=DEV, dtype=torch.float32).to(dtype)


def _check(out_rows, q_rows, k, v, tight=5e-3, k_scale=None, v_scale=None):
    """out_rows [Hq, D] from the GPU against the oracle on one sequence's q [Hq, D], k/v [Hkv, S, D]."""
    ref, _ = c_oracle.attend(q_rows.cpu(), k.cpu(), v.cpu(),
                             None if k_scale is None else k_scale.cpu(),
                             None if v_scale is None else v_scale.cpu())
    ok, ratio, mx = within_tolerance(out_rows.cpu(), ref)
    assert ok, f"worst |d|/tol = {ratio:.3f}, max abs {mx:.3e}"
    assert not torch.isnan(out_rows.float()).any()
    if tight is not None:
        assert mx <= tight * max(1.0, float(ref.abs().max())), mx
    return ratio


def test_config1_single_sequence(G):
    """B=1, Hq=32, Hkv=8, D=128, S=16384 bf16 through the drop-in entry."""
    q, k, v = _randn((32, 128), 1), _randn((8, 16384, 128), 2), _randn((8, 16384, 128), 3)
    out = G.gqa_decode_attention(q, k, v)
    assert G.read_status() == 0
    _check(out, q, k, v)
    out = G.gqa_decode_attention_persistent(q, k, v)
    _check(out, q, k, v)


def test_config2_ragged_batch_with_the_benchmark_lengths(G):
    """B=16 ragged, packed K/V, the very length list bench.py times (1, 7, 32768 + 13 drawn)."""
    import bench

    lens = bench.make_lengths(1234)
    assert lens[:3] == [1, 7, 32768] and len(lens) == 16
    hq, hkv, d = 32, 8, 128
    q = _randn((16, hq, d), 10)
    ks = [_randn((hkv, l, d), 100 + i) for i, l in enumerate(lens)]
    vs = [_randn((hkv, l, d), 200 + i) for i, l in enumerate(lens)]
    K = torch.cat([x.reshape(-1, d) for x in ks])
    V = torch.cat([x.reshape(-1, d) for x in vs])
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = G.gqa_decode_attention_batched(q, K, V, sl, layout="packed", max_seq_len=32768, num_kv_heads=hkv)
    assert G.read_status() == 0
    del K, V
    # every sequence is checked: the long ones cost the oracle a second each
    for i in range(16):
        _check(out[i], q[i], ks[i], vs[i])


def test_config3_fp8_batch_with_outliers(G):
    """B=8, S=32768, E4M3 K/V with 0.1 % outliers x20 and per-(sequence, head) scales, against
    the reference's dequantise-then-attend path."""
    from gqa_decode_b200 import fp8_utils

    b, hq, hkv, d, s = 8, 32, 8, 128, 32768
    q = _randn((b, hq, d), 20)

    def outlier(seed):
        g = torch.Generator(device=DEV).manual_seed(seed)
        x = torch.randn((b, hkv, s, d), generator=g, device=DEV)
        hit = torch.rand(x.shape, generator=g, device=DEV) < 1e-3
        return torch.where(hit, x * 20.0, x).to(torch.bfloat16)

    kk, vv = outlier(21), outlier(22)
    quant = [fp8_utils.quantize_kv_fp8(kk[i], vv[i]) for i in range(b)]
    del kk, vv
    k8, v8 = torch.stack([x[0] for x in quant]), torch.stack([x[1] for x in quant])
    ks, vs = torch.stack([x[2] for x in quant]), torch.stack([x[3] for x in quant])
    refs = [c_oracle.attend(q[i].cpu(), k8[i].cpu(), v8[i].cpu(), ks[i].cpu(), vs[i].cpu())[0] for i in range(b)]
    for exact_v in (False, True):
        out = G.gqa_decode_attention_batched(q, k8, v8, None, k_scale=ks, v_scale=vs, fp8_exact_v=exact_v)
        assert G.read_status() == 0
        assert not torch.isnan(out.float()).any()
        for i in range(b):
            ok, ratio, mx = within_tolerance(out[i].cpu(), refs[i])
            assert ok, f"sequence {i}, exact_v={exact_v}: worst |d|/tol = {ratio:.3f}, max abs {mx:.3e}"


def test_config4_long_sequence_all_heads(G):
    """B=1, Hq=64, Hkv=8, S=131072 bf16: every query head, the whole sequence; also as eight
    sequence shards merged by (O, LSE) on the device."""
    hq, hkv, d, s = 64, 8, 128, 131072
    q, k, v = _randn((hq, d), 30), _randn((hkv, s, d), 31), _randn((hkv, s, d), 32)
    out = G.gqa_decode_attention(q, k, v)
    assert G.read_status() == 0
    ref, lse_ref = c_oracle.attend(q.cpu(), k.cpu(), v.cpu())
    ok, ratio, mx = within_tolerance(out.cpu(), ref)
    assert ok and mx <= 5e-3, (ratio, mx)
    parts_o, parts_l = [], []
    for r in range(8):
        lo, hi = r * s // 8, (r + 1) * s // 8
        _, o32, lse = G.gqa_decode_attention_batched(
            q[None], k[None, :, lo:hi].contiguous(), v[None, :, lo:hi].contiguous(), None,
            return_f32=True, return_lse=True)
        parts_o.append(o32[0]), parts_l.append(lse[0])
    merged, lse = G.merge_partials(torch.stack(parts_o), torch.stack(parts_l), torch.bfloat16, return_lse=True)
    assert G.read_status() == 0
    ok, ratio, mx = within_tolerance(merged.cpu(), ref)
    assert ok and mx <= 5e-3, (ratio, mx)
    assert float((lse.cpu().double() - lse_ref).abs().max()) < 1e-3


@pytest.mark.parametrize("fp8", [False, True])
def test_config5_batch64_group8(G, fp8):
    """B=64, Hq=64, Hkv=8, S=8192: the 70B-shaped batch, bf16 and E4M3; a sample of six whole
    sequences (first, last and four in between), all 64 query heads each; then one KV head
    with its eight query heads on its own, as a rank of an 8-way head split runs it."""
    from gqa_decode_b200 import fp8_utils

    b, hq, hkv, d, s = 64, 64, 8, 128, 8192
    q = _randn((b, hq, d), 40)
    k, v = _randn((b, hkv, s, d), 41), _randn((b, hkv, s, d), 42)
    sample = [0, 13, 27, 38, 50, 63]
    if fp8:
        ks = torch.empty(b, hkv, device=DEV)
        vs = torch.empty(b, hkv, device=DEV)
        k8 = torch.empty(b, hkv, s, d, dtype=torch.float8_e4m3fn, device=DEV)
        v8 = torch.empty_like(k8)
        for i in range(b):
            k8[i], v8[i], ks[i], vs[i] = fp8_utils.quantize_kv_fp8(k[i], v[i])
        del k, v
        out = G.gqa_decode_attention_batched(q, k8, v8, None, k_scale=ks, v_scale=vs)
        assert G.read_status() == 0
        for i in sample:
            _check(out[i], q[i], k8[i], v8[i], tight=None, k_scale=ks[i], v_scale=vs[i])
        one = G.gqa_decode_attention_batched(
            q[:, 24:32].contiguous(), k8[:, 3:4].contiguous(), v8[:, 3:4].contiguous(), None,
            k_scale=ks[:, 3:4].contiguous(), v_scale=vs[:, 3:4].contiguous())
        for i in sample[:3]:
            _check(one[i], q[i, 24:32], k8[i, 3:4], v8[i, 3:4], tight=None,
                   k_scale=ks[i, 3:4], v_scale=vs[i, 3:4])
    else:
        out = G.gqa_decode_attention_batched(q, k, v, None)
        assert G.read_status() == 0
        for i in sample:
            _check(out[i], q[i], k[i], v[i])
        one = G.gqa_decode_attention_batched(
            q[:, 24:32].contiguous(), k[:, 3:4].contiguous(), v[:, 3:4].contiguous(), None)
        for i in sample[:3]:
            _check(one[i], q[i, 24:32], k[i, 3:4], v[i, 3:4])
    assert G.read_status() == 0
