"""Paged K/V caches (block tables): parity with the CPU oracle and bit equality with the
contiguous layouts.

The reference holds K and V as contiguous [Hkv, S, D] tensors only
(gqa_decode/gqa_decode.py:44); serving engines hand over pages and a block table.  The
schedule does not depend on where rows live, so a paged launch must return exactly the
bits of the padded launch on the same keys.
"""
import pytest
import torch

from oracle import gqa_oracle as O
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


def _pages(ks, vs, page_size, layout, seed, poison, smax=0):
    """Scatter per-sequence [Hkv, len, D] tensors into a shuffled page pool.
    Unused rows of a sequence's last page and unused pages hold `poison`; table entries
    past the last page of a sequence hold an out-of-range page number."""
    hkv, _, d = ks[0].shape
    need = [(k.shape[1] + page_size - 1) // page_size for k in ks]
    num_pages = sum(need) + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g).tolist()
    shape = (num_pages, hkv, page_size, d)
    kp = torch.full(shape, poison, dtype=torch.float32).to(ks[0].dtype)
    vp = kp.clone()
    cols = max(max(need) + 2, (smax + page_size - 1) // page_size)
    table = torch.full((len(ks), cols), 2 ** 30, dtype=torch.int32)
    nxt = 0
    for b, (k, v) in enumerate(zip(ks, vs)):
        for p in range(need[b]):
            page = perm[nxt]
            nxt += 1
            table[b, p] = page
            rows = min(page_size, k.shape[1] - p * page_size)
            kp[page, :, :rows] = k[:, p * page_size:p * page_size + rows]
            vp[page, :, :rows] = v[:, p * page_size:p * page_size + rows]
    if layout == "paged_nhd":
        kp, vp = kp.transpose(1, 2).contiguous(), vp.transpose(1, 2).contiguous()
    return kp, vp, table


def _case(lens, hq, hkv, d, seed):
    g = torch.Generator().manual_seed(seed)
    q = O.randn_bf16((len(lens), hq, d), g)
    ks = [O.randn_bf16((hkv, l, d), g) for l in lens]
    vs = [O.randn_bf16((hkv, l, d), g) for l in lens]
    return q, ks, vs


def _padded(ks, vs, smax):
    hkv, _, d = ks[0].shape
    K = torch.zeros(len(ks), hkv, smax, d, dtype=ks[0].dtype)
    V = torch.zeros_like(K)
    for b, (k, v) in enumerate(zip(ks, vs)):
        K[b, :, :k.shape[1]], V[b, :, :k.shape[1]] = k, v
    return K, V


@pytest.mark.parametrize("layout", ["paged_hnd", "paged_nhd"])
@pytest.mark.parametrize("page_size", [16, 32, 64, 128, 256])
def test_paged_equals_padded_and_oracle(G, layout, page_size):
    lens = [1, 7, 5000, 0, 2500, 64, 65, 16, 17, 4096]
    q, ks, vs = _case(lens, 32, 8, 128, seed=21)
    smax = 5120
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    K, V = _padded(ks, vs, smax)
    want = G.gqa_decode_attention_batched(q.to(DEV), K.to(DEV), V.to(DEV), sl)
    kp, vp, table = _pages(ks, vs, page_size, layout, seed=page_size, poison=float("nan"), smax=smax)
    got, lse = G.gqa_decode_attention_batched(
        q.to(DEV), kp.to(DEV), vp.to(DEV), sl, layout=layout, block_table=table.to(DEV),
        max_seq_len=smax, return_lse=True)
    assert G.read_status() == 0
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    ref = torch.stack([
        O.attend_one_sequence(q[b], ks[b], vs[b]) if l else torch.zeros(32, 128, dtype=torch.bfloat16)
        for b, l in enumerate(lens)])
    ok, ratio, mx = within_tolerance(got.cpu(), ref)
    assert ok, f"worst |d|/tol = {ratio:.3f}, max abs {mx:.3e}"
    assert torch.isinf(lse[3]).all() and (got[3] == 0).all()


@pytest.mark.parametrize("hq,hkv,d,dtype", [(16, 4, 64, torch.bfloat16), (16, 2, 256, torch.float16),
                                            (32, 2, 128, torch.float16)])
@pytest.mark.parametrize("page_size", [16, 128, 512])
def test_paged_other_shapes(G, hq, hkv, d, dtype, page_size):
    """Head dims 64 / 256, fp16, G = 8 and 16, pages smaller and larger than the tile."""
    lens = [3000, 129, 1, 1024]
    q, ks, vs = _case(lens, hq, hkv, d, seed=5)
    q, ks, vs = q.to(dtype), [k.to(dtype) for k in ks], [v.to(dtype) for v in vs]
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    K, V = _padded(ks, vs, 3072)
    want = G.gqa_decode_attention_batched(q.to(DEV), K.to(DEV), V.to(DEV), sl)
    for layout in ("paged_hnd", "paged_nhd"):
        kp, vp, table = _pages(ks, vs, page_size, layout, seed=3, poison=float("nan"), smax=3072)
        got = G.gqa_decode_attention_batched(
            q.to(DEV), kp.to(DEV), vp.to(DEV), sl, layout=layout, block_table=table.to(DEV),
            max_seq_len=3072)
        assert G.read_status() == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    ref = torch.stack([O.attend_one_sequence(q[b], ks[b], vs[b]) for b in range(len(lens))])
    ok, ratio, mx = within_tolerance(want.cpu(), ref)
    assert ok, f"worst |d|/tol = {ratio:.3f}, max abs {mx:.3e}"


@pytest.mark.parametrize("splits", [1, 3, 7])
def test_paged_explicit_splits(G, splits):
    lens = [2000, 130, 64]
    q, ks, vs = _case(lens, 32, 8, 128, seed=8)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    K, V = _padded(ks, vs, 2048)
    want = G.gqa_decode_attention_batched(q.to(DEV), K.to(DEV), V.to(DEV), sl, num_splits=splits)
    kp, vp, table = _pages(ks, vs, 32, "paged_hnd", seed=1, poison=float("nan"), smax=2048)
    got = G.gqa_decode_attention_batched(
        q.to(DEV), kp.to(DEV), vp.to(DEV), sl, layout="paged_hnd", block_table=table.to(DEV),
        max_seq_len=2048, num_splits=splits)
    assert G.read_status() == 0
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))


@pytest.mark.parametrize("layout", ["paged_hnd", "paged_nhd"])
@pytest.mark.parametrize("page_size", [16, 64, 256, 512])
def test_paged_fp8(G, layout, page_size):
    """E4M3 pages: same bits as the padded FP8 launch, and inside the tolerance of
    quantise -> dequantise -> oracle on data with outliers."""
    from gqa_decode_b200 import fp8_utils

    lens = [3000, 1, 255, 257, 1024]
    hq, hkv, d = 32, 8, 128
    g = torch.Generator().manual_seed(17)
    q = O.randn_bf16((len(lens), hq, d), g)
    ks = [O.outlier_kv((hkv, l, d), g) for l in lens]
    vs = [O.outlier_kv((hkv, l, d), g) for l in lens]
    quant = [fp8_utils.quantize_kv_fp8(k, v) for k, v in zip(ks, vs)]
    kq, vq = [x[0] for x in quant], [x[1] for x in quant]
    ksc = torch.stack([x[2] for x in quant])
    vsc = torch.stack([x[3] for x in quant])
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    K = torch.zeros(len(lens), hkv, 3072, d, dtype=torch.uint8)
    V = torch.zeros_like(K)
    for b, l in enumerate(lens):
        K[b, :, :l], V[b, :, :l] = kq[b].view(torch.uint8), vq[b].view(torch.uint8)
    K, V = K.view(torch.float8_e4m3fn), V.view(torch.float8_e4m3fn)
    want = G.gqa_decode_attention_batched(
        q.to(DEV), K.to(DEV), V.to(DEV), sl, k_scale=ksc.to(DEV), v_scale=vsc.to(DEV))
    # 0x7f is an E4M3 NaN: unused rows must never reach the result
    kp, vp, table = _pages([x.view(torch.uint8) for x in kq], [x.view(torch.uint8) for x in vq],
                           page_size, layout, seed=2, poison=127.0, smax=3072)
    got = G.gqa_decode_attention_batched(
        q.to(DEV), kp.view(torch.float8_e4m3fn).to(DEV), vp.view(torch.float8_e4m3fn).to(DEV), sl,
        layout=layout, block_table=table.to(DEV), max_seq_len=3072,
        k_scale=ksc.to(DEV), v_scale=vsc.to(DEV))
    assert G.read_status() == 0
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    ref = torch.stack([
        O.attend_one_sequence_e4m3(q[b], kq[b], vq[b], ksc[b], vsc[b]) for b in range(len(lens))])
    ok, ratio, mx = within_tolerance(got.cpu(), ref)
    assert ok, f"worst |d|/tol = {ratio:.3f}, max abs {mx:.3e}"


def test_paged_plan_graph_replay_follows_table_updates(G):
    """A captured plan re-reads the block table and the lengths on every replay: append a
    page to one sequence, replay, and compare with a fresh padded launch."""
    lens = [100, 900]
    q, ks, vs = _case([164, 900], 32, 8, 128, seed=30)
    page = 64
    kp, vp, table = _pages(ks, vs, page, "paged_hnd", seed=4, poison=0.0, smax=1024)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    qd, kpd, vpd, td = q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV)
    plan = G.plan_decode(qd, kpd, vpd, sl, layout="paged_hnd", block_table=td, max_seq_len=1024)
    plan.run()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        plan.run()
    for l0 in (100, 128, 129, 164):
        sl.copy_(torch.tensor([l0, 900], dtype=torch.int32))
        graph.replay()
        torch.cuda.synchronize()
        K, V = _padded([ks[0][:, :l0], ks[1]], [vs[0][:, :l0], vs[1]], 1024)
        want = G.gqa_decode_attention_batched(qd, K.to(DEV), V.to(DEV), sl)
        assert torch.equal(plan.result.view(torch.int16), want.view(torch.int16))
    assert G.read_status() == 0


def test_paged_argument_errors(G):
    q, ks, vs = _case([64], 32, 8, 128, seed=1)
    sl = torch.tensor([64], dtype=torch.int32, device=DEV)
    kp, vp, table = _pages(ks, vs, 64, "paged_hnd", seed=1, poison=0.0)
    qd, kpd, vpd, td = q.to(DEV), kp.to(DEV), vp.to(DEV), table.to(DEV)
    with pytest.raises(ValueError):
        G.gqa_decode_attention_batched(qd, kpd, vpd, sl, layout="paged_hnd")  # no table
    with pytest.raises(ValueError):
        G.gqa_decode_attention_batched(qd, kpd, vpd, None, layout="paged_hnd", block_table=td)
    with pytest.raises(ValueError):
        G.gqa_decode_attention_batched(qd, kpd, vpd, sl, layout="paged_hnd", block_table=td.long())
    with pytest.raises(ValueError):  # 24 rows per page: neither divides nor is a multiple of 64
        bad = torch.zeros(4, 8, 24, 128, dtype=torch.bfloat16, device=DEV)
        G.gqa_decode_attention_batched(qd, bad, bad, sl, layout="paged_hnd", block_table=td)
    with pytest.raises(ValueError):
        G.gqa_decode_attention_batched(qd, kpd, vpd, sl, layout="paged_hnd", block_table=td,
                                       max_seq_len=10 ** 6)


@pytest.mark.parametrize("layout", ["padded", "paged_hnd", "paged_nhd"])
def test_append_token_fp8(G, layout):
    """Decode loop on an E4M3 cache: quantise the prompt, then append tokens one step at a time
    with the prompt's scales.  Codes must equal the CPU restatement bit for bit, the rest of
    the cache must stay untouched, and decoding over the grown cache must stay inside the
    tolerance of dequantise -> oracle."""
    from gqa_decode_b200 import fp8_utils

    hq, hkv, d, page, smax = 32, 8, 128, 16, 512
    lens = [100, 255, 31, 1]
    steps = 3
    g = torch.Generator().manual_seed(3)
    q = O.randn_bf16((len(lens), hq, d), g)
    full_k = [O.randn_bf16((hkv, l + steps, d), g) for l in lens]
    full_v = [O.randn_bf16((hkv, l + steps, d), g) for l in lens]
    # one appended value far outside the prompt's range: must saturate and be counted
    full_k[0][2, lens[0] + 1, 5] = 1000.0
    quant = [fp8_utils.quantize_kv_fp8(k[:, :l].contiguous(), v[:, :l].contiguous())
             for k, v, l in zip(full_k, full_v, lens)]
    ksc = torch.stack([x[2] for x in quant])
    vsc = torch.stack([x[3] for x in quant])
    # reference codes of every row under the prompt scales (rows < len are the prompt itself)
    want_k = [torch.cat([quant[b][0], O.append_codes_e4m3(
        full_k[b][:, lens[b]:], ksc[b][:, None].expand(-1, steps))], 1) for b in range(len(lens))]
    want_v = [torch.cat([quant[b][1], O.append_codes_e4m3(
        full_v[b][:, lens[b]:], vsc[b][:, None].expand(-1, steps))], 1) for b in range(len(lens))]
    u8 = lambda t: t.view(torch.uint8)
    if layout == "padded":
        K = torch.full((len(lens), hkv, smax, d), 0x55, dtype=torch.uint8)
        V = K.clone()
        for b, l in enumerate(lens):
            K[b, :, :l], V[b, :, :l] = u8(quant[b][0]), u8(quant[b][1])
        table = None
    else:
        # pages for the final lengths; rows past the prompt hold a marker byte
        grown_k = [torch.cat([u8(quant[b][0]), torch.full((hkv, steps, d), 0x55, dtype=torch.uint8)], 1)
                   for b in range(len(lens))]
        grown_v = [torch.cat([u8(quant[b][1]), torch.full((hkv, steps, d), 0x55, dtype=torch.uint8)], 1)
                   for b in range(len(lens))]
        K, V, table = _pages(grown_k, grown_v, page, layout, seed=6, poison=float(0x55), smax=smax)
    Kd, Vd = K.to(DEV).view(torch.float8_e4m3fn), V.to(DEV).view(torch.float8_e4m3fn)
    td = table.to(DEV) if table is not None else None
    sat = torch.zeros(1, dtype=torch.int32, device=DEV)
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    kw = dict(layout=layout, block_table=td) if td is not None else {}
    dkw = dict(kw, max_seq_len=smax) if td is not None else {}
    for step in range(steps):
        kn = torch.stack([full_k[b][:, lens[b] + step] for b in range(len(lens))]).to(DEV)
        vn = torch.stack([full_v[b][:, lens[b] + step] for b in range(len(lens))]).to(DEV)
        fp8_utils.append_kv_fp8(kn, vn, Kd, Vd, ksc.to(DEV), vsc.to(DEV), sl, saturated=sat, **kw)
        sl += 1
        out = G.gqa_decode_attention_batched(q.to(DEV), Kd, Vd, sl, k_scale=ksc.to(DEV),
                                             v_scale=vsc.to(DEV), **dkw)
        assert G.read_status() == 0
        n = [l + step + 1 for l in lens]
        ref = torch.stack([O.attend_one_sequence_e4m3(
            q[b], want_k[b][:, :n[b]], want_v[b][:, :n[b]], ksc[b], vsc[b]) for b in range(len(lens))])
        ok, ratio, mx = within_tolerance(out.cpu(), ref)
        assert ok, f"step {step}: worst |d|/tol = {ratio:.3f}, max abs {mx:.3e}"
    # clamped elements: the planted outlier plus whatever exceeds a short prompt's range
    expect = 0
    for b, l in enumerate(lens):
        for x, sc in ((full_k[b], ksc[b]), (full_v[b], vsc[b])):
            f = x[:, l:].float() / (sc * 448.0).clamp(min=1e-12)[:, None, None] * 448.0
            expect += int((f.abs() > 448.0).sum())
    assert expect >= 1 and int(sat.item()) == expect
    # every written row equals the CPU restatement; everything else still holds the marker / prompt
    Kc, Vc = Kd.view(torch.uint8).cpu(), Vd.view(torch.uint8).cpu()
    for b, l in enumerate(lens):
        for r in range(l + steps + 1):
            if layout == "padded":
                gk, gv = Kc[b, :, r], Vc[b, :, r]
            else:
                pg, off = int(table[b, r // page]), r % page
                if r >= l + steps and (r // page) >= (l + steps + page - 1) // page:
                    break  # past the last allocated page
                gk = Kc[pg, :, off] if layout == "paged_hnd" else Kc[pg, off]
                gv = Vc[pg, :, off] if layout == "paged_hnd" else Vc[pg, off]
            if r < l + steps:
                assert torch.equal(gk, u8(want_k[b])[:, r]) and torch.equal(gv, u8(want_v[b])[:, r]), (b, r)
            else:
                assert (gk == 0x55).all() and (gv == 0x55).all(), (b, r)
