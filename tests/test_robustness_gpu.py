"""Failure detection and workspace hygiene on one GPU.

* A bounded device-side wait is made to run out - a peer's flag that nothing ever raises,
  with a limit of a few milliseconds - and the kernel must return with status bit 16, leave
  the outputs alone and leave the context usable; the next launch is correct.  No GPU is
  faulted, trapped or hung: the peer "GPU" is a second buffer in local memory.
* Workspaces: a captured plan replays correctly after launches of other geometries ran in
  between; one caller-owned workspace serves launches of different geometries in turn.
"""
import ctypes

import pytest
import torch

from oracle import gqa_oracle as O
from tests.golden_io import within_tolerance

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
WAIT_EXCHANGE = 16


@pytest.fixture(scope="module")
def G():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import gqa_decode_b200 as g
    from gqa_decode_b200 import _native, build

    build.build()
    _native.load()
    return g


def _merge_two(o_parts, lse_parts):
    return O.merge_lse_partials(o_parts.cpu(), lse_parts.cpu())


def test_exchange_wait_expires_and_recovers(G):
    """gqa_exchange_merge as rank 0 of a world of two whose rank 1 does not exist."""
    from gqa_decode_b200 import _native

    lib = _native.load()
    rows, d, world = 64, 128, 2
    nbytes = int(lib.gqa_exchange_buffer_bytes(world, rows, d))
    mine = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)    # rank 0's receive buffer
    theirs = torch.zeros(nbytes, dtype=torch.uint8, device=DEV)  # stands in for rank 1's
    ptrs = torch.tensor([mine.data_ptr(), theirs.data_ptr()], dtype=torch.int64, device=DEV)
    g = torch.Generator().manual_seed(3)
    o = torch.randn(world, rows, d, generator=g).to(DEV)
    lse = torch.randn(world, rows, generator=g).to(DEV)
    out = torch.full((rows, d), 7.0, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream

    def call(epoch, limit_ns):
        return lib.gqa_exchange_merge(
            o[0].data_ptr(), lse[0].data_ptr(), ptrs.data_ptr(), 0, world, epoch, rows, d,
            out.data_ptr(), _native.DTYPE_BF16, None, None, status.data_ptr(), limit_ns, stream)

    # epoch 1: nobody raises rank 1's flag -> the wait runs out after 3 ms
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    assert call(1, 3_000_000) == 0
    t1.record()
    torch.cuda.synchronize()
    assert int(status.item()) == WAIT_EXCHANGE
    assert 2.0 < t0.elapsed_time(t1) < 500.0  # it did wait, and it did give up
    assert bool((out == 7.0).all()), "outputs must stay untouched when a peer never arrived"
    # the kernel pushed rank 0's partial into "rank 1" and raised its flag there
    # (epoch 1 = parity half 1, source rank 0: slot index 1 * world + 0)
    hdr, slot = 256, rows * (d + 1)
    at = hdr + (1 * world + 0) * slot * 4
    got = theirs[at:at + rows * d * 4].view(torch.float32).view(rows, d)
    assert torch.equal(got, o[0])
    assert int(theirs[:16].view(torch.int32)[1 * world + 0].item()) == 1

    # epoch 2 (other parity half): play rank 1 by hand - its partial and its flag - and the
    # same call completes and merges both partials
    status.zero_()
    recv = mine[hdr:].view(torch.float32)
    base = (0 * world + 1) * slot  # parity 0 (epoch 2), source rank 1
    recv[base:base + rows * d] = o[1].reshape(-1)
    recv[base + rows * d:base + slot] = lse[1]
    mine[:8].view(torch.int32)[1] = 2  # flag[parity 0][rank 1] = epoch 2
    torch.cuda.synchronize()
    assert call(2, 3_000_000) == 0
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = _merge_two(o, lse)
    ok, ratio, mx = within_tolerance(out.cpu(), ref)
    assert ok and mx < 2e-2, (ratio, mx)


@pytest.mark.parametrize("mode", ["heads", "sequence"])
def test_gather_wait_expires_and_recovers(G, mode):
    """The decode kernel's own hand-off tail (head gather / sequence exchange) as rank 0 of a
    world of two without a rank 1: status bit 16 after the limit, and the workspace serves a
    correct ordinary launch afterwards."""
    from gqa_decode_b200 import _native

    lib = _native.load()
    b, hq, hkv, d, s = 2, 32, 8, 128, 3000
    gen = torch.Generator().manual_seed(17)
    q, k, v = O.randn_bf16((b, hq, d), gen), O.randn_bf16((b, hkv, s, d), gen), O.randn_bf16((b, hkv, s, d), gen)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    ws = torch.zeros(G.workspace_bytes(b, hq, hkv, d), dtype=torch.uint8, device=DEV)
    world, rows = 2, b * hq
    if mode == "heads":
        bufs = [torch.zeros(2 * b * world * hq * d, dtype=torch.bfloat16, device=DEV) for _ in range(world)]
    else:
        nbytes = int(lib.gqa_sequence_exchange_bytes(world, rows, d))
        bufs = [torch.zeros(nbytes // 4, dtype=torch.float32, device=DEV) for _ in range(world)]
    flags = [torch.zeros(2 * world, dtype=torch.int32, device=DEV) for _ in range(world)]
    arr = ctypes.c_void_p * world
    ga = _native.GatherArgs()
    po, pf = arr(*[t.data_ptr() for t in bufs]), arr(*[t.data_ptr() for t in flags])
    ga.peer_out = ctypes.cast(po, ctypes.POINTER(ctypes.c_void_p))
    ga.peer_flags = ctypes.cast(pf, ctypes.POINTER(ctypes.c_void_p))
    ga.world, ga.rank, ga.epoch = world, 0, 1
    ga.mode = _native.GATHER_HEADS if mode == "heads" else _native.GATHER_SEQUENCE
    out = torch.full((b, hq, d), 5.0, dtype=torch.bfloat16, device=DEV)
    a = _native.DecodeArgs()
    a.q, a.k, a.v, a.out = qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), out.data_ptr()
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = b, hq, hkv, d
    a.max_seq_len, a.total_rows = s, b * hkv * s
    a.q_dtype = a.kv_dtype = _native.DTYPE_BF16
    a.kv_layout = _native.LAYOUT_PADDED
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    a.wait_limit_ns = 3_000_000
    a.stream = torch.cuda.current_stream().cuda_stream
    assert lib.gqa_decode_attention_gather(ctypes.byref(a), ctypes.byref(ga)) == 0
    torch.cuda.synchronize()
    st = ctypes.c_int32(-1)
    assert lib.gqa_decode_read_status(ws.data_ptr(), None, ctypes.byref(st)) == 0
    assert st.value == WAIT_EXCHANGE
    if mode == "sequence":
        assert bool((out == 5.0).all()), "no merge may run when a peer's partial never arrived"
    if mode == "heads":
        # this rank's flag was raised on the stand-in peer: [parity 1][rank 0] = epoch 1
        assert int(flags[1][world * 1 + 0].item()) == 1
    else:
        # this rank's rows reached the stand-in peer, every word tagged with epoch 1
        slot = rows * d + ((rows + 1) & ~1)
        words = bufs[1].view(torch.int32).view(-1, 2)[(1 * world + 0) * slot:(1 * world + 0) * slot + rows * d + rows]
        assert bool((words[:, 1] == 1).all())
    # recovery: zero the workspace, then an ordinary launch on it is correct
    assert lib.gqa_decode_workspace_reset(ws.data_ptr(), ws.numel(), None) == 0
    got = G.gqa_decode_attention_batched(qd, kd, vd, None, workspace=ws)
    assert G.read_status(ws) == 0
    ref = O.attend_batch(q, [k[i] for i in range(b)], [v[i] for i in range(b)])
    ok, ratio, mx = within_tolerance(got.cpu(), ref)
    assert ok, (ratio, mx)


def _case(b, hq, hkv, s, seed):
    gen = torch.Generator().manual_seed(seed)
    q, k, v = O.randn_bf16((b, hq, 128), gen), O.randn_bf16((b, hkv, s, 128), gen), O.randn_bf16((b, hkv, s, 128), gen)
    ref = O.attend_batch(q, [k[i] for i in range(b)], [v[i] for i in range(b)])
    return q.to(DEV), k.to(DEV), v.to(DEV), ref


def test_captured_plan_survives_other_geometries(G):
    """Plan A is captured in a CUDA graph; launches of other geometries (eager, on the shared
    workspace, and a second plan) run in between; replaying A returns the same bits."""
    qa, ka, va, ref_a = _case(4, 32, 8, 6000, 1)   # many groups, many partials
    qb, kb, vb, ref_b = _case(1, 32, 8, 900, 2)    # small geometry: its partials lie where A's tickets would
    qc, kc, vc, ref_c = _case(2, 64, 8, 2500, 3)
    plan = G.plan_decode(qa, ka, va, None)
    first = plan.run().clone()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        plan.run()
    for _ in range(3):
        out_b = G.gqa_decode_attention_batched(qb, kb, vb, None)
        out_c = G.gqa_decode_attention_batched(qc, kc, vc, None)
        out_a = G.gqa_decode_attention_batched(qa, ka, va, None)   # A's geometry on the shared workspace too
        plan.result.fill_(0)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(plan.result, first)
        assert torch.equal(out_a, first)
        assert within_tolerance(out_b.cpu(), ref_b)[0] and within_tolerance(out_c.cpu(), ref_c)[0]
    assert plan.status() == 0 and G.read_status() == 0
    assert within_tolerance(first.cpu(), ref_a)[0]


def test_one_caller_workspace_many_geometries(G):
    """A caller-owned workspace passed to launches of different geometries in turn, explicit
    splits included, and a fresh (uninitialised) workspace tensor on every call."""
    cases = [_case(4, 32, 8, 6000, 11), _case(1, 32, 8, 900, 12), _case(2, 64, 8, 2500, 13)]
    need = max(G.workspace_bytes(q.shape[0], q.shape[1], k.shape[1], 128, 7) for q, k, _, _ in cases)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)
    for rnd in range(2):
        for splits in (None, 7):
            for q, k, v, ref in cases:
                out = G.gqa_decode_attention_batched(q, k, v, None, num_splits=splits, workspace=ws)
                assert G.read_status(ws) == 0
                assert within_tolerance(out.cpu(), ref)[0]
    for q, k, v, ref in cases:
        junk = torch.empty(need, dtype=torch.uint8, device=DEV)
        junk.fill_(0xAB)  # whatever the allocator hands back
        out = G.gqa_decode_attention_batched(q, k, v, None, workspace=junk)
        assert G.read_status(junk) == 0
        assert within_tolerance(out.cpu(), ref)[0]


@pytest.mark.parametrize("mode", ["balanced", "splits", "stealing", "ticket", "separate", "fp8"])
def test_workspace_guards_stay_intact(G, mode):
    """A workspace of exactly the advertised size between two guard areas: a launch may write
    nothing outside [workspace, workspace + workspace_bytes), leaves the guards' pattern alone
    and hands the workspace itself back all zero (what the next launch relies on)."""
    from gqa_decode_b200 import fp8_utils

    b, hq, hkv, d = 5, 32, 8, 128
    lens = [1, 4097, 0, 9000, 650]
    gen = torch.Generator().manual_seed(23)
    q = O.randn_bf16((b, hq, d), gen)
    ks = [O.randn_bf16((hkv, l, d), gen) for l in lens]
    vs = [O.randn_bf16((hkv, l, d), gen) for l in lens]
    smax = 9000
    k = torch.zeros(b, hkv, smax, d, dtype=torch.bfloat16)
    v = torch.zeros_like(k)
    for i, l in enumerate(lens):
        k[i, :, :l], v[i, :, :l] = ks[i], vs[i]
    sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
    splits = 5 if mode == "splits" else 0
    need = G.workspace_bytes(b, hq, hkv, d, splits)
    guard = 1 << 16
    buf = torch.full((guard + need + guard,), 0xAB, dtype=torch.uint8, device=DEV)
    ws = buf[guard:guard + need]
    assert ws.data_ptr() % 256 == 0
    ws.zero_()
    kw = dict(workspace=ws, num_splits=splits or None)
    if mode == "stealing":
        kw["work_stealing"] = True
    if mode == "ticket":
        kw["ticket_merge"] = True
    if mode == "separate":
        kw["separate_merge"] = True
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    if mode == "fp8":
        k8, v8, kscale, vscale = fp8_utils.quantize_kv_fp8(kd.view(b * hkv, smax, d), vd.view(b * hkv, smax, d))
        kd, vd = k8.view(b, hkv, smax, d), v8.view(b, hkv, smax, d)
        kw.update(k_scale=kscale.view(b, hkv), v_scale=vscale.view(b, hkv))
    for _ in range(3):
        out = G.gqa_decode_attention_batched(qd, kd, vd, sl, **kw)
    assert G.read_status(ws) == 0
    assert bool((buf[:guard] == 0xAB).all()) and bool((buf[guard + need:] == 0xAB).all())
    if mode in ("balanced", "splits", "fp8"):
        # the default merge hands every partial back as zeros (the ticket-based modes only
        # promise zero control words and leave old partials behind)
        assert int(ws.count_nonzero().item()) == 0
    if mode != "fp8":
        ref = O.attend_batch(q, ks, vs)
        ok, ratio, mx = within_tolerance(out.cpu(), ref)
        assert ok, (mode, ratio, mx)
