"""Host replay of the device scheduler's static schedule (gqa_schedule_dump): every key of
every (sequence, KV head) group is covered exactly once, partial slots never collide, each
group's bookkeeping (first_slot, n_parts) agrees across the CTAs that share it, and the
groups' slot ranges leave room for one partial per work chunk (what stealing can produce)."""
import numpy as np
import pytest


def dump(lib, lens, hkv, max_seq, tile, ctas, splits, layout):
    cap = 1 << 16
    rec = np.zeros((cap, 9), dtype=np.int64)
    arr = None if lens is None else np.asarray(lens, dtype=np.int32)
    batch = len(lens) if lens is not None else 3
    n = lib.gqa_schedule_dump(None if arr is None else arr.ctypes.data, batch, hkv, max_seq, tile,
                              ctas, splits, layout, rec.ctypes.data, cap)
    assert 0 <= n <= cap
    return rec[:n], batch


def check(rec, lens, batch, hkv, max_seq, tile, ctas, splits, layout):
    lens = [max_seq] * batch if lens is None else [min(l, max_seq) if layout == 0 else l for l in lens]
    covered = {}
    slots = set()
    info = {}
    cu = np.concatenate([[0], np.cumsum(lens)])
    for cta, b, h, r0, r1, slot, first, nparts, row0 in rec:
        assert 0 <= cta < ctas and 0 <= b < batch and 0 <= h < hkv
        assert r0 % tile == 0 and r0 <= r1 <= lens[b]
        assert slot not in slots
        slots.add(slot)
        # explicit splits: K slots per group; balanced: one per group and CTA (what the library
        # lays out in the workspace)
        bound = batch * hkv * splits if splits else ctas + batch * hkv + 1
        assert 0 <= slot < bound
        assert first <= slot < first + nparts
        g = (b, h)
        assert info.setdefault(g, (first, nparts)) == (first, nparts)
        covered.setdefault(g, []).append((r0, r1))
        want_row0 = (b * hkv + h) * max_seq if layout == 0 else cu[b] * hkv + h * lens[b]
        assert row0 == want_row0
    for b in range(batch):
        for h in range(hkv):
            segs = sorted(s for s in covered.get((b, h), []) if s[0] != s[1] or splits)
            if lens[b] == 0 and not splits:
                assert not segs
                continue
            pos = 0
            for r0, r1 in segs:
                if r0 == r1:
                    continue  # empty chunk of an explicit split
                assert r0 == pos
                pos = r1
            assert pos == lens[b]
            first, nparts = info[(b, h)]
            assert len(covered[(b, h)]) == nparts
    if not splits:
        # balanced: CTAs own equal numbers (+-1) of cost units, where a unit is a tile or one of
        # the 2 overhead units every group carries (a range may end inside a group's overhead,
        # which this reconstruction charges to the CTA that holds the group's first tile)
        per = np.zeros(ctas, dtype=np.int64)
        for cta, b, h, r0, r1, *_ in rec:
            per[cta] += -(-(r1 - r0) // tile) + (2 if r0 == 0 else 0)
        used = per[per > 0]
        assert used.max() - used.min() <= 1 + 2 + 2
        # slot ranges of different groups are disjoint
        spans = sorted((first, first + nparts) for first, nparts in info.values())
        firsts = sorted(set(first for first, _ in info.values()))
        assert len(firsts) == len(info)


CASES = [
    ([1, 7, 32768, 500, 12345], 8, 32768, 64, 148, 0),
    ([1, 7, 32768, 500, 12345], 8, 32768, 64, 148, 5),
    ([16384], 8, 16384, 64, 148, 0),
    ([16384], 8, 16384, 64, 148, 264),
    ([131072], 8, 131072, 64, 148, 0),
    ([0, 5, 0, 0, 64, 65, 0], 4, 128, 64, 148, 0),
    ([0, 5, 0, 0, 64, 65, 0], 4, 128, 64, 7, 3),
    ([3], 1, 3, 128, 148, 0),
    (None, 2, 1000, 128, 5, 0),
    (None, 2, 1000, 128, 5, 1),
    (list(range(1, 80)), 2, 100, 64, 148, 0),
    ([8192] * 64, 8, 8192, 64, 148, 0),
    ([8192] * 64, 1, 8192, 128, 148, 0),
]


@pytest.mark.parametrize("layout", [0, 1])
@pytest.mark.parametrize("lens,hkv,max_seq,tile,ctas,splits", CASES)
def test_schedule_invariants(native_lib, lens, hkv, max_seq, tile, ctas, splits, layout):
    if layout == 1 and lens is None:
        pytest.skip("packed layout needs lengths")
    rec, batch = dump(native_lib, lens, hkv, max_seq, tile, ctas, splits, layout)
    check(rec, lens, batch, hkv, max_seq, tile, ctas, splits, layout)


def test_schedule_random(native_lib):
    rng = np.random.default_rng(0)
    for _ in range(200):
        batch = int(rng.integers(1, 40))
        hkv = int(rng.choice([1, 2, 4, 8]))
        max_seq = int(rng.integers(1, 3000))
        lens = rng.integers(0, max_seq + 1, batch).tolist()
        tile = int(rng.choice([64, 128]))
        ctas = int(rng.integers(1, 200))
        splits = int(rng.choice([0, 0, 1, 3, 17]))
        layout = int(rng.integers(0, 2))
        rec, _ = dump(native_lib, lens, hkv, max_seq, tile, ctas, splits, layout)
        check(rec, lens, batch, hkv, max_seq, tile, ctas, splits, layout)


@pytest.mark.parametrize("splits", [0, 3])
def test_paged_layouts_share_the_padded_schedule(native_lib, splits):
    """Where rows live does not enter the schedule: paged layouts (2, 3) replay to exactly the
    padded layout's segments and slots (lengths clamped to max_seq alike); only the row base is
    left to the block table (reported as 0)."""
    lens = [1, 7, 5000, 0, 2500, 64, 65, 9000]
    padded, _ = dump(native_lib, lens, 8, 5120, 64, 148, splits, 0)
    for layout in (2, 3):
        paged, _ = dump(native_lib, lens, 8, 5120, 64, 148, splits, layout)
        assert paged.shape == padded.shape
        assert np.array_equal(paged[:, :8], padded[:, :8])
        assert (paged[:, 8] == 0).all()


def test_closed_form_setup_matches_general_path(native_lib):
    """Uniform batches take a closed-form scheduler set-up (host-prepared geometry and
    multiply-shift reciprocals).  gqa_schedule_dump replays such a launch both ways and returns
    an error unless the two agree segment for segment; sweep shapes, tiles and CTA counts."""
    rng = np.random.default_rng(7)
    cases = [(1, 8, 16384, 64, 148), (1, 8, 131072, 64, 148), (64, 8, 8192, 64, 148), (64, 1, 8192, 64, 148),
             (8, 8, 32768, 256, 148), (1, 1, 1, 64, 148), (3, 5, 63, 64, 7), (2, 32, 4096, 128, 132),
             (300, 8, 777, 64, 148), (1, 8, 16384, 64, 1)]
    for _ in range(150):
        cases.append((int(rng.integers(1, 70)), int(rng.integers(1, 33)), int(rng.integers(1, 40000)),
                      int(rng.choice([64, 128, 256])), int(rng.integers(1, 300))))
    for batch, hkv, max_seq, tile, ctas in cases:
        cap = 1 << 18
        rec = np.zeros((cap, 9), dtype=np.int64)
        n = native_lib.gqa_schedule_dump(None, batch, hkv, max_seq, tile, ctas, 0, 0, rec.ctypes.data, cap)
        assert n >= 0, (batch, hkv, max_seq, tile, ctas, n)
        # and the schedule itself covers every key exactly once
        keys = sum(int(r[4] - r[3]) for r in rec[:min(n, cap)])
        if n <= cap:
            assert keys == batch * hkv * max_seq
