"""The entry point for callers that cannot allocate device memory
(gqa_decode_attention_static_scratch): its scratch is an array inside the library image,
so a serving engine that owns all of HBM, or a language binding that cannot own a device
buffer, can still run the decode step.

Called through the C ABI exactly as such a caller would, twice in a row with different
batches (the second call finds the first call's partials and tickets in the shared array),
and compared with the workspace-taking entry on the same inputs.  Collected last so that a
failure here cannot hide the result of any other test."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _args(native, q, k, v, seq_lens, out, workspace=None, num_splits=0, flags=0):
    b, hq, d = q.shape
    _, hkv, smax, _ = k.shape
    a = native.DecodeArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    a.seq_lens = seq_lens.data_ptr()
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim = b, hq, hkv, d
    a.max_seq_len, a.total_rows = smax, b * hkv * smax
    a.q_dtype = a.kv_dtype = native.DTYPE_BF16
    a.kv_layout = native.LAYOUT_PADDED
    a.num_splits = num_splits
    a.flags = flags
    if workspace is not None:
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
    a.stream = torch.cuda.current_stream().cuda_stream
    return a


def test_static_scratch_entry_matches_workspace_entry():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gqa_decode_b200 import _native, build
    from oracle import gqa_oracle as O

    build.build()
    lib = _native.load()
    torch.cuda.set_device(0)
    gen = torch.Generator().manual_seed(2024)
    # two different batches: long sequences first (many partials and tickets), then short ones
    for lens, splits in (([9000, 1, 4097, 7], 0), ([300, 5000, 64, 2500], 3)):
        b, hq, hkv, d, smax = len(lens), 32, 8, 128, max(lens)
        q = O.randn_bf16((b, hq, d), gen).to(DEV)
        k = O.randn_bf16((b, hkv, smax, d), gen).to(DEV)
        v = O.randn_bf16((b, hkv, smax, d), gen).to(DEV)
        sl = torch.tensor(lens, dtype=torch.int32, device=DEV)
        need = ctypes.c_size_t()
        assert lib.gqa_decode_workspace_bytes(b, hq, hkv, d, splits, 0, ctypes.byref(need)) == 0
        ws = torch.zeros(need.value, dtype=torch.uint8, device=DEV)
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        fl = 0  # default static schedule: both entries sum in the same order
        assert lib.gqa_decode_attention(ctypes.byref(_args(_native, q, k, v, sl, want, ws, splits, fl))) == 0
        # no workspace is passed: the library's own array is the scratch
        assert lib.gqa_decode_attention_static_scratch(
            ctypes.byref(_args(_native, q, k, v, sl, got, None, splits, fl))) == 0
        torch.cuda.synchronize()
        # the workspace-taking launch reports its status word; the library's own array cannot be
        # read from outside, so for the other launch the output comparison below is the evidence
        st = ctypes.c_int32(-1)
        assert lib.gqa_decode_read_status(ws.data_ptr(), None, ctypes.byref(st)) == 0 and st.value == 0
        assert not torch.isnan(got.float()).any()
        err = (got.float() - want.float()).abs()
        assert bool((err <= 2e-2 + 1e-2 * want.float().abs()).all()), float(err.max())
        # same schedule, same arithmetic: in fact the two entries agree bit for bit
        assert torch.equal(got, want)
        # and with work stealing switched on it stays inside the tolerance
        got2 = torch.full_like(q, float("nan"))
        assert lib.gqa_decode_attention_static_scratch(
            ctypes.byref(_args(_native, q, k, v, sl, got2, None, splits, _native.FLAG_WORK_STEALING))) == 0
        torch.cuda.synchronize()
        err = (got2.float() - want.float()).abs()
        assert bool((err <= 2e-2 + 1e-2 * want.float().abs()).all()), float(err.max())
        ref = O.attend_batch(q.cpu(), [k[i, :, :l].cpu() for i, l in enumerate(lens)],
                             [v[i, :, :l].cpu() for i, l in enumerate(lens)])
        err = (got.cpu().float() - ref.float()).abs()
        assert bool((err <= 2e-2 + 1e-2 * ref.float().abs()).all())


def test_static_scratch_entry_rejects_oversized_launch():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from gqa_decode_b200 import _native, build

    build.build()
    lib = _native.load()
    torch.cuda.set_device(0)
    q = torch.zeros(1, 32, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, 8, 128, 128, dtype=torch.bfloat16, device=DEV)
    out = torch.empty_like(q)
    sl = torch.tensor([128], dtype=torch.int32, device=DEV)
    # 8 KV heads x 1400 explicit splits x 4 heads x 129 floats > 16 MiB of partials
    a = _args(_native, q, k, k, sl, out, None, num_splits=1400)
    assert lib.gqa_decode_attention_static_scratch(ctypes.byref(a)) == -5  # GQA_ERR_LIMIT
    assert lib.gqa_decode_attention_static_scratch(None) == -1
    # requests the entry does not serve are turned away by the argument checks, before anything
    # is enqueued that would touch the shared array: E4M3 caches, an unsupported head_dim
    a = _args(_native, q, k, k, sl, out, None)
    a.kv_dtype = _native.DTYPE_E4M3
    assert lib.gqa_decode_attention_static_scratch(ctypes.byref(a)) == -2  # GQA_ERR_SHAPE
    a = _args(_native, q, k, k, sl, out, None)
    a.head_dim = 96
    assert lib.gqa_decode_attention_static_scratch(ctypes.byref(a)) == -2
    # and an accepted call right after them is still correct
    a = _args(_native, q, k, k, sl, out, None)
    assert lib.gqa_decode_attention_static_scratch(ctypes.byref(a)) == 0
    torch.cuda.synchronize()
    assert bool((out == 0).all())  # zero K and V: uniform weights over zero rows
