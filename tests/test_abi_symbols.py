"""The shared library loads without a GPU and exports every function that
include/gqa_decode_b200.h declares (no compute call is made here)."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "gqa_decode_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gqa_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(native_lib):
    names = declared_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(native_lib, n), f"{n} declared in the header but not exported"


def test_binding_covers_header():
    from gqa_decode_b200 import _native

    assert sorted(_native.SIGNATURES) == declared_functions()


def test_struct_matches_header_fields():
    from gqa_decode_b200 import _native

    text = open(os.path.join(ROOT, "include", "gqa_decode_b200.h")).read()
    body = re.search(r"typedef struct gqa_decode_args \{(.*?)\} gqa_decode_args_t;", text, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = [re.split(r"[\s\*]+", ln.strip().rstrip(";"))[-1] for ln in body.split(";") if ln.strip()]
    assert fields == [f[0] for f in _native.DecodeArgs._fields_]


def test_host_only_entries(native_lib):
    assert b"sm_100a" in native_lib.gqa_decode_version()
    assert native_lib.gqa_decode_tile_rows(128, 0) == 64
    assert native_lib.gqa_decode_tile_rows(128, 2) == 256
    assert native_lib.gqa_decode_tile_rows(96, 0) < 0
    n = ctypes.c_size_t(0)
    assert native_lib.gqa_decode_workspace_bytes(16, 32, 8, 128, 0, 148, ctypes.byref(n)) == 0
    assert n.value >= (16 * 8 + 148) * 4 * 129 * 4
    assert native_lib.gqa_decode_workspace_bytes(0, 32, 8, 128, 0, 148, ctypes.byref(n)) < 0
    assert native_lib.gqa_decode_attention(None) == -1
    assert native_lib.gqa_decode_attention_fp8(None) == -1
    assert native_lib.gqa_merge_partials(None, None, 1, 1, 128, None, 0, None, None, None) == -1


def _struct_fields(name):
    text = open(os.path.join(ROOT, "include", "gqa_decode_b200.h")).read()
    body = re.search(r"typedef struct %s \{(.*?)\} %s_t;" % (name, name), text, re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    return [re.split(r"[\s\*]+", ln.strip().rstrip(";"))[-1] for ln in body.split(";") if ln.strip()]


def test_auxiliary_structs_match_header():
    from gqa_decode_b200 import _native

    assert _struct_fields("gqa_gather_args") == [f[0] for f in _native.GatherArgs._fields_]
    assert _struct_fields("gqa_append_args") == [f[0] for f in _native.AppendArgs._fields_]


def test_argument_checks_need_no_gpu(native_lib):
    """Every entry validates its arguments before the first CUDA call: bad requests come back
    as negative codes on a machine without a GPU (the pointers below are never dereferenced)."""
    from gqa_decode_b200 import _native

    fake = 0x1000  # non-null, 16-byte aligned, never touched
    a = _native.DecodeArgs()
    for f in ("q", "k", "v", "out", "workspace"):
        setattr(a, f, fake)
    a.batch, a.num_q_heads, a.num_kv_heads, a.head_dim, a.max_seq_len, a.total_rows = 1, 32, 8, 128, 64, 512
    a.workspace_bytes = 1 << 20
    ptrs = (ctypes.c_void_p * 9)(*([fake] * 9))
    g = _native.GatherArgs()
    g.peer_out = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p))
    g.peer_flags = ctypes.cast(ptrs, ctypes.POINTER(ctypes.c_void_p))
    g.world, g.rank, g.epoch, g.mode = 9, 0, 1, 0           # more ranks than one NVLink domain
    assert native_lib.gqa_decode_attention_gather(ctypes.byref(a), ctypes.byref(g)) == -1
    g.world, g.rank = 2, 2                                   # rank outside the world
    assert native_lib.gqa_decode_attention_gather(ctypes.byref(a), ctypes.byref(g)) == -1
    g.rank, g.epoch = 0, 0                                   # epochs start at 1
    assert native_lib.gqa_decode_attention_gather(ctypes.byref(a), ctypes.byref(g)) == -1
    g.epoch, g.mode = 1, 7                                   # unknown mode
    assert native_lib.gqa_decode_attention_gather(ctypes.byref(a), ctypes.byref(g)) == -1
    g.mode, a.flags = 0, _native.FLAG_WORK_STEALING          # hand-off needs the static schedule
    assert native_lib.gqa_decode_attention_gather(ctypes.byref(a), ctypes.byref(g)) == -1
    assert native_lib.gqa_decode_attention_gather(None, ctypes.byref(g)) == -1
    a.flags, a.kv_layout = 0, _native.LAYOUT_PAGED_HND        # paged without a block table
    assert native_lib.gqa_decode_attention(ctypes.byref(a)) == -1
    a.block_table, a.page_size, a.block_table_stride = fake, 48, 8   # 48 rows: neither divides 64 nor is a multiple
    assert native_lib.gqa_decode_attention(ctypes.byref(a)) == -2
    a.page_size, a.block_table_stride, a.max_seq_len = 16, 2, 64      # table too short for max_seq_len
    assert native_lib.gqa_decode_attention(ctypes.byref(a)) == -1

    p = _native.AppendArgs()
    for f in ("k_new", "v_new", "k_cache", "v_cache", "k_scale", "v_scale", "positions"):
        setattr(p, f, fake)
    p.batch, p.num_kv_heads, p.head_dim, p.max_seq_len = 1, 8, 126, 64   # head_dim not a multiple of 4
    assert native_lib.gqa_quantize_append_fp8(ctypes.byref(p)) == -2
    p.head_dim, p.kv_layout = 128, _native.LAYOUT_PACKED                  # packed caches cannot grow
    assert native_lib.gqa_quantize_append_fp8(ctypes.byref(p)) == -1
    p.kv_layout = _native.LAYOUT_PAGED_NHD                                # paged without a table
    assert native_lib.gqa_quantize_append_fp8(ctypes.byref(p)) == -1
    assert native_lib.gqa_quantize_append_fp8(None) == -1
