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
