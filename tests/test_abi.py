"""The C-ABI library loads on a machine without a GPU and exports every declared entry point."""
import ctypes
import re

import pytest


def _declared(header_path):
    text = open(header_path).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(w4a16_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol(pkg):
    names = _declared(pkg.HEADER_PATH)
    assert len(names) >= 18
    raw = ctypes.CDLL(pkg.LIB_PATH)
    missing = [n for n in names if not hasattr(raw, n)]
    assert not missing, f"declared in the header but not exported: {missing}"
    # and the Python binding covers the same set
    assert sorted(pkg.exported_symbols()) == names
    pkg.lib()


def test_host_side_argument_errors_need_no_gpu(pkg):
    L = pkg.lib()
    w = pkg.Weights()
    assert L.w4a16_weights_alloc(ctypes.byref(w), 100, 512, 128, None) == -1  # out_f not a multiple of 16
    assert b"out_f" in L.w4a16_last_error()
    assert L.w4a16_weights_alloc(ctypes.byref(w), 128, 512, 32, None) == -1   # group 32 unsupported
    assert L.w4a16_weights_alloc(ctypes.byref(w), 128, 500, 128, None) == -1
    b, e = ctypes.c_int(), ctypes.c_int()
    assert L.w4a16_shard_rows(34816, 8, 3, ctypes.byref(b), ctypes.byref(e)) == 0
    assert (b.value, e.value) == (3 * 4352, 4 * 4352)
    assert L.w4a16_shard_rows(248320, 8, 7, ctypes.byref(b), ctypes.byref(e)) == 0
    assert (b.value, e.value) == (7 * 31040, 248320)
    assert L.w4a16_shard_rows(5120, 8, 8, ctypes.byref(b), ctypes.byref(e)) == -5   # rank out of range
    assert L.w4a16_shard_rows(5136, 8, 0, ctypes.byref(b), ctypes.byref(e)) == -5   # not whole blocks
    assert L.w4a16_gemv(None, 0, None, None, None, None) == -1
    w8 = pkg.W8Weights()
    assert L.w4a16_w8_quantize(ctypes.byref(w8), None, 128, 512, 128, None) == -1   # null source
    assert L.w4a16_w8_gemv(None, None, None, None, None) == -1
    assert L.w4a16_selftest_wait_timeout(0, None) == -1


def test_struct_layouts_match_header(pkg):
    # 3 pointers + 4 ints; 3 pointers + 5 ints (+pad) + size_t; pointer + size_t + int (+pad) + pointer
    assert ctypes.sizeof(pkg.Weights) == 40
    assert ctypes.sizeof(pkg.Scratch) == 56
    assert ctypes.sizeof(pkg.Workspace) == 32
    assert ctypes.sizeof(pkg.W8Weights) == 32   # 2 pointers + 4 ints
