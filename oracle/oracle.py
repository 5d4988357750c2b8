"""ctypes binding of the CPU oracle (oracle/w4a16_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests, by the smoke check and by the
benchmark's CPU-baseline leg. The product path never imports this module.

All tensors are numpy arrays in the on-disk compressed-tensors layout:
  packed uint32 [N, K/8], scale uint16 (bf16 bits) [N, G], zp uint32 [N/8, G],
  activations uint16 (bf16 bits) [M, K].
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libw4a16_oracle.so")
_REF_PATH = os.path.join(_HERE, "_ref", "libw4a16_ref.so")


def build(force: bool = False) -> None:
    """Compile the oracle (and the reference-header wrapper when the reference
    checkout is present) with the Makefile next to this file."""
    if force or not os.path.exists(_LIB_PATH) or (
            os.path.getmtime(_LIB_PATH) < os.path.getmtime(os.path.join(_HERE, "w4a16_oracle.c"))):
        subprocess.check_call(["make", "-C", _HERE, "-s", "libw4a16_oracle.so"])
    subprocess.check_call(["make", "-C", _HERE, "-s", "ref"], stdout=subprocess.DEVNULL)


_lib = None
_ref = None

_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_i64 = C.c_int64


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        L.oracle_num_threads.restype = C.c_int
        L.oracle_set_num_threads.argtypes = [C.c_int]
        L.oracle_set_num_threads.restype = None
        L.oracle_f32_to_bf16.argtypes = [_f32p, _u16p, _i64]
        L.oracle_bf16_to_f32.argtypes = [_u16p, _f32p, _i64]
        L.oracle_unpack_q.argtypes = [_u32p, _i64, _i64, _i8p]
        L.oracle_unpack_zp.argtypes = [_u32p, _i64, _i64, _i8p]
        L.oracle_dequant_f32.argtypes = [_u32p, _u16p, _u32p, _i64, _i64, _i64, _i64, _i64, _f32p]
        L.oracle_dequant_bf16.argtypes = [_u32p, _u16p, _u32p, _i64, _i64, _i64, _i64, _i64, _u16p]
        L.oracle_gemm_f64.argtypes = [_u32p, _u16p, _u32p, _i64, _i64, _i64, _u16p, _i64,
                                      C.c_void_p, _i64, _f64p]
        L.oracle_gemm_f32.argtypes = [_u32p, _u16p, _u32p, _i64, _i64, _i64, _u16p, _i64, _f32p]
        L.oracle_argmax_bf16.argtypes = [_u16p, _i64, _i64, _i32p]
        L.oracle_lm_head_argmax.argtypes = [_u32p, _u16p, _u32p, _i64, _i64, _i64, _u16p, _i64,
                                            _i32p, C.c_void_p, C.c_void_p]
        L.oracle_quant_i4.argtypes = [_u16p, _i64, _i64, _i64, _u32p, _u16p, _u32p]
        L.oracle_quant_w8.argtypes = [_u16p, _i64, _i64, _i64, _i8p, _u16p]
        L.oracle_rmsnorm.argtypes = [_u16p, _u16p, _i64, _i64, C.c_float, _u16p]
        L.oracle_residual_add.argtypes = [_u16p, _u16p, _i64]
        L.oracle_swiglu.argtypes = [_u16p, _i64, _i64, _u16p]
        L.oracle_gemm_w8_f64.argtypes = [_i8p, _u16p, _i64, _i64, _i64, _u16p, _i64, C.c_void_p, _i64, _f64p]
        for f in ("oracle_f32_to_bf16", "oracle_bf16_to_f32", "oracle_unpack_q", "oracle_unpack_zp",
                  "oracle_dequant_f32", "oracle_dequant_bf16", "oracle_gemm_f64", "oracle_gemm_f32",
                  "oracle_argmax_bf16", "oracle_lm_head_argmax", "oracle_quant_i4", "oracle_quant_w8",
                  "oracle_gemm_w8_f64", "oracle_rmsnorm", "oracle_residual_add", "oracle_swiglu"):
            getattr(L, f).restype = None
        _lib = L
    return _lib


def ref_lib():
    """The reference's own unpack header behind a C ABI, or None if it was never built."""
    global _ref
    if _ref is None and os.path.exists(_REF_PATH):
        R = C.CDLL(_REF_PATH)
        R.ref_unpack_q.argtypes = [_u32p, _i64, _i64, _i8p]
        R.ref_unpack_zp.argtypes = [_u32p, _i64, _i64, _i8p]
        R.ref_dequant_f32.argtypes = [_u32p, _u16p, _u32p, _i64, _i64, _i64, _f32p]
        for f in ("ref_unpack_q", "ref_unpack_zp", "ref_dequant_f32"):
            getattr(R, f).restype = None
        _ref = R
    return _ref


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP thread count of the oracle (torchrun exports OMP_NUM_THREADS=1 to its children)."""
    lib().oracle_set_num_threads(int(n))


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def f32_to_bf16(a: np.ndarray) -> np.ndarray:
    a = _c(a, np.float32)
    out = np.empty(a.shape, np.uint16)
    lib().oracle_f32_to_bf16(a.reshape(-1), out.reshape(-1), a.size)
    return out


def bf16_to_f32(a: np.ndarray) -> np.ndarray:
    a = _c(a, np.uint16)
    out = np.empty(a.shape, np.float32)
    lib().oracle_bf16_to_f32(a.reshape(-1), out.reshape(-1), a.size)
    return out


def _dims(packed, scale):
    N, K = packed.shape[0], packed.shape[1] * 8
    G = scale.shape[1]
    return N, K, G, K // G


def unpack_q(packed):
    packed = _c(packed, np.uint32)
    N, K = packed.shape[0], packed.shape[1] * 8
    out = np.empty((N, K), np.int8)
    lib().oracle_unpack_q(packed, N, K, out)
    return out


def unpack_zp(zp, N):
    zp = _c(zp, np.uint32)
    G = zp.shape[1]
    out = np.empty((N, G), np.int8)
    lib().oracle_unpack_zp(zp, N, G, out)
    return out


def dequant_f32(packed, scale, zp, row0=0, nrows=None):
    packed, scale, zp = _c(packed, np.uint32), _c(scale, np.uint16), _c(zp, np.uint32)
    N, K, G, group = _dims(packed, scale)
    nrows = N - row0 if nrows is None else nrows
    out = np.empty((nrows, K), np.float32)
    lib().oracle_dequant_f32(packed, scale, zp, N, K, group, row0, nrows, out)
    return out


def dequant_bf16(packed, scale, zp, row0=0, nrows=None):
    packed, scale, zp = _c(packed, np.uint32), _c(scale, np.uint16), _c(zp, np.uint32)
    N, K, G, group = _dims(packed, scale)
    nrows = N - row0 if nrows is None else nrows
    out = np.empty((nrows, K), np.uint16)
    lib().oracle_dequant_bf16(packed, scale, zp, N, K, group, row0, nrows, out)
    return out


def gemm_f64(packed, scale, zp, x, rows=None):
    """fp64 reference Y[M, N] (or Y[M, len(rows)])."""
    packed, scale, zp = _c(packed, np.uint32), _c(scale, np.uint16), _c(zp, np.uint32)
    x = _c(x, np.uint16).reshape(-1, packed.shape[1] * 8)
    N, K, G, group = _dims(packed, scale)
    M = x.shape[0]
    if rows is None:
        out = np.empty((M, N), np.float64)
        lib().oracle_gemm_f64(packed, scale, zp, N, K, group, x, M, None, 0, out)
    else:
        rows = _c(rows, np.int64)
        out = np.empty((M, rows.size), np.float64)
        lib().oracle_gemm_f64(packed, scale, zp, N, K, group, x, M,
                              rows.ctypes.data_as(C.c_void_p), rows.size, out)
    return out


def gemm_f32(packed, scale, zp, x):
    """Dequant-then-fp32-matmul Y[M, N] (the timed CPU baseline)."""
    packed, scale, zp = _c(packed, np.uint32), _c(scale, np.uint16), _c(zp, np.uint32)
    x = _c(x, np.uint16).reshape(-1, packed.shape[1] * 8)
    N, K, G, group = _dims(packed, scale)
    M = x.shape[0]
    out = np.empty((M, N), np.float32)
    lib().oracle_gemm_f32(packed, scale, zp, N, K, group, x, M, out)
    return out


def argmax_bf16(logits):
    logits = _c(logits, np.uint16)
    M, N = logits.shape
    ids = np.empty(M, np.int32)
    lib().oracle_argmax_bf16(logits, M, N, ids)
    return ids


def lm_head_argmax(packed, scale, zp, x, want_logits=False):
    """Returns (ids int32 [M], gap_ulps float64 [M], logits uint16 [M,N] or None)."""
    packed, scale, zp = _c(packed, np.uint32), _c(scale, np.uint16), _c(zp, np.uint32)
    x = _c(x, np.uint16).reshape(-1, packed.shape[1] * 8)
    N, K, G, group = _dims(packed, scale)
    M = x.shape[0]
    ids = np.empty(M, np.int32)
    gaps = np.empty(M, np.float64)
    logits = np.empty((M, N), np.uint16) if want_logits else None
    lib().oracle_lm_head_argmax(packed, scale, zp, N, K, group, x, M, ids,
                                logits.ctypes.data_as(C.c_void_p) if want_logits else None,
                                gaps.ctypes.data_as(C.c_void_p))
    return ids, gaps, logits


def quant_i4(src_bf16, group=128):
    """bf16 [rows, cols] -> (packed, scale, zp) in on-disk layout (min/max asymmetric)."""
    src = _c(src_bf16, np.uint16)
    rows, cols = src.shape
    G = cols // group
    packed = np.zeros((rows, cols // 8), np.uint32)
    scale = np.zeros((rows, G), np.uint16)
    zp = np.zeros((rows // 8, G), np.uint32)
    lib().oracle_quant_i4(src, rows, cols, group, packed, scale, zp)
    return packed, scale, zp


# ------------------------------------------------------------------ INT8 g128 lm_head variant
def quant_w8(src_bf16, group=128):
    """bf16 [rows, cols] -> (q int8 [rows, cols], scale uint16 [rows, G]), symmetric per group."""
    src = _c(src_bf16, np.uint16)
    rows, cols = src.shape
    q = np.zeros((rows, cols), np.int8)
    scale = np.zeros((rows, cols // group), np.uint16)
    lib().oracle_quant_w8(src, rows, cols, group, q, scale)
    return q, scale


def gemm_w8_f64(q, scale, x, rows=None):
    """fp64 reference Y[M, N] (or Y[M, len(rows)]) of the int8 weights."""
    q, scale = _c(q, np.int8), _c(scale, np.uint16)
    N, K = q.shape
    group = K // scale.shape[1]
    x = _c(x, np.uint16).reshape(-1, K)
    M = x.shape[0]
    if rows is None:
        out = np.empty((M, N), np.float64)
        lib().oracle_gemm_w8_f64(q, scale, N, K, group, x, M, None, 0, out)
    else:
        rows = _c(rows, np.int64)
        out = np.empty((M, rows.size), np.float64)
        lib().oracle_gemm_w8_f64(q, scale, N, K, group, x, M, rows.ctypes.data_as(C.c_void_p), rows.size, out)
    return out


def argmax_with_gaps(y64):
    """fp64 logits [M, N] -> (ids, top-2 gap in bf16 ulps of the best, bf16 logits): the tail of
    oracle_lm_head_argmax for logits computed elsewhere (rounded fp64 -> fp32 -> bf16, as there)."""
    logits = f32_to_bf16(np.asarray(y64, np.float64).astype(np.float32))
    ids = argmax_bf16(logits)
    lf = bf16_to_f32(logits)
    gaps = np.empty(len(ids), np.float64)
    for m, i in enumerate(ids):
        best = float(lf[m, i])
        rest = np.delete(lf[m], i)
        second = float(rest.max()) if rest.size else -3.4e38
        e = np.frexp(abs(best) if best != 0 else 1e-30)[1]
        gaps[m] = (best - second) / 2.0 ** (e - 8)
    return ids, gaps, logits


# ------------------------------------------------------------------ elementwise neighbours of a linear layer
def rmsnorm(x, w, eps=1e-6):
    """bf16 bits [rows, dim], weights bf16 bits [dim] -> bf16 bits [rows, dim]: x * rsqrt(mean(x^2)+eps) * (1 + w)."""
    x, w = _c(x, np.uint16), _c(w, np.uint16)
    rows, dim = x.shape
    out = np.empty((rows, dim), np.uint16)
    lib().oracle_rmsnorm(x, w, rows, dim, eps, out)
    return out


def residual_add(h, x):
    """bf16 bits: returns bf16(float(h) + float(x)) (the reference updates h in place)."""
    out = _c(h, np.uint16).copy()
    lib().oracle_residual_add(out.reshape(-1), _c(x, np.uint16).reshape(-1), out.size)
    return out


def swiglu(fused):
    """bf16 bits [rows, 2*inter] laid out [gate | up] -> bf16 bits [rows, inter] = silu(gate) * up."""
    fused = _c(fused, np.uint16)
    rows, two = fused.shape
    out = np.empty((rows, two // 2), np.uint16)
    lib().oracle_swiglu(fused, rows, two // 2, out)
    return out
