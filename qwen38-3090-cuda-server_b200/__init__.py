"""B200 (sm_100a) W4A16 matmul path: Python binding of the C ABI in include/w4a16_b200.h.

The product is the shared library `libw4a16_b200.so` (hand-written CUDA behind
`extern "C"` entry points) plus the C++ drop-in headers in `dropin/kernels/`.
This module is the thin ctypes layer the tests and the benchmark use: torch only
supplies device memory and streams. There is no CPU fallback: if the library is
missing or cannot be loaded, importing an entry point raises.

Function names mirror the reference launchers they stand in for
(src/kernels/gemv_w4a16.cuh, src/kernels/gemm_w4a16.cuh of the reference project).
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libw4a16_b200.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "w4a16_b200.h")


class W4A16Error(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"w4a16 error {code}: {msg}")
        self.code = code


class Weights(C.Structure):
    """w4a16_weights_t == qwen::W4A16Weights (src/kernels/gemv_w4a16.cuh:50-60)."""
    _fields_ = [("qweight", C.c_void_p), ("scale", C.c_void_p), ("zp", C.c_void_p),
                ("out_f", C.c_int), ("in_f", C.c_int), ("group_size", C.c_int), ("num_groups", C.c_int)]

    def qweight_bytes(self):
        return self.out_f * self.in_f // 2

    def scale_bytes(self):
        return self.out_f * self.num_groups * 2

    def zp_bytes(self):
        return self.out_f * self.num_groups

    def total_bytes(self):
        return self.qweight_bytes() + self.scale_bytes() + self.zp_bytes()


class W8Weights(C.Structure):
    """w4a16_w8_weights_t == qwen::W8A16Weights (src/kernels/gemv_w4a16.cuh:148-155)."""
    _fields_ = [("qweight", C.c_void_p), ("scale", C.c_void_p),
                ("out_f", C.c_int), ("in_f", C.c_int), ("group_size", C.c_int), ("num_groups", C.c_int)]

    def total_bytes(self):
        return self.out_f * self.in_f + self.out_f * self.num_groups * 2


class Comm(C.Structure):
    """w4a16_comm_t: every rank's 256-byte flag block (peer-mapped), number of ranks, this rank."""
    _fields_ = [("blocks", C.c_void_p * 8), ("nranks", C.c_int), ("rank", C.c_int)]


class Scratch(C.Structure):
    """w4a16_scratch_t == qwen::GemvScratch (src/kernels/gemv_w4a16.cuh:94-104)."""
    _fields_ = [("xf", C.c_void_p), ("xgsum", C.c_void_p), ("partial", C.c_void_p),
                ("max_in", C.c_int), ("max_groups", C.c_int), ("max_out", C.c_int),
                ("max_splits", C.c_int), ("max_m", C.c_int), ("partial_elems", C.c_size_t)]


class Workspace(C.Structure):
    """w4a16_workspace_t == qwen::GemmWorkspace (src/kernels/gemm_w4a16.cuh:30-35)."""
    _fields_ = [("wbuf", C.c_void_p), ("bytes", C.c_size_t), ("max_rows", C.c_int),
                ("cublas", C.c_void_p)]


_SIGNATURES = {
    "w4a16_last_error": (C.c_char_p, []),
    "w4a16_device_status": (C.c_int, []),
    "w4a16_device_status_clear": (C.c_int, []),
    "w4a16_selftest_wait_timeout": (C.c_int, [C.c_int, C.c_void_p]),
    "w4a16_scratch_reset": (C.c_int, [C.POINTER(Scratch), C.c_void_p]),
    "w4a16_gemv_static_reset": (C.c_int, [C.c_void_p]),
    "w4a16_w8_quantize": (C.c_int, [C.POINTER(W8Weights), C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "w4a16_w8_free": (C.c_int, [C.POINTER(W8Weights)]),
    "w4a16_w8_unpack_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(W8Weights), C.c_int, C.c_int, C.c_void_p]),
    "w4a16_w8_gemv": (C.c_int, [C.c_void_p, C.POINTER(W8Weights), C.c_void_p, C.POINTER(Scratch), C.c_void_p]),
    "w4a16_w8_gemm_skinny": (C.c_int, [C.c_void_p, C.POINTER(W8Weights), C.c_void_p, C.c_int,
                                       C.POINTER(Scratch), C.c_void_p]),
    "w4a16_w8_lm_head_argmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(W8Weights),
                                          C.c_void_p, C.c_int, C.POINTER(Scratch), C.c_void_p]),
    "w4a16_weights_alloc": (C.c_int, [C.POINTER(Weights), C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "w4a16_repack_into": (C.c_int, [C.POINTER(Weights), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                    C.c_int, C.c_void_p]),
    "w4a16_weights_free": (C.c_int, [C.POINTER(Weights)]),
    "w4a16_scratch_alloc": (C.c_int, [C.POINTER(Scratch), C.c_int, C.c_int, C.c_int, C.c_int]),
    "w4a16_scratch_free": (C.c_int, [C.POINTER(Scratch)]),
    "w4a16_scratch_check": (C.c_int, [C.POINTER(Scratch), C.c_int, C.c_int]),
    "w4a16_choose_splits": (C.c_int, [C.c_int, C.c_int]),
    "w4a16_gemv": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(Weights), C.c_void_p, C.POINTER(Scratch),
                             C.c_void_p]),
    "w4a16_gemv_static": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(Weights), C.c_void_p, C.c_void_p]),
    "w4a16_gemm_skinny": (C.c_int, [C.c_void_p, C.POINTER(Weights), C.c_void_p, C.c_int,
                                    C.POINTER(Scratch), C.c_void_p]),
    "w4a16_lm_head_argmax": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(Weights),
                                       C.c_void_p, C.c_int, C.POINTER(Scratch), C.c_void_p]),
    "w4a16_argmax_pairs_reduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "w4a16_dequant_rows": (C.c_int, [C.c_void_p, C.POINTER(Weights), C.c_int, C.c_int, C.c_void_p]),
    "w4a16_workspace_alloc": (C.c_int, [C.POINTER(Workspace), C.c_size_t]),
    "w4a16_workspace_free": (C.c_int, [C.POINTER(Workspace)]),
    "w4a16_gemm_prefill": (C.c_int, [C.c_void_p, C.POINTER(Weights), C.c_void_p, C.c_int,
                                     C.POINTER(Workspace), C.c_void_p]),
    "w4a16_gemm_skinny_gather": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(Comm), C.c_int, C.c_int, C.c_int,
                                           C.POINTER(Weights), C.c_void_p, C.c_int, C.POINTER(Scratch), C.c_void_p]),
    "w4a16_gemm_skinny_partial": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(Comm), C.POINTER(Weights), C.c_void_p,
                                            C.c_int, C.POINTER(Scratch), C.c_void_p]),
    "w4a16_reduce_partials": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(Comm), C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "w4a16_wait_gather": (C.c_int, [C.POINTER(Comm), C.c_void_p]),
    "w4a16_lm_head_argmax_sharded": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(Comm), C.c_int, C.c_int,
                                               C.POINTER(Weights), C.c_void_p, C.c_int, C.POINTER(Scratch), C.c_void_p]),
    "w4a16_w8_lm_head_argmax_sharded": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p), C.POINTER(Comm), C.c_int, C.c_int,
                                                  C.POINTER(W8Weights), C.c_void_p, C.c_int, C.POINTER(Scratch),
                                                  C.c_void_p]),
    "w4a16_gemm_prefill_sharded": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(Comm), C.c_int, C.c_int,
                                             C.POINTER(Weights), C.c_void_p, C.c_int, C.POINTER(Workspace), C.c_void_p]),
    "w4a16_linear_fused": (C.c_int, [C.c_void_p, C.POINTER(Weights), C.c_void_p, C.c_int, C.c_void_p, C.c_float,
                                     C.c_void_p, C.c_int, C.POINTER(Scratch), C.c_void_p]),
    "w4a16_repack_into_swiglu": (C.c_int, [C.POINTER(Weights), C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                           C.c_int, C.c_void_p]),
    "w4a16_shard_rows": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "w4a16_gemm_skinny_sharded": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.POINTER(Weights), C.c_void_p, C.c_int, C.POINTER(Scratch),
                                            C.c_void_p]),
}

_lib = None


def lib():
    """The loaded C-ABI library. Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python {os.path.join(_HERE, 'build.py')}` "
                              "(nvcc, sm_100a). The W4A16 path has no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(L, name)  # AttributeError if the library lacks a declared entry point
            fn.restype = res
            fn.argtypes = args
        _lib = L
    return _lib


def exported_symbols():
    return list(_SIGNATURES)


def check(rc: int):
    if rc != 0:
        raise W4A16Error(rc, lib().w4a16_last_error().decode())


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream(stream=None):
    import torch
    s = torch.cuda.current_stream() if stream is None else stream
    return C.c_void_p(s.cuda_stream)


# --------------------------------------------------------------------- weights
def awq_alloc_fused(out_f: int, in_f: int, group_size: int = 128) -> Weights:
    w = Weights()
    check(lib().w4a16_weights_alloc(C.byref(w), out_f, in_f, group_size, _stream()))
    return w


def awq_repack_into(w: Weights, dst_row_offset: int, packed, scale, zp, stream=None):
    """packed int32/uint32 [out,in/8], scale bf16 [out,G], zp int32 [out/8,G]: device tensors."""
    check(lib().w4a16_repack_into(C.byref(w), dst_row_offset, _ptr(packed), _ptr(scale), _ptr(zp),
                                  packed.shape[0], _stream(stream)))


def awq_repack(packed, scale, zp, group_size: int = 128) -> Weights:
    out_f, in_f = packed.shape[0], packed.shape[1] * 8
    w = awq_alloc_fused(out_f, in_f, group_size)
    awq_repack_into(w, 0, packed, scale, zp)
    return w


def awq_free(w: Weights):
    check(lib().w4a16_weights_free(C.byref(w)))


def weights_from_numpy(packed, scale, zp, group_size: int = 128) -> Weights:
    """Host arrays in on-disk layout (uint32, bf16 bits as uint16, uint32) -> device container."""
    import numpy as np
    import torch
    dp = torch.from_numpy(np.ascontiguousarray(packed).view(np.int32)).cuda()
    ds = torch.from_numpy(np.ascontiguousarray(scale).view(np.int16)).cuda()
    dz = torch.from_numpy(np.ascontiguousarray(zp).view(np.int32)).cuda()
    w = awq_repack(dp, ds, dz, group_size)
    torch.cuda.synchronize()
    return w


# --------------------------------------------------------------------- scratch
def gemv_scratch_alloc(max_in: int, max_out: int, min_group: int = 128, max_m: int = 1) -> Scratch:
    s = Scratch()
    check(lib().w4a16_scratch_alloc(C.byref(s), max_in, max_out, min_group, max_m))
    return s


def gemv_scratch_free(s: Scratch):
    check(lib().w4a16_scratch_free(C.byref(s)))


# --------------------------------------------------------------------- launchers
def gemv_w4a16(y, w: Weights, x, s: Scratch, stream=None):
    """y bf16 [out_f] = W x."""
    check(lib().w4a16_gemv(_ptr(y), 0, C.byref(w), _ptr(x), C.byref(s), _stream(stream)))


def gemv_w4a16_f32(y, w: Weights, x, s: Scratch, stream=None):
    check(lib().w4a16_gemv(_ptr(y), 1, C.byref(w), _ptr(x), C.byref(s), _stream(stream)))


def gemv_w4a16_static(y, w: Weights, x, f32: bool = False, stream=None):
    """The GEMV with the library's built-in scratch: nothing is allocated, no Scratch is passed."""
    check(lib().w4a16_gemv_static(_ptr(y), 1 if f32 else 0, C.byref(w), _ptr(x), _stream(stream)))


def gemm_small_w4a16(y, w: Weights, x, M: int, s: Scratch, stream=None):
    """Y bf16 [M,out_f] = X[M,in_f] W^T, 1 <= M <= 16."""
    check(lib().w4a16_gemm_skinny(_ptr(y), C.byref(w), _ptr(x), M, C.byref(s), _stream(stream)))


gemm_mma_w4a16 = gemm_small_w4a16  # same contract in the reference; one kernel here


def lm_head_argmax(ids, w: Weights, x, M: int, s: Scratch, logits=None, pairs=None, row_offset: int = 0,
                   stream=None):
    check(lib().w4a16_lm_head_argmax(_ptr(ids), _ptr(logits), _ptr(pairs), row_offset, C.byref(w), _ptr(x),
                                     M, C.byref(s), _stream(stream)))


def argmax_pairs_reduce(ids, pairs, nranks: int, M: int, stream=None):
    check(lib().w4a16_argmax_pairs_reduce(_ptr(ids), _ptr(pairs), nranks, M, _stream(stream)))


def w4a16_dequant_rows(dst, w: Weights, row0: int, nrows: int, stream=None):
    check(lib().w4a16_dequant_rows(_ptr(dst), C.byref(w), row0, nrows, _stream(stream)))


def gemm_workspace_alloc(nbytes: int) -> Workspace:
    ws = Workspace()
    check(lib().w4a16_workspace_alloc(C.byref(ws), nbytes))
    return ws


def gemm_workspace_free(ws: Workspace):
    check(lib().w4a16_workspace_free(C.byref(ws)))


def gemm_w4a16(Cout, w: Weights, A, M: int, ws: Workspace, stream=None):
    check(lib().w4a16_gemm_prefill(_ptr(Cout), C.byref(w), _ptr(A), M, C.byref(ws), _stream(stream)))


def shard_rows(out_f: int, nranks: int, rank: int):
    b, e = C.c_int(), C.c_int()
    check(lib().w4a16_shard_rows(out_f, nranks, rank, C.byref(b), C.byref(e)))
    return b.value, e.value


def gemm_skinny_sharded(y_peer_ptrs, rank: int, out_f_total: int, row_begin: int, w: Weights, x, M: int,
                        s: Scratch, stream=None):
    n = len(y_peer_ptrs)
    arr = (C.c_void_p * n)(*[C.c_void_p(p) for p in y_peer_ptrs])
    check(lib().w4a16_gemm_skinny_sharded(arr, n, rank, out_f_total, row_begin, C.byref(w), _ptr(x), M,
                                          C.byref(s), _stream(stream)))


COMM_BLOCK_BYTES = 256


def make_comm(block_ptrs, rank: int) -> Comm:
    """block_ptrs: every rank's zero-initialised 256-byte flag block as mapped on this rank."""
    c = Comm()
    for i, ptr in enumerate(block_ptrs):
        c.blocks[i] = ptr
    c.nranks, c.rank = len(block_ptrs), rank
    return c


def _ptr_table(ptrs):
    return (C.c_void_p * len(ptrs))(*[C.c_void_p(p) for p in ptrs])


def gemm_skinny_gather(y_peer_ptrs, comm: Comm, out_f_total: int, row_begin: int, w: Weights, x, M: int, s: Scratch,
                       wait_prev: bool = False, stream=None):
    """Sharded skinny GEMM with the fused all-gather and its completion flag; wait_prev: x is the gathered
    output of the previous launch on this communicator."""
    check(lib().w4a16_gemm_skinny_gather(_ptr_table(y_peer_ptrs), C.byref(comm), 1 if wait_prev else 0, out_f_total,
                                         row_begin, C.byref(w), _ptr(x), M, C.byref(s), _stream(stream)))


def gemm_skinny_partial(partial_peer_ptrs, comm: Comm, w_kshard: Weights, x_slice, M: int, s: Scratch, stream=None):
    """K-sharded layer: this rank's fp32 partial goes into slot `rank` of every rank's buffer, then the flag."""
    check(lib().w4a16_gemm_skinny_partial(_ptr_table(partial_peer_ptrs), C.byref(comm), C.byref(w_kshard), _ptr(x_slice),
                                          M, C.byref(s), _stream(stream)))


def reduce_partials(y, partials_local, comm: Comm, M: int, out_f: int, residual: bool = False, stream=None):
    """Waits for every rank's partial, adds them in rank order, writes (or adds to) the bf16 y [M, out_f]."""
    check(lib().w4a16_reduce_partials(_ptr(y), _ptr(partials_local), C.byref(comm), M, out_f, 1 if residual else 0,
                                      _stream(stream)))


def wait_gather(comm: Comm, stream=None):
    check(lib().w4a16_wait_gather(C.byref(comm), _stream(stream)))


def lm_head_argmax_sharded(ids, pair_table_ptrs, comm: Comm, row_offset: int, w, x, M: int, s: Scratch,
                           wait_prev: bool = False, stream=None):
    """Vocab-sharded lm_head in one launch (int4 or int8 weights): ids[M] complete on every rank."""
    fn = lib().w4a16_w8_lm_head_argmax_sharded if isinstance(w, W8Weights) else lib().w4a16_lm_head_argmax_sharded
    check(fn(_ptr(ids), _ptr_table(pair_table_ptrs), C.byref(comm), 1 if wait_prev else 0, row_offset, C.byref(w),
             _ptr(x), M, C.byref(s), _stream(stream)))


def gemm_w4a16_sharded(c_peer_ptrs, comm: Comm, out_f_total: int, row_begin: int, w: Weights, A, M: int,
                       ws: Workspace, stream=None):
    check(lib().w4a16_gemm_prefill_sharded(_ptr_table(c_peer_ptrs), C.byref(comm), out_f_total, row_begin, C.byref(w),
                                           _ptr(A), M, C.byref(ws), _stream(stream)))


EPILOGUE_NONE, EPILOGUE_SWIGLU, EPILOGUE_RESIDUAL = 0, 1, 2


def awq_repack_into_swiglu(w: Weights, dst_row_offset: int, packed, scale, zp, inter: int, stream=None):
    """awq_repack_into for a gate|up container that will run with the fused SwiGLU epilogue (rows interleaved)."""
    check(lib().w4a16_repack_into_swiglu(C.byref(w), dst_row_offset, _ptr(packed), _ptr(scale), _ptr(zp),
                                         packed.shape[0], inter, _stream(stream)))


def linear_fused(y, w: Weights, x, M: int, s: Scratch, ln_weight=None, ln_eps: float = 1e-6, xn_out=None,
                 epilogue: int = EPILOGUE_NONE, stream=None):
    """A linear layer with RMSNorm in front and / or SwiGLU or the residual add behind, in one call."""
    check(lib().w4a16_linear_fused(_ptr(y), C.byref(w), _ptr(x), M, _ptr(ln_weight), ln_eps, _ptr(xn_out), epilogue,
                                   C.byref(s), _stream(stream)))


def device_status() -> int:
    return int(lib().w4a16_device_status())


def device_status_clear():
    check(lib().w4a16_device_status_clear())


def selftest_wait_timeout(polls: int = 64, stream=None):
    """One tiny kernel whose only wait can never be satisfied: it gives up and sets the status word."""
    check(lib().w4a16_selftest_wait_timeout(polls, _stream(stream)))


def gemv_scratch_reset(s: Scratch, stream=None):
    check(lib().w4a16_scratch_reset(C.byref(s), _stream(stream)))


def gemv_static_reset(stream=None):
    check(lib().w4a16_gemv_static_reset(_stream(stream)))


# --------------------------------------------------------------------- INT8 lm_head (W8A16)
def quantize_w8a16(src, group_size: int = 128, stream=None) -> W8Weights:
    """src: device bf16 [out_f, in_f] -> symmetric int8 g128 container."""
    w = W8Weights()
    check(lib().w4a16_w8_quantize(C.byref(w), _ptr(src), src.shape[0], src.shape[1], group_size, _stream(stream)))
    return w


def w8a16_free(w: W8Weights):
    check(lib().w4a16_w8_free(C.byref(w)))


def w8a16_unpack_rows(q, scale, w: W8Weights, row0: int, nrows: int, stream=None):
    check(lib().w4a16_w8_unpack_rows(_ptr(q), _ptr(scale), C.byref(w), row0, nrows, _stream(stream)))


def gemv_w8a16(y, w: W8Weights, x, s: Scratch, stream=None):
    check(lib().w4a16_w8_gemv(_ptr(y), C.byref(w), _ptr(x), C.byref(s), _stream(stream)))


def gemm_small_w8a16(y, w: W8Weights, x, M: int, s: Scratch, stream=None):
    check(lib().w4a16_w8_gemm_skinny(_ptr(y), C.byref(w), _ptr(x), M, C.byref(s), _stream(stream)))


def lm_head_argmax_w8(ids, w: W8Weights, x, M: int, s: Scratch, logits=None, pairs=None, row_offset: int = 0,
                      stream=None):
    check(lib().w4a16_w8_lm_head_argmax(_ptr(ids), _ptr(logits), _ptr(pairs), row_offset, C.byref(w), _ptr(x),
                                        M, C.byref(s), _stream(stream)))
