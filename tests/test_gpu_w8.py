"""GPU parity of the INT8 (W8A16) lm_head variant through the C ABI against the CPU oracle.

The quantiser is checked bit for bit (codes and bf16 scales, read back with w4a16_w8_unpack_rows);
GEMV / skinny outputs with the tolerances of the int4 path (bf16 outputs: max|y-ref|/max|ref| <= 1e-2
plus the per-element bound); fused-argmax ids identical to the oracle's unless its own two bf16
logits are equal. The reference's functions: src/kernels/gemv_w4a16.cu:479-634.
"""
import numpy as np
import pytest
import torch

from gpu_util import Guarded, dev_bf16, host_bits
from test_gpu_parity import _check_bf16

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def scratch(pkg):
    s = pkg.gemv_scratch_alloc(17408, 248320, 128, 16)
    yield s
    pkg.gemv_scratch_free(s)


def _w8(pkg, oracle, synth, N, K, seed, sigma=0.02):
    src = synth.make_activations(N, K, seed=seed, sigma=sigma)  # bf16 [N, K] ~ N(0, sigma): an lm_head-like matrix
    q, scale = oracle.quant_w8(src)
    w = pkg.quantize_w8a16(dev_bf16(src))
    torch.cuda.synchronize()
    return src, q, scale, w


@pytest.mark.parametrize("N,K", [(32, 128), (208, 1024), (1040, 5120), (4096, 640)])
def test_w8_quantize_bit_exact(pkg, oracle, synth, N, K):
    src, q, scale, w = _w8(pkg, oracle, synth, N, K, seed=N)
    src[5, :128] = 0  # an all-zero group
    pkg.w8a16_free(w)
    q, scale = oracle.quant_w8(src)
    w = pkg.quantize_w8a16(dev_bf16(src))
    gq = Guarded((N, K), torch.int8)
    gs = Guarded((N, K // 128), torch.int16)
    pkg.w8a16_unpack_rows(gq.t, gs.t, w, 0, N)
    torch.cuda.synchronize()
    assert gq.intact() and gs.intact()
    assert np.array_equal(gq.t.cpu().numpy(), q)
    assert np.array_equal(gs.t.cpu().numpy().view(np.uint16), scale)
    if N >= 48:  # a row window
        part = torch.empty((16, K), dtype=torch.int8, device="cuda")
        pkg.w8a16_unpack_rows(part, None, w, 23, 16)
        assert np.array_equal(part.cpu().numpy(), q[23:39])
    assert w.total_bytes() == N * K + N * (K // 128) * 2
    pkg.w8a16_free(w)


@pytest.mark.parametrize("N,K", [(32, 128), (208, 1024), (2048, 5120), (5120, 17408), (31040, 5120)])
def test_w8_gemv_matches_fp64_oracle(pkg, oracle, synth, scratch, N, K):
    src, q, scale, w = _w8(pkg, oracle, synth, N, K, seed=N + K)
    x = synth.make_activations(1, K, seed=N)
    ref = oracle.gemm_w8_f64(q, scale, x)[0]
    y = Guarded((N,), torch.bfloat16)
    pkg.gemv_w8a16(y.t, w, dev_bf16(x[0]), scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and y.intact()
    _check_bf16(host_bits(y.t), ref, synth)
    pkg.w8a16_free(w)


@pytest.mark.parametrize("M", [1, 2, 3, 5, 7, 8, 9, 12, 16])
def test_w8_skinny(pkg, oracle, synth, scratch, M):
    N, K = 1056, 2048
    src, q, scale, w = _w8(pkg, oracle, synth, N, K, seed=200 + M)
    x = synth.make_activations(M, K, seed=M)
    ref = oracle.gemm_w8_f64(q, scale, x)
    y = Guarded((M, N), torch.bfloat16)
    pkg.gemm_small_w8a16(y.t, w, dev_bf16(x), M, scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and y.intact()
    _check_bf16(host_bits(y.t), ref, synth)
    # run-to-run bitwise equality
    y2 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w8a16(y2, w, dev_bf16(x), M, scratch)
    assert torch.equal(y2.view(torch.int16), y.t.view(torch.int16))
    pkg.w8a16_free(w)


def _w8_argmax_case(pkg, oracle, synth, scratch, N, K, M, seed, with_logits):
    src, q, scale, w = _w8(pkg, oracle, synth, N, K, seed=seed)
    del src
    x = synth.make_activations(M, K, seed=seed + 1)
    want, gaps, ref_logits = oracle.argmax_with_gaps(oracle.gemm_w8_f64(q, scale, x))
    ids = Guarded((M,), torch.int32)
    logits = Guarded((M, N), torch.bfloat16) if with_logits else None
    pkg.lm_head_argmax_w8(ids.t, w, dev_bf16(x), M, scratch, logits=logits.t if logits else None)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and ids.intact()
    got = ids.t.cpu().numpy()
    lf = synth.bf16_bits_to_f32(ref_logits)
    ties = 0
    for m in range(M):
        if got[m] != want[m]:
            assert lf[m, want[m]] == lf[m, got[m]], f"row {m}: id {got[m]} vs oracle {want[m]} (top-2 gap {gaps[m]} ulp)"
            ties += 1
    print(f"int8 lm_head argmax N={N} M={M}: {ties} of {M} rows used the tie allowance")
    if logits is not None:
        assert logits.intact()
        assert np.array_equal(oracle.argmax_bf16(host_bits(logits.t)), got)
    pkg.w8a16_free(w)


@pytest.mark.parametrize("N,K,M", [(4096, 1024, 9), (31040, 5120, 9), (1200 * 16, 512, 16)])
def test_w8_lm_head_argmax_small(pkg, oracle, synth, scratch, N, K, M):
    _w8_argmax_case(pkg, oracle, synth, scratch, N, K, M, seed=N % 89, with_logits=True)


@pytest.mark.parametrize("M", [1, 9])
def test_w8_lm_head_argmax_full_vocab(pkg, oracle, synth, scratch, M):
    _w8_argmax_case(pkg, oracle, synth, scratch, 248320, 5120, M, seed=3, with_logits=False)
