"""GPU edge cases of the decode kernel's arithmetic and launch logic, against the fp64 oracle.

The decode kernel turns the activations of every (token, 128-k group) into 22-bit block fixed point
before the integer tensor-core product; these cases stress exactly that step (dynamic range inside
and across groups, zeros, tiny values, non-finite inputs) and the launcher's splitting of the
work (odd numbers of k groups, rows that do not fill a tile, token batches)."""
import numpy as np
import pytest
import torch

from gpu_util import Guarded, dev_bf16, host_bits, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def scratch(pkg):
    s = pkg.gemv_scratch_alloc(17408, 40960, 128, 16)
    yield s
    pkg.gemv_scratch_free(s)


def _weights(pkg, synth, N, K, seed):
    packed, scale, zp = synth.make_weights(N, K, seed=seed)
    return (packed, scale, zp), pkg.weights_from_numpy(packed, scale, zp)


def _bf16(a, synth):
    return synth.f32_to_bf16_bits(np.asarray(a, dtype=np.float32))


@pytest.mark.parametrize("case", ["outliers", "tiny", "group_scales", "zeros", "signs"])
def test_activation_dynamic_range(pkg, oracle, synth, scratch, case):
    """fp32 output within 1e-4 of the fp64 oracle (max|err| / max|ref|) whatever the activations look like."""
    N, K, M = 1056, 2048, 3
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=31)
    rng = np.random.Generator(np.random.PCG64(5))
    x = rng.standard_normal((M, K)).astype(np.float32)
    if case == "outliers":  # a few activations 10^4 times the rest, as LLM residual streams have
        x[:, rng.integers(0, K, 6)] *= 1e4
    elif case == "tiny":  # everything far below 1 (groups whose largest magnitude is under 2^-102 would be
        x *= np.float32(1e-20)  # kept with fewer than 22 bits; no activation of a real model is near that)
        x[1] *= np.float32(1e-8)
    elif case == "group_scales":  # every 128-k group at its own scale, 2^-40 .. 2^40
        x *= np.exp2(rng.integers(-40, 41, K // 128)).astype(np.float32).repeat(128)[None, :]
    elif case == "zeros":  # whole groups and whole tokens of zeros (and negative zeros)
        x[:, 256:768] = 0.0
        x[2] = -0.0
    elif case == "signs":  # one sign per group: no cancellation inside the group sums
        x = np.abs(x) * np.where(rng.random(K // 128) < 0.5, -1.0, 1.0).astype(np.float32).repeat(128)[None, :]
    xb = _bf16(x, synth)
    ref = oracle.gemm_f64(packed, scale, zp, xb)
    for m in range(M):
        y = Guarded((N,), torch.float32)
        pkg.gemv_w4a16_f32(y.t, w, dev_bf16(xb[m]), scratch)
        torch.cuda.synchronize()
        assert pkg.device_status() == 0 and y.intact()
        got = y.t.cpu().numpy().astype(np.float64)
        scale_m = np.max(np.abs(ref[m]))
        if scale_m == 0.0:
            assert not got.any()
        else:
            assert np.max(np.abs(got - ref[m])) / scale_m <= 1e-4, (case, m)
    pkg.awq_free(w)


def test_nonfinite_activation_poisons_only_its_token(pkg, oracle, synth, scratch):
    """An inf or NaN activation makes that token's outputs NaN (as a floating-point product would) and
    leaves the other tokens of the block exact."""
    N, K, M = 544, 1024, 4
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=77)
    x = synth.bf16_bits_to_f32(synth.make_activations(M, K, seed=3)).copy()
    x[1, 300] = np.inf
    x[3, 901] = np.nan
    xb = _bf16(x, synth)
    y = Guarded((M, N), torch.bfloat16)
    pkg.gemm_small_w4a16(y.t, w, dev_bf16(xb), M, scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and y.intact()
    got = synth.bf16_bits_to_f32(host_bits(y.t))
    assert np.isnan(got[1]).all() and np.isnan(got[3]).all()
    clean = xb[[0, 2]]
    ref = oracle.gemm_f64(packed, scale, zp, clean)
    assert rel_err(got[[0, 2]].astype(np.float64), ref) <= 1e-2
    pkg.awq_free(w)


@pytest.mark.parametrize("N,K,M", [(16, 128, 1), (272, 384, 1), (272, 640, 2), (144, 896, 5), (1040, 1152, 3),
                                   (2064, 384, 10), (128, 128, 16)])
def test_odd_group_counts_and_ragged_tiles(pkg, oracle, synth, scratch, N, K, M):
    """Odd numbers of k groups (steps with a single group), rows that do not fill the last 128-row tile, and
    more CTAs than units."""
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=N + K + M)
    x = synth.make_activations(M, K, seed=M)
    ref = oracle.gemm_f64(packed, scale, zp, x)
    y = Guarded((M, N), torch.bfloat16)
    pkg.gemm_small_w4a16(y.t, w, dev_bf16(x), M, scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and y.intact()
    assert rel_err(synth.bf16_bits_to_f32(host_bits(y.t)).astype(np.float64), ref) <= 1e-2
    pkg.awq_free(w)


def test_token_batches_on_a_wide_layer(pkg, oracle, synth, scratch):
    """in_f = 17408 with enough rows that every CTA multiplies all 136 groups, M = 7 in one launch. Sampled rows
    against fp64, and equal to M single-token calls bit for bit (the same integer sums, added in the same order)."""
    N, K, M = 20480, 17408, 7
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=9)
    x = synth.make_activations(M, K, seed=21)
    dx = dev_bf16(x)
    y = Guarded((M, N), torch.bfloat16)
    pkg.gemm_small_w4a16(y.t, w, dx, M, scratch)
    y1 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    for m in range(M):
        pkg.gemv_w4a16(y1[m], w, dx[m], scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and y.intact()
    assert torch.equal(y.t.view(torch.int16), y1.view(torch.int16))
    rows = np.random.Generator(np.random.PCG64(2)).choice(N, 96, replace=False).astype(np.int64)
    ref = oracle.gemm_f64(packed, scale, zp, x, rows=rows)
    got = synth.bf16_bits_to_f32(host_bits(y.t))[:, rows].astype(np.float64)
    assert rel_err(got, ref) <= 1e-2
    pkg.awq_free(w)
