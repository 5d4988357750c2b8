"""A linear layer with its elementwise neighbours fused in (RMSNorm in front, SwiGLU or the residual add
behind), through the C ABI against the unfused path and the CPU oracle.

The unfused chain of the reference: rmsnorm -> linear -> swiglu -> linear -> residual_add
(src/model/model.cu:774-785; src/kernels/elementwise.cu:8-49). The fused kernels round at the same places
(bf16 after the norm, bf16 after every linear, bf16 after SwiGLU and after the residual add), so:
  * residual epilogue: bit-exact against "unfused GPU linear, then the oracle's residual_add";
  * SwiGLU epilogue: against "unfused GPU linear, then the oracle's swiglu", a few bf16 ulps apart at most
    (the device's exp differs from the host's in the last place, and the interleaved weight container
    sums its K ranges in a different split), and within 2e-2 of the fp64 chain;
  * RMSNorm prologue: the normalised activations within 1 bf16 ulp of the oracle's (summation order), the
    layer output within the 1e-2 bound of the bf16 GEMV tests against the fp64 chain.
"""
import numpy as np
import pytest
import torch

from gpu_util import dev_bf16, host_bits, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def scratch(pkg):
    s = pkg.gemv_scratch_alloc(17408, 40960, 128, 16)
    yield s
    pkg.gemv_scratch_free(s)


def _dev(a, dt=np.int32):
    return torch.from_numpy(np.ascontiguousarray(a).view(dt)).cuda()


def _ulps(a, b):
    """distance of two bf16 bit arrays in units in the last place (same sign assumed where it matters)."""
    def key(v):
        v = v.astype(np.int32)
        return np.where(v & 0x8000, 0x8000 - (v & 0x7FFF), 0x8000 + v)
    return np.abs(key(a) - key(b))


@pytest.mark.parametrize("I,K,M", [(1024, 512, 1), (1024, 512, 9), (17408, 5120, 1), (4352, 5120, 16), (1040, 1024, 5)])
def test_swiglu_epilogue(pkg, oracle, synth, scratch, I, K, M):
    gate = synth.make_weights(I, K, seed=I + 1)
    up = synth.make_weights(I, K, seed=I + 2)
    # the unfused container: [gate | up] along the rows, as the reference fuses them
    plain = pkg.awq_alloc_fused(2 * I, K)
    fused = pkg.awq_alloc_fused(2 * I, K)
    for off, (pk, sc, zp) in ((0, gate), (I, up)):
        pkg.awq_repack_into(plain, off, _dev(pk), _dev(sc, np.int16), _dev(zp))
        pkg.awq_repack_into_swiglu(fused, off, _dev(pk), _dev(sc, np.int16), _dev(zp), I)
    x = dev_bf16(synth.make_activations(M, K, seed=M))
    gu = torch.empty((M, 2 * I), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w4a16(gu, plain, x, M, scratch)
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device="cuda")
    pkg.linear_fused(out, fused, x, M, scratch, epilogue=pkg.EPILOGUE_SWIGLU)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    want = oracle.swiglu(host_bits(gu))
    got = host_bits(out)
    # The interleaved container splits its K ranges over the CTAs differently from the plain one, so a gate or
    # up sum may round to the neighbouring bf16 value before SwiGLU: a few outputs move by a couple of ulps.
    d = _ulps(got, want)
    assert d.max() <= 3, f"{(d > 3).sum()} of {d.size} outputs more than three bf16 ulp from swiglu(unfused output)"
    assert (d != 0).mean() < 0.02
    # and against the fp64 chain: fp64 gate|up -> bf16 -> swiglu, with the bound of the bf16 GEMV tests
    rows = (np.arange(128, dtype=np.int64) * 7919) % I
    xb = host_bits(x)
    g64 = oracle.gemm_f64(*gate, xb, rows=rows)
    u64 = oracle.gemm_f64(*up, xb, rows=rows)
    ref = oracle.swiglu(np.concatenate([oracle.f32_to_bf16(g64.astype(np.float32)),
                                        oracle.f32_to_bf16(u64.astype(np.float32))], axis=1))
    assert rel_err(synth.bf16_bits_to_f32(got[:, rows]), synth.bf16_bits_to_f32(ref).astype(np.float64)) <= 2e-2
    pkg.awq_free(plain)
    pkg.awq_free(fused)


@pytest.mark.parametrize("N,K,M", [(512, 1024, 1), (5120, 17408, 1), (5120, 17408, 9), (1040, 256, 16)])
def test_residual_epilogue(pkg, oracle, synth, scratch, N, K, M):
    w = pkg.weights_from_numpy(*synth.make_weights(N, K, seed=N + K))
    x = dev_bf16(synth.make_activations(M, K, seed=3))
    h0 = synth.make_activations(M, N, seed=4, sigma=5.0)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w4a16(y, w, x, M, scratch)
    h = dev_bf16(h0).clone()
    pkg.linear_fused(h, w, x, M, scratch, epilogue=pkg.EPILOGUE_RESIDUAL)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    want = oracle.residual_add(h0, host_bits(y))
    assert np.array_equal(host_bits(h), want)
    pkg.awq_free(w)


@pytest.mark.parametrize("N,K,M", [(512, 1024, 1), (16384, 5120, 1), (8192, 5120, 9), (1040, 640, 16)])
def test_rmsnorm_prologue(pkg, oracle, synth, scratch, N, K, M):
    packed, scale, zp = synth.make_weights(N, K, seed=N)
    w = pkg.weights_from_numpy(packed, scale, zp)
    x0 = synth.make_activations(M, K, seed=5, sigma=3.0)
    lnw = synth.make_activations(1, K, seed=6, sigma=0.2)[0]
    eps = 1e-6
    xn = torch.zeros((M, K), dtype=torch.bfloat16, device="cuda")
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    pkg.linear_fused(y, w, dev_bf16(x0), M, scratch, ln_weight=dev_bf16(lnw), ln_eps=eps, xn_out=xn)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    want_xn = oracle.rmsnorm(x0, lnw, eps)
    d = _ulps(host_bits(xn), want_xn)
    assert d.max() <= 1 and (d != 0).mean() < 0.01, "normalised activations differ from the oracle's rmsnorm"
    # the layer multiplies exactly the activations it reports
    y2 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w4a16(y2, w, xn, M, scratch)
    assert torch.equal(y.view(torch.int16), y2.view(torch.int16))
    rows = (np.arange(256, dtype=np.int64) * 7919) % N
    ref = oracle.gemm_f64(packed, scale, zp, want_xn, rows=rows)
    got = synth.bf16_bits_to_f32(host_bits(y))[:, rows]
    assert rel_err(got, ref) <= 1e-2
    pkg.awq_free(w)


def test_fused_mlp_block_against_the_unfused_chain(pkg, oracle, synth, scratch):
    """post_ln -> gate|up -> swiglu -> down -> residual, fused into two launches, against the five-step chain."""
    H, I, M = 1024, 2048, 8
    gate, up = synth.make_weights(I, H, seed=31), synth.make_weights(I, H, seed=32)
    down = synth.make_weights(H, I, seed=33)
    plain = pkg.awq_alloc_fused(2 * I, H)
    fused = pkg.awq_alloc_fused(2 * I, H)
    for off, (pk, sc, zp) in ((0, gate), (I, up)):
        pkg.awq_repack_into(plain, off, _dev(pk), _dev(sc, np.int16), _dev(zp))
        pkg.awq_repack_into_swiglu(fused, off, _dev(pk), _dev(sc, np.int16), _dev(zp), I)
    wd = pkg.weights_from_numpy(*down)
    h0 = synth.make_activations(M, H, seed=34, sigma=1.0)
    lnw = synth.make_activations(1, H, seed=35, sigma=0.1)[0]
    # fused: two launches
    h = dev_bf16(h0).clone()
    act = torch.empty((M, I), dtype=torch.bfloat16, device="cuda")
    pkg.linear_fused(act, fused, h, M, scratch, ln_weight=dev_bf16(lnw), ln_eps=1e-6, epilogue=pkg.EPILOGUE_SWIGLU)
    pkg.linear_fused(h, wd, act, M, scratch, epilogue=pkg.EPILOGUE_RESIDUAL)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    # unfused: oracle elementwise ops around the plain GPU linears
    h2 = dev_bf16(oracle.rmsnorm(h0, lnw, 1e-6))
    gu = torch.empty((M, 2 * I), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w4a16(gu, plain, h2, M, scratch)
    a2 = dev_bf16(oracle.swiglu(host_bits(gu)))
    y = torch.empty((M, H), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w4a16(y, wd, a2, M, scratch)
    want = synth.bf16_bits_to_f32(oracle.residual_add(h0, host_bits(y))).astype(np.float64)
    got = synth.bf16_bits_to_f32(host_bits(h)).astype(np.float64)
    assert rel_err(got, want) <= 1e-2
    for c in (plain, fused, wd):
        pkg.awq_free(c)
