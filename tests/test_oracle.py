"""The CPU oracle against everything that pins it (no GPU needed)."""
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# the reference checkout: W4A16_REFERENCE_DIR, else a directory named "reference" beside this repository
REFERENCE = os.environ.get("W4A16_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
REF_FIXTURES = os.path.join(REFERENCE, "tests", "fixtures", "dequant")


def test_golden_has_all_reference_tensors(golden):
    assert len(golden) == 7
    for g in golden.values():
        assert g["packed"].shape == (64, 64) and g["deq"].shape == (64, 512)


def test_oracle_unpack_matches_golden_codes(oracle, golden):
    for stem, g in golden.items():
        assert np.array_equal(oracle.unpack_q(g["packed"]), g["q"]), stem


def test_oracle_dequant_bit_exact_vs_golden(oracle, golden):
    # tests/gate_dequant.cpp:87 of the reference requires max|diff| == 0
    for stem, g in golden.items():
        got = oracle.dequant_f32(g["packed"], g["scale"], g["zp"])
        assert np.array_equal(got.view(np.uint32), g["deq"].view(np.uint32)), stem


@pytest.mark.skipif(not os.path.isdir(REF_FIXTURES), reason="reference checkout absent")
def test_golden_matches_reference_fixture_files(golden):
    for stem, g in golden.items():
        q = np.fromfile(os.path.join(REF_FIXTURES, stem + ".q8"), np.int8).reshape(64, 512)
        d = np.fromfile(os.path.join(REF_FIXTURES, stem + ".f32"), np.float32).reshape(64, 512)
        assert np.array_equal(q, g["q"]) and np.array_equal(d.view(np.uint32), g["deq"].view(np.uint32))


def test_oracle_matches_reference_header(oracle, synth):
    ref = oracle.ref_lib()
    if ref is None:
        pytest.skip("reference header wrapper was not built")
    N, K = 96, 512
    packed, scale, zp = synth.make_weights(N, K, seed=3)
    q = np.empty((N, K), np.int8)
    ref.ref_unpack_q(packed, N, K, q)
    assert np.array_equal(q, oracle.unpack_q(packed))
    z = np.empty((N, K // 128), np.int8)
    ref.ref_unpack_zp(zp, N, K // 128, z)
    assert np.array_equal(z, oracle.unpack_zp(zp, N))
    d = np.empty((N, K), np.float32)
    ref.ref_dequant_f32(packed, scale, zp, N, K, 128, d)
    assert np.array_equal(d.view(np.uint32), oracle.dequant_f32(packed, scale, zp).view(np.uint32))


def test_oracle_matches_compressed_tensors(oracle, synth):
    torch = pytest.importorskip("torch")
    helpers = pytest.importorskip("compressed_tensors.compressors.pack_quantized.helpers")
    rng = np.random.default_rng(5)
    N, K, G = 64, 256, 2
    q = rng.integers(-8, 8, size=(N, K), dtype=np.int8)
    z = rng.integers(-8, 8, size=(N, G), dtype=np.int8)
    packed = helpers.pack_to_int32(torch.from_numpy(q), 4, packed_dim=1).numpy().view(np.uint32)
    zpp = helpers.pack_to_int32(torch.from_numpy(z), 4, packed_dim=0).numpy().view(np.uint32)
    assert np.array_equal(oracle.unpack_q(packed), q)
    assert np.array_equal(oracle.unpack_zp(zpp, N), z)
    # and the synthetic packers write the same words as the library
    assert np.array_equal(synth.pack_weight((q + 8).astype(np.uint8)), packed)
    assert np.array_equal(synth.pack_zero_point((z + 8).astype(np.uint8)), zpp)


def test_bf16_rounding(oracle, synth):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    a = (rng.standard_normal(100000) * 10 ** rng.uniform(-6, 6, 100000)).astype(np.float32)
    a[:4] = [0.0, -0.0, 1.00390625, 3.3895314e38]
    want = torch.from_numpy(a).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16(a), want)
    assert np.array_equal(synth.f32_to_bf16_bits(a), want)
    assert np.array_equal(oracle.bf16_to_f32(want), synth.bf16_bits_to_f32(want))


def test_dequant_bf16_is_single_rounding(oracle, synth):
    packed, scale, zp = synth.make_weights(64, 512, seed=1)
    f = oracle.dequant_f32(packed, scale, zp)
    assert np.array_equal(oracle.dequant_bf16(packed, scale, zp), oracle.f32_to_bf16(f))
    part = oracle.dequant_bf16(packed, scale, zp, row0=32, nrows=16)
    assert np.array_equal(part, oracle.f32_to_bf16(f[32:48]))


def test_gemm_f64_equals_numpy(oracle, synth):
    N, K, M = 128, 640, 5
    packed, scale, zp = synth.make_weights(N, K, seed=2)
    x = synth.make_activations(M, K, seed=2)
    w = oracle.dequant_f32(packed, scale, zp).astype(np.float64)
    want = synth.bf16_bits_to_f32(x).astype(np.float64) @ w.T
    got = oracle.gemm_f64(packed, scale, zp, x)
    assert np.allclose(got, want, rtol=1e-12, atol=1e-12)
    rows = np.array([3, 77, 127], np.int64)
    assert np.array_equal(oracle.gemm_f64(packed, scale, zp, x, rows=rows), got[:, rows])
    got32 = oracle.gemm_f32(packed, scale, zp, x)
    assert np.max(np.abs(got32 - want)) / np.max(np.abs(want)) < 1e-5


def test_argmax_ties_take_lowest_index(oracle, synth):
    logits = synth.f32_to_bf16_bits(np.array([[1.0, 3.0, 3.0, -2.0], [-5.0, -5.0, -7.0, -5.0]],
                                             np.float32))
    assert list(oracle.argmax_bf16(logits)) == [1, 0]


def test_lm_head_argmax_consistent(oracle, synth):
    N, K, M = 512, 256, 3
    packed, scale, zp = synth.make_weights(N, K, seed=4)
    x = synth.make_activations(M, K, seed=4)
    ids, gaps, logits = oracle.lm_head_argmax(packed, scale, zp, x, want_logits=True)
    y = oracle.gemm_f64(packed, scale, zp, x)
    assert np.array_equal(logits, oracle.f32_to_bf16(y.astype(np.float32)))
    assert np.array_equal(ids, oracle.argmax_bf16(logits))
    assert np.all(gaps >= 0)


def test_quantizer_round_trip(oracle, synth):
    # src/model/model.cu:140-172 of the reference: min/max asymmetric int4, error <= scale/2 (+bf16 scale rounding)
    rng = np.random.default_rng(9)
    src = synth.f32_to_bf16_bits(rng.standard_normal((16, 256)).astype(np.float32))
    packed, scale, zp = oracle.quant_i4(src, 128)
    deq = oracle.dequant_f32(packed, scale, zp)
    s = np.repeat(synth.bf16_bits_to_f32(scale), 128, axis=1)
    assert np.all(np.abs(deq - synth.bf16_bits_to_f32(src)) <= 0.5 * s * 1.02 + 16 * s * 2 ** -8)
    q = oracle.unpack_q(packed)
    assert q.min() == -8 and q.max() == 7


def test_w8_quantizer_properties(oracle, synth):
    # src/kernels/gemv_w4a16.cu:479-499 of the reference: symmetric int8 per group of 128
    rng = np.random.default_rng(10)
    v = rng.standard_normal((32, 384)).astype(np.float32) * 0.03
    v[3, 128:256] = 0.0           # an all-zero group: scale 0, codes 0
    src = synth.f32_to_bf16_bits(v)
    q, scale = oracle.quant_w8(src, 128)
    f = synth.bf16_bits_to_f32(src)
    assert q.min() >= -127 and q.max() <= 127
    assert np.all(q[3, 128:256] == 0) and scale[3, 1] == 0
    g = f.reshape(32, 3, 128)
    mx = np.abs(g).max(axis=2)
    # the largest element of every non-zero group maps to +-127, the scale is bf16(max/127)
    assert np.all(np.abs(q.reshape(32, 3, 128)).max(axis=2)[mx > 0] == 127)
    assert np.array_equal(scale, synth.f32_to_bf16_bits((mx / np.float32(127.0)).astype(np.float32)))
    # codes are rn(v * (127/max)) in fp32, recomputed here with numpy's fp32 arithmetic
    inv = np.where(mx > 0, np.float32(127.0) / np.where(mx > 0, mx, 1).astype(np.float32), np.float32(0)).astype(np.float32)
    want = np.clip(np.rint(g * inv[:, :, None]), -127, 127).astype(np.int8).reshape(32, 384)
    assert np.array_equal(q, want)
    # round trip: |q*s - v| <= s/2 plus the bf16 rounding of the scale
    s = np.repeat(synth.bf16_bits_to_f32(scale), 128, axis=1)
    assert np.all(np.abs(q * s - f) <= 0.5 * s * 1.01 + 127 * s * 2 ** -8)


def test_w8_gemm_f64_equals_numpy(oracle, synth):
    src = synth.make_activations(96, 512, seed=12, sigma=0.05)
    q, scale = oracle.quant_w8(src)
    x = synth.make_activations(4, 512, seed=13)
    w = q.astype(np.float64) * np.repeat(synth.bf16_bits_to_f32(scale).astype(np.float64), 128, axis=1)
    want = synth.bf16_bits_to_f32(x).astype(np.float64) @ w.T
    got = oracle.gemm_w8_f64(q, scale, x)
    assert np.allclose(got, want, rtol=1e-12, atol=1e-12)
    rows = np.array([0, 50, 95], np.int64)
    assert np.array_equal(oracle.gemm_w8_f64(q, scale, x, rows=rows), got[:, rows])
    ids, gaps, logits = oracle.argmax_with_gaps(got)
    assert np.array_equal(ids, oracle.argmax_bf16(logits)) and np.all(gaps >= 0)


def test_elementwise_neighbours_match_torch(oracle, synth):
    """rmsnorm / residual_add / swiglu (src/kernels/elementwise.cu:8-49 of the reference) against torch fp32."""
    torch = pytest.importorskip("torch")

    def bits(t):
        return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)

    x = synth.make_activations(4, 5120, seed=21)
    w = synth.make_activations(1, 5120, seed=22, sigma=0.1)[0]
    xf, wf = torch.from_numpy(synth.bf16_bits_to_f32(x)), torch.from_numpy(synth.bf16_bits_to_f32(w))
    want = bits(xf * torch.rsqrt((xf * xf).mean(1, keepdim=True) + 1e-6) * (1 + wf))
    got = oracle.rmsnorm(x, w, 1e-6)
    # the summation order differs from torch's: at most a unit in the last place of a few outputs
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.01
    h = synth.make_activations(2, 256, seed=23)
    y = synth.make_activations(2, 256, seed=24)
    want = bits(torch.from_numpy(synth.bf16_bits_to_f32(h)) + torch.from_numpy(synth.bf16_bits_to_f32(y)))
    assert np.array_equal(oracle.residual_add(h, y), want)
    f = synth.make_activations(3, 2048, seed=25, sigma=2.0)
    ff = torch.from_numpy(synth.bf16_bits_to_f32(f))
    g, u = ff[:, :1024], ff[:, 1024:]
    want = bits((g / (1 + torch.exp(-g))) * u)
    d = np.abs(oracle.swiglu(f).astype(np.int32) - want.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 0.01


def test_synthetic_config_totals(synth):
    shapes = synth.decode_pass_shapes()
    assert len(shapes) == 256
    weights = sum(N * K // 2 + N * (K // 128) * 2 + N * (K // 128) // 2 for _, N, K in shapes)
    acts = sum(2 * K + 2 * N for _, N, K in shapes)
    assert weights == 12_638_617_600 and acts == 12_124_160
    assert synth.algorithmic_bytes(17408, 5120) == 46_350_336
    assert synth.algorithmic_bytes(248320, 5120, out_bytes=4) == 660_541_444
