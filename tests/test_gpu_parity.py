"""GPU parity tests: the CUDA path through the C ABI against the CPU oracle.

Tolerances (from the benchmark's statement of the path):
  dequantised weights ........ bit-exact
  GEMV / skinny outputs ...... max|y-ref| / max|ref| <= 1e-2 for bf16 outputs (the
                               observed error is the bf16 rounding of the output, ~2e-3),
                               and every element within 1e-2*|ref| + 1 bf16 ulp + 1e-2*max|ref|*2^-8;
                               fp32 outputs: <= 1e-4 (the reference's own gate uses 1e-5 on its
                               fp32 CUDA-core path; tensor-core fp32 accumulation is given 10x)
  lm_head argmax ids ......... identical, unless the oracle's own top-2 gap is 0 bf16 ulp
"""
import numpy as np
import pytest
import torch

from gpu_util import Guarded, bf16_ulp, dev_bf16, host_bits, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def scratch(pkg):
    s = pkg.gemv_scratch_alloc(17408, 248320, 128, 16)
    yield s
    pkg.gemv_scratch_free(s)


def _weights(pkg, synth, N, K, seed):
    packed, scale, zp = synth.make_weights(N, K, seed=seed)
    return (packed, scale, zp), pkg.weights_from_numpy(packed, scale, zp)


# ----------------------------------------------------------------- dequant (bit-exact anchor)
def test_dequant_rows_golden_bit_exact(pkg, oracle, golden):
    """Real checkpoint tiles (the reference's gate_dequant fixtures) through repack + dequant_rows."""
    for stem, g in golden.items():
        w = pkg.weights_from_numpy(g["packed"], g["scale"], g["zp"])
        dst = Guarded((64, 512), torch.bfloat16)
        pkg.w4a16_dequant_rows(dst.t, w, 0, 64)
        torch.cuda.synchronize()
        want = oracle.f32_to_bf16(g["deq"])
        assert np.array_equal(host_bits(dst.t), want), stem
        assert dst.intact()
        pkg.awq_free(w)


@pytest.mark.parametrize("N,K", [(32, 128), (48, 640), (256, 5120), (1040, 1024)])
def test_dequant_rows_synthetic_bit_exact(pkg, oracle, synth, N, K):
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=11)
    want = oracle.dequant_bf16(packed, scale, zp)
    dst = torch.empty((N, K), dtype=torch.bfloat16, device="cuda")
    pkg.w4a16_dequant_rows(dst, w, 0, N)
    assert np.array_equal(host_bits(dst), want)
    if N >= 48:  # a row window
        part = torch.empty((16, K), dtype=torch.bfloat16, device="cuda")
        pkg.w4a16_dequant_rows(part, w, 23, 16)
        assert np.array_equal(host_bits(part), want[23:39])
    pkg.awq_free(w)


def test_repack_into_concatenates_fused_projections(pkg, oracle, synth):
    """awq_alloc_fused + awq_repack_into at row offsets (q|k|v, gate|up fusing in the reference)."""
    K = 512
    parts = [synth.make_weights(n, K, seed=20 + i) for i, n in enumerate((64, 32, 160))]
    w = pkg.awq_alloc_fused(256, K)
    off = 0
    for packed, scale, zp in parts:
        pkg.awq_repack_into(w, off, torch.from_numpy(packed.view(np.int32)).cuda(),
                            torch.from_numpy(scale.view(np.int16)).cuda(),
                            torch.from_numpy(zp.view(np.int32)).cuda())
        off += packed.shape[0]
    dst = torch.empty((256, K), dtype=torch.bfloat16, device="cuda")
    pkg.w4a16_dequant_rows(dst, w, 0, 256)
    want = np.concatenate([oracle.dequant_bf16(*p) for p in parts])
    assert np.array_equal(host_bits(dst), want)
    pkg.awq_free(w)


# ----------------------------------------------------------------- GEMV / skinny
def _check_bf16(got_bits, ref, synth):
    got = synth.bf16_bits_to_f32(got_bits).astype(np.float64)
    r = rel_err(got, ref)
    assert r <= 1e-2, f"relative error {r:.3e}"
    tol = 1e-2 * np.abs(ref) + bf16_ulp(ref) + 1e-2 * np.max(np.abs(ref)) * 2.0 ** -8
    bad = np.abs(got - ref) > tol
    assert not bad.any(), f"{bad.sum()} elements outside the per-element tolerance"
    return r


GEMV_SHAPES = [(32, 128), (16, 256), (128, 17408), (208, 1024), (2048, 5120), (17408, 5120),
               (5120, 17408), (5120, 6144)]


@pytest.mark.parametrize("N,K", GEMV_SHAPES)
def test_gemv_matches_fp64_oracle(pkg, oracle, synth, scratch, N, K):
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=N + K)
    x = synth.make_activations(1, K, seed=N)
    ref = oracle.gemm_f64(packed, scale, zp, x)[0]
    dx = dev_bf16(x[0])
    y32 = Guarded((N,), torch.float32)
    pkg.gemv_w4a16_f32(y32.t, w, dx, scratch)
    y16 = Guarded((N,), torch.bfloat16)
    pkg.gemv_w4a16(y16.t, w, dx, scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    assert y32.intact() and y16.intact()
    r32 = rel_err(y32.t.cpu().numpy(), ref)
    assert r32 <= 1e-4, f"fp32 output relative error {r32:.3e}"
    _check_bf16(host_bits(y16.t), ref, synth)
    # bf16 output is exactly the rounding of the fp32 output
    assert np.array_equal(host_bits(y16.t), oracle.f32_to_bf16(y32.t.cpu().numpy()))
    pkg.awq_free(w)


@pytest.mark.parametrize("M", list(range(1, 17)))
def test_skinny_every_m(pkg, oracle, synth, scratch, M):
    N, K = 1056, 2048
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=100 + M)
    x = synth.make_activations(M, K, seed=M)
    ref = oracle.gemm_f64(packed, scale, zp, x)
    y = Guarded((M, N), torch.bfloat16)
    pkg.gemm_small_w4a16(y.t, w, dev_bf16(x), M, scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and y.intact()
    _check_bf16(host_bits(y.t), ref, synth)
    pkg.awq_free(w)


@pytest.mark.parametrize("N,K,M", [(34816, 5120, 9), (5120, 17408, 16), (8192, 5120, 8), (16384, 5120, 16),
                                   (31040, 5120, 9)])
def test_skinny_model_shapes(pkg, oracle, synth, scratch, N, K, M):
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=7)
    x = synth.make_activations(M, K, seed=3)
    rows = (np.arange(512, dtype=np.int64) * 7919) % N  # sampled rows, as tests/gate_gemv.cu:102 does
    rows[:3] = [0, N - 1, N // 2]
    ref = oracle.gemm_f64(packed, scale, zp, x, rows=rows)
    y = Guarded((M, N), torch.bfloat16)
    pkg.gemm_mma_w4a16(y.t, w, dev_bf16(x), M, scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and y.intact()
    got = host_bits(y.t)
    _check_bf16(got[:, rows], ref, synth)
    assert np.all(np.isfinite(synth.bf16_bits_to_f32(got)))
    pkg.awq_free(w)


def _edge_activations(synth, K):
    """Rows of activations at the corners of the block fixed-point conversion (one exponent per token and
    128-k group): all zero; an outlier channel 2^13 above its group; magnitudes of 1e-20 and 1e20; a group whose largest value is an exact power of two; one non-zero per group."""
    rng = np.random.Generator(np.random.PCG64(99))
    base = rng.standard_normal((6, K)).astype(np.float32)
    base[0] = 0.0
    base[1, 5::128] *= 8192.0
    base[2] *= 1e-20
    base[3] *= 1e20
    base[4] = np.exp2(-rng.integers(0, 12, K)).astype(np.float32) * rng.choice([-1.0, 1.0], K)
    base[4, 17::128] = -4.0
    base[5] = 0.0
    base[5, 100::128] = -0.3
    return synth.f32_to_bf16_bits(base)


def test_activation_corner_cases(pkg, oracle, synth, scratch):
    """Every token is checked on its own scale (the rows differ by 40 orders of magnitude), through the
    M = 1 kernel (conversion inside the kernel) and the M = 6 kernel (conversion in the pre-pass)."""
    N, K = 384, 1024
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=77)
    x = _edge_activations(synth, K)
    M = x.shape[0]
    ref = oracle.gemm_f64(packed, scale, zp, x)
    Y = Guarded((M, N), torch.bfloat16)
    pkg.gemm_small_w4a16(Y.t, w, dev_bf16(x), M, scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and Y.intact()
    got = host_bits(Y.t)
    for m in range(M):
        y = Guarded((N,), torch.bfloat16)
        pkg.gemv_w4a16(y.t, w, dev_bf16(x[m]), scratch)
        torch.cuda.synchronize()
        assert y.intact()
        for bits in (got[m], host_bits(y.t)):
            if m == 0:
                assert not synth.bf16_bits_to_f32(bits).any()  # zero activations give exact zeros
            else:
                _check_bf16(bits, ref[m], synth)
    assert pkg.device_status() == 0
    pkg.awq_free(w)


def test_non_finite_activations_stay_in_their_token(pkg, oracle, synth, scratch):
    """An inf in one token makes that token's outputs non-finite (the reference gives inf or NaN there,
    0 * inf where a weight equals its zero point) and leaves the other tokens' outputs as they were."""
    N, K, M = 256, 512, 4
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=78)
    x = synth.make_activations(M, K, seed=78)
    clean = Guarded((M, N), torch.bfloat16)
    pkg.gemm_small_w4a16(clean.t, w, dev_bf16(x), M, scratch)
    x2 = x.copy()
    x2[2, 200] = 0x7F80  # +inf
    dirty = Guarded((M, N), torch.bfloat16)
    pkg.gemm_small_w4a16(dirty.t, w, dev_bf16(x2), M, scratch)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and dirty.intact()
    a, b = host_bits(clean.t), host_bits(dirty.t)
    for m in (0, 1, 3):
        assert np.array_equal(a[m], b[m])
    assert not np.isfinite(synth.bf16_bits_to_f32(b[2])).any()
    pkg.awq_free(w)


def test_skinny_rows_agree_with_gemv(pkg, synth, scratch):
    """Row m of the M-row product equals the GEMV of x[m] to within the reference's 2e-2 gate
    (bench/bench_verify.cu:55-75); here the two use the same kernel and k order, so bitwise."""
    N, K, M = 4096, 5120, 9
    _, w = _weights(pkg, synth, N, K, seed=5)
    x = dev_bf16(synth.make_activations(M, K, seed=5))
    Y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w4a16(Y, w, x, M, scratch)
    for m in (0, 4, 8):
        y = torch.empty((N,), dtype=torch.bfloat16, device="cuda")
        pkg.gemv_w4a16(y, w, x[m].contiguous(), scratch)
        assert torch.equal(y.view(torch.int16), Y[m].view(torch.int16))
    pkg.awq_free(w)


def test_bitwise_reproducible_and_graph_equals_eager(pkg, synth, scratch):
    """Run-to-run and eager-vs-graph results are bitwise equal (tests/gate_graph.cu:46-55)."""
    N, K, M = 5120, 17408, 9
    _, w = _weights(pkg, synth, N, K, seed=9)
    x = dev_bf16(synth.make_activations(M, K, seed=9))
    outs = []
    for _ in range(3):
        y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        pkg.gemm_small_w4a16(y, w, x, M, scratch)
        outs.append(y)
    torch.cuda.synchronize()
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(outs[0].view(torch.int16), outs[2].view(torch.int16))
    yg = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        pkg.gemm_small_w4a16(yg, w, x, M, scratch, stream=st)  # eager warm-up on the capture stream
        yg.zero_()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            pkg.gemm_small_w4a16(yg, w, x, M, scratch, stream=st)
            pkg.gemm_small_w4a16(yg, w, x, M, scratch, stream=st)
        g.replay()
    torch.cuda.synchronize()
    assert torch.equal(outs[0].view(torch.int16), yg.view(torch.int16))
    assert pkg.device_status() == 0
    pkg.awq_free(w)


def test_golden_real_weights_gemv(pkg, oracle, synth, scratch, golden):
    """GEMV on real checkpoint tiles (64 rows x 512 k from the reference's fixtures), x ~ 0.05 N(0,1)
    as in tests/gate_gemv.cu:81."""
    for i, (stem, g) in enumerate(golden.items()):
        w = pkg.weights_from_numpy(g["packed"], g["scale"], g["zp"])
        x = synth.make_activations(1, 512, seed=i, sigma=0.05)
        ref = oracle.gemm_f64(g["packed"], g["scale"], g["zp"], x)[0]
        y = torch.empty((64,), dtype=torch.float32, device="cuda")
        pkg.gemv_w4a16_f32(y, w, dev_bf16(x[0]), scratch)
        assert rel_err(y.cpu().numpy(), ref) <= 1e-4, stem
        pkg.awq_free(w)


# ----------------------------------------------------------------- lm_head + argmax
def _argmax_case(pkg, oracle, synth, scratch, N, K, M, seed, with_logits):
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=seed)
    x = synth.make_activations(M, K, seed=seed)
    want, gaps, ref_logits = oracle.lm_head_argmax(packed, scale, zp, x, want_logits=True)
    ids = Guarded((M,), torch.int32)
    logits = Guarded((M, N), torch.bfloat16) if with_logits else None
    pairs = torch.zeros((M, 2), dtype=torch.int32, device="cuda")
    pkg.lm_head_argmax(ids.t, w, dev_bf16(x), M, scratch, logits=logits.t if logits else None, pairs=pairs)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and ids.intact()
    got = ids.t.cpu().numpy()
    ties = 0
    for m in range(M):
        if got[m] != want[m]:
            # a different id is acceptable only when the oracle's own two bf16 logits are EQUAL (0 ulp apart:
            # a true tie, where fp32-vs-fp64 accumulation may round the two candidates differently)
            lg = synth.bf16_bits_to_f32(ref_logits[m])
            a, b = float(lg[want[m]]), float(lg[got[m]])
            assert a == b, (f"row {m}: id {got[m]} vs oracle {want[m]}, logits {b} vs {a}: "
                            f"{abs(a - b) / bf16_ulp(a)} bf16 ulp apart (top-2 gap {gaps[m]})")
            ties += 1
    print(f"lm_head argmax N={N} M={M}: {ties} of {M} rows used the tie allowance")
    assert np.array_equal(pairs[:, 1].cpu().numpy(), got)
    if logits is not None:
        assert logits.intact()
        lb = host_bits(logits.t)
        # the ids must be the argmax of the logits the kernel itself wrote
        assert np.array_equal(oracle.argmax_bf16(lb), got)
        _check_bf16(lb, oracle.gemm_f64(packed, scale, zp, x), synth)
    pkg.awq_free(w)
    return int((got != want).sum())


@pytest.mark.parametrize("N,K,M", [(512, 256, 1), (4096, 1024, 9), (31040, 5120, 9), (1200 * 16, 512, 16)])
def test_lm_head_argmax_small(pkg, oracle, synth, scratch, N, K, M):
    _argmax_case(pkg, oracle, synth, scratch, N, K, M, seed=N % 97, with_logits=True)


@pytest.mark.parametrize("M", [1, 9])
def test_lm_head_argmax_full_vocab(pkg, oracle, synth, scratch, M):
    _argmax_case(pkg, oracle, synth, scratch, 248320, 5120, M, seed=0, with_logits=(M == 1))


def test_lm_head_argmax_ties_take_lowest_index(pkg, synth, scratch):
    """Two identical weight rows give identical logits: the lower row index must win."""
    N, K = 2048, 256
    packed, scale, zp = synth.make_weights(N, K, seed=1)
    x = synth.make_activations(1, K, seed=1)
    from oracle import oracle as o
    ids0, _, _ = o.lm_head_argmax(packed, scale, zp, x)
    top = int(ids0[0])
    dup = (top + 777) % N if (top + 777) % N > top else top // 2
    lo, hi = min(top, dup), max(top, dup)
    # copy row `top` (codes, scales and zero-point nibble) into row `dup`
    packed[dup] = packed[top]
    scale[dup] = scale[top]
    znib = (zp[top // 8] >> np.uint32(4 * (top % 8))) & np.uint32(0xF)
    zp[dup // 8] = (zp[dup // 8] & ~(np.uint32(0xF) << np.uint32(4 * (dup % 8)))) | (znib << np.uint32(4 * (dup % 8)))
    want, _, _ = o.lm_head_argmax(packed, scale, zp, x)
    assert want[0] == lo
    w = pkg.weights_from_numpy(packed, scale, zp)
    ids = torch.zeros(1, dtype=torch.int32, device="cuda")
    pkg.lm_head_argmax(ids, w, dev_bf16(x), 1, scratch)
    assert int(ids.item()) == lo and hi != lo
    pkg.awq_free(w)


def test_quantised_lm_head_through_the_boundary(pkg, oracle, synth, scratch):
    """The lm_head producer path of the reference (src/model/model.cu:140-194): a bf16 matrix is quantised to
    asymmetric int4 in the on-disk packing, handed to awq_repack_into, and multiplied with the argmax fused."""
    rows, cols, M = 4096, 1024, 9
    src = synth.make_activations(rows, cols, seed=51, sigma=0.02)
    packed, scale, zp = oracle.quant_i4(src, 128)
    w = pkg.awq_alloc_fused(rows, cols)
    pkg.awq_repack_into(w, 0, torch.from_numpy(packed.view(np.int32)).cuda(),
                        torch.from_numpy(scale.view(np.int16)).cuda(), torch.from_numpy(zp.view(np.int32)).cuda())
    deq = torch.empty((rows, cols), dtype=torch.bfloat16, device="cuda")
    pkg.w4a16_dequant_rows(deq, w, 0, rows)
    assert np.array_equal(host_bits(deq), oracle.dequant_bf16(packed, scale, zp))
    x = synth.make_activations(M, cols, seed=52)
    want, gaps, ref_logits = oracle.lm_head_argmax(packed, scale, zp, x, want_logits=True)
    ids = torch.zeros(M, dtype=torch.int32, device="cuda")
    logits = torch.empty((M, rows), dtype=torch.bfloat16, device="cuda")
    pkg.lm_head_argmax(ids, w, dev_bf16(x), M, scratch, logits=logits)
    torch.cuda.synchronize()
    got = ids.cpu().numpy()
    lf = synth.bf16_bits_to_f32(ref_logits)
    for m in range(M):
        assert got[m] == want[m] or lf[m, got[m]] == lf[m, want[m]], (m, got[m], want[m], gaps[m])
    _check_bf16(host_bits(logits), oracle.gemm_f64(packed, scale, zp, x), synth)
    pkg.awq_free(w)


def test_sharded_argmax_pairs_reduce(pkg, oracle, synth, scratch):
    """Vocab-sharded lm_head on one GPU: each shard yields (max, global index) pairs, and the
    pair reduction gives the unsharded ids."""
    N, K, M, R = 4096, 512, 9, 4
    packed, scale, zp = synth.make_weights(N, K, seed=2)
    x = synth.make_activations(M, K, seed=2)
    want, _, _ = oracle.lm_head_argmax(packed, scale, zp, x)
    dx = dev_bf16(x)
    allpairs = torch.zeros((R, M, 2), dtype=torch.int32, device="cuda")
    for r in range(R):
        b, e = pkg.shard_rows(N, R, r)
        w = pkg.weights_from_numpy(packed[b:e], scale[b:e], zp[b // 8:e // 8])
        pkg.lm_head_argmax(None, w, dx, M, scratch, pairs=allpairs[r], row_offset=b)
        torch.cuda.synchronize()
        pkg.awq_free(w)
    ids = torch.zeros(M, dtype=torch.int32, device="cuda")
    pkg.argmax_pairs_reduce(ids, allpairs, R, M)
    assert np.array_equal(ids.cpu().numpy(), want)


# ----------------------------------------------------------------- errors (host side only)
def test_launch_argument_errors(pkg, synth, scratch):
    _, w = _weights(pkg, synth, 64, 256, seed=0)
    x = torch.zeros(17 * 256 + 8, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(17 * 64, dtype=torch.bfloat16, device="cuda")
    for M in (0, 17):
        with pytest.raises(pkg.W4A16Error) as e:
            pkg.gemm_small_w4a16(y, w, x, M, scratch)
        assert e.value.code == -1
    with pytest.raises(pkg.W4A16Error):  # misaligned activations
        pkg.gemv_w4a16(y, w, x[1:], scratch)
    small = pkg.gemv_scratch_alloc(256, 32, 128, 1)
    with pytest.raises(pkg.W4A16Error) as e:  # scratch sized for a narrower layer
        pkg.gemv_w4a16(y, w, x, small)
    assert e.value.code == -3
    pkg.gemv_scratch_free(small)
    with pytest.raises(pkg.W4A16Error):
        pkg.w4a16_dequant_rows(y, w, 60, 16)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    pkg.awq_free(w)


# ----------------------------------------------------------------- prefill GEMM
def _prefill_case(pkg, oracle, synth, N, K, M, seed):
    (packed, scale, zp), w = _weights(pkg, synth, N, K, seed=seed)
    x = synth.make_activations(M, K, seed=seed)
    ws = pkg.gemm_workspace_alloc(1 << 20)
    c = Guarded((M, N), torch.bfloat16)
    pkg.gemm_w4a16(c.t, w, dev_bf16(x), M, ws)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0 and c.intact()
    got = synth.bf16_bits_to_f32(host_bits(c.t)).astype(np.float64)
    assert np.all(np.isfinite(got))
    pkg.gemm_workspace_free(ws)
    pkg.awq_free(w)
    return (packed, scale, zp), x, got


@pytest.mark.parametrize("N,K,M", [(128, 128, 1), (128, 256, 256), (256, 512, 300), (1056, 1024, 129), (208, 384, 17)])
def test_prefill_small_full_check(pkg, oracle, synth, N, K, M):
    """Every element against the fp64 oracle; tolerance 2e-2 on max|err|/max|ref| as the reference's
    prefill gate uses for bf16 outputs (tests/gate_gemm.cu:104-105)."""
    (packed, scale, zp), x, got = _prefill_case(pkg, oracle, synth, N, K, M, seed=N + M)
    ref = oracle.gemm_f64(packed, scale, zp, x)
    r = rel_err(got, ref)
    assert r <= 2e-2, f"relative error {r:.3e}"
    # and elementwise: bf16 weights + bf16 output rounding
    tol = 2e-2 * np.abs(ref) + 4e-3 * np.max(np.abs(ref))
    assert not (np.abs(got - ref) > tol).any()


def test_prefill_matches_dequant_then_matmul(pkg, oracle, synth):
    """The fused kernel multiplies exactly the bf16 weights w4a16_dequant_rows produces: compare with a
    float64 matmul on the oracle's bf16-rounded weights (tighter than the fp64 path: 1e-2 -> 6e-3, the
    bf16 rounding of the output)."""
    N, K, M = 512, 1024, 96
    (packed, scale, zp), x, got = _prefill_case(pkg, oracle, synth, N, K, M, seed=77)
    wb = synth.bf16_bits_to_f32(oracle.dequant_bf16(packed, scale, zp)).astype(np.float64)
    ref = synth.bf16_bits_to_f32(x).astype(np.float64) @ wb.T
    assert rel_err(got, ref) <= 6e-3


@pytest.mark.parametrize("N,K", [(34816, 5120), (5120, 17408)])
def test_prefill_model_shapes_sampled(pkg, oracle, synth, N, K):
    """M = 4096 on the model's MLP shapes, 64 sampled (m, n) against fp64 (tests/gate_gemm.cu:78-90)."""
    M = 4096
    (packed, scale, zp), x, got = _prefill_case(pkg, oracle, synth, N, K, M, seed=5)
    rng = np.random.default_rng(99)
    rows = np.unique(rng.integers(0, N, 64)).astype(np.int64)
    ms = rng.integers(0, M, 64)
    ref = oracle.gemm_f64(packed, scale, zp, x[ms], rows=rows)
    r = rel_err(got[np.ix_(ms, rows)], ref)
    assert r <= 2e-2, f"relative error {r:.3e}"
