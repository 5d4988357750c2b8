"""The cross-rank completion flags and the sharded entry points, as far as ONE GPU can show them.

Ranks are emulated one after the other on the same device (never as kernels that wait for each
other): every "rank" has its own output buffer and flag block, a launch of rank r stores its
column slice into all of them and raises flag r everywhere. What needs kernels of different ranks
to run at the same time (the in-kernel pair exchange of the vocab-sharded lm_head with more than
one rank) is covered by the multi-GPU worker.

The wait that runs out: a communicator of two ranks of which only one ever signals. The bounded
wait gives up after about a second, the status word reads W4A16_ETIMEOUT, nothing hangs or faults.
"""
import numpy as np
import pytest
import torch

from gpu_util import dev_bf16, host_bits

pytestmark = pytest.mark.gpu


def _blocks(n):
    t = torch.zeros((n, 64), dtype=torch.int32, device="cuda")  # 256 bytes per rank
    return t, [t[i].data_ptr() for i in range(n)]


def _shards(pkg, synth, sharding, N, K, R, seed):
    packed, scale, zp = synth.make_weights(N, K, seed=seed)
    full = pkg.weights_from_numpy(packed, scale, zp)
    parts = []
    for r in range(R):
        sp, ss, sz, row0 = sharding.shard_on_disk(packed, scale, zp, R, r)
        parts.append((pkg.weights_from_numpy(sp, ss, sz), row0))
    return (packed, scale, zp), full, parts


@pytest.fixture(scope="module")
def sharding():
    import importlib
    return importlib.import_module("qwen38-3090-cuda-server_b200.sharding")


@pytest.mark.parametrize("M", [1, 9])
def test_gather_with_flags_two_emulated_ranks(pkg, synth, sharding, M):
    N, K, R = 4096, 1024, 2
    _, full, parts = _shards(pkg, synth, sharding, N, K, R, seed=61)
    s = pkg.gemv_scratch_alloc(K, N, 128, 16)
    x = dev_bf16(synth.make_activations(M, K, seed=61))
    ys = [torch.zeros((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    flags, ptrs = _blocks(R)
    torch.cuda.synchronize()
    comms = [pkg.make_comm(ptrs, r) for r in range(R)]
    for r in range(R):
        pkg.gemm_skinny_gather([y.data_ptr() for y in ys], comms[r], N, parts[r][1], parts[r][0], x, M, s)
    for r in range(R):
        pkg.wait_gather(comms[r])
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    f = flags.cpu().numpy()
    assert (f[:, :R] == 65536).all() and (f[:, 16] == 1).all()   # one launch: 65536 per rank's counter, seq 1
    # the slices are what the same shard gives on its own, bit for bit, in every rank's copy
    for r in range(R):
        w, row0 = parts[r]
        yr = torch.empty((M, N // R), dtype=torch.bfloat16, device="cuda")
        pkg.gemm_small_w4a16(yr, w, x, M, s)
        for y in ys:
            assert torch.equal(y[:, row0:row0 + N // R].view(torch.int16), yr.view(torch.int16))
    # a second round: the sequence numbers move on together
    for r in range(R):
        pkg.gemm_skinny_gather([y.data_ptr() for y in ys], comms[r], N, parts[r][1], parts[r][0], x, M, s)
    for r in range(R):
        pkg.wait_gather(comms[r])
    assert pkg.device_status() == 0
    assert (flags.cpu().numpy()[:, :R] == 2 * 65536).all()
    pkg.gemv_scratch_free(s)
    pkg.awq_free(full)
    for w, _ in parts:
        pkg.awq_free(w)


@pytest.mark.parametrize("M", [1, 8])
def test_chained_layers_wait_for_the_previous_gather(pkg, oracle, synth, M):
    """One rank: layer B reads the output of layer A and waits for A's flag in its own prologue (the converter
    warps at M = 1, the pre-pass kernel otherwise) instead of a host barrier; also inside a CUDA graph."""
    K, N1, N2 = 1024, 2048, 512
    wa = synth.make_weights(N1, K, seed=71)
    wb = synth.make_weights(N2, N1, seed=72)
    A, B = pkg.weights_from_numpy(*wa), pkg.weights_from_numpy(*wb)
    s = pkg.gemv_scratch_alloc(N1, N1, 128, 16)
    x = dev_bf16(synth.make_activations(M, K, seed=71, sigma=0.05))
    y1 = torch.zeros((M, N1), dtype=torch.bfloat16, device="cuda")
    y2 = torch.zeros((M, N2), dtype=torch.bfloat16, device="cuda")
    flags, ptrs = _blocks(1)
    torch.cuda.synchronize()
    comm = pkg.make_comm(ptrs, 0)

    def chain():
        pkg.gemm_skinny_gather([y1.data_ptr()], comm, N1, 0, A, x, M, s)
        pkg.gemm_skinny_gather([y2.data_ptr()], comm, N2, 0, B, y1, M, s, wait_prev=True)

    chain()
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    r1 = torch.empty_like(y1)
    r2 = torch.empty_like(y2)
    pkg.gemm_small_w4a16(r1, A, x, M, s)
    pkg.gemm_small_w4a16(r2, B, r1, M, s)
    assert torch.equal(y1.view(torch.int16), r1.view(torch.int16))
    assert torch.equal(y2.view(torch.int16), r2.view(torch.int16))
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(st):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=st):
            pkg.gemm_skinny_gather([y1.data_ptr()], comm, N1, 0, A, x, M, s, stream=st)
            pkg.gemm_skinny_gather([y2.data_ptr()], comm, N2, 0, B, y1, M, s, wait_prev=True, stream=st)
        y2.zero_()
        for _ in range(3):  # replays: the sequence number lives in device memory, so it keeps counting
            g.replay()
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    assert torch.equal(y2.view(torch.int16), r2.view(torch.int16))
    assert int(flags[0, 16].item()) == 2 + 6
    pkg.gemv_scratch_free(s)
    pkg.awq_free(A)
    pkg.awq_free(B)


def test_wait_for_a_rank_that_never_signals_runs_out(pkg, synth):
    N, K = 512, 256
    w = pkg.weights_from_numpy(*synth.make_weights(N // 2, K, seed=81))
    s = pkg.gemv_scratch_alloc(K, N, 128, 1)
    x = dev_bf16(synth.make_activations(1, K, seed=81)[0])
    ys = [torch.zeros(N, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    flags, ptrs = _blocks(2)
    torch.cuda.synchronize()
    comm0 = pkg.make_comm(ptrs, 0)
    pkg.gemm_skinny_gather([y.data_ptr() for y in ys], comm0, N, 0, w, x, 1, s)  # rank 0 signals; "rank 1" never runs
    pkg.wait_gather(comm0)
    assert pkg.device_status() == -4      # the bounded wait for rank 1's flag gave up; the kernel returned
    pkg.device_status_clear()
    assert pkg.device_status() == 0
    y = torch.empty(N // 2, dtype=torch.bfloat16, device="cuda")
    pkg.gemv_w4a16(y, w, x, s)            # the context is fine
    assert torch.equal(y.view(torch.int16), ys[0][: N // 2].view(torch.int16))
    assert pkg.device_status() == 0
    pkg.gemv_scratch_free(s)
    pkg.awq_free(w)


@pytest.mark.parametrize("M", [1, 9])
def test_sharded_lm_head_single_rank_equals_unsharded(pkg, oracle, synth, M):
    N, K = 4096, 512
    packed, scale, zp = synth.make_weights(N, K, seed=91)
    w = pkg.weights_from_numpy(packed, scale, zp)
    s = pkg.gemv_scratch_alloc(K, N, 128, 16)
    x = dev_bf16(synth.make_activations(M, K, seed=91))
    flags, ptrs = _blocks(1)
    table = torch.zeros((1, 16, 2), dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    comm = pkg.make_comm(ptrs, 0)
    ids = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    pkg.lm_head_argmax_sharded(ids, [table.data_ptr()], comm, 0, w, x, M, s)
    want = torch.full((M,), -1, dtype=torch.int32, device="cuda")
    pkg.lm_head_argmax(want, w, x, M, s)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    assert torch.equal(ids, want)
    assert np.array_equal(table[0, :M, 1].cpu().numpy(), want.cpu().numpy())
    pkg.gemv_scratch_free(s)
    pkg.awq_free(w)


def test_sharded_prefill_two_emulated_ranks(pkg, synth, sharding):
    N, K, M, R = 512, 512, 300, 2
    _, full, parts = _shards(pkg, synth, sharding, N, K, R, seed=95)
    x = dev_bf16(synth.make_activations(M, K, seed=95))
    ws = pkg.gemm_workspace_alloc(4096)
    cs = [torch.zeros((M, N), dtype=torch.bfloat16, device="cuda") for _ in range(R)]
    flags, ptrs = _blocks(R)
    torch.cuda.synchronize()
    comms = [pkg.make_comm(ptrs, r) for r in range(R)]
    for r in range(R):
        pkg.gemm_w4a16_sharded([c.data_ptr() for c in cs], comms[r], N, parts[r][1], parts[r][0], x, M, ws)
    for r in range(R):
        pkg.wait_gather(comms[r])
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    want = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_w4a16(want, full, x, M, ws)
    torch.cuda.synchronize()
    for c in cs:
        assert torch.equal(c.view(torch.int16), want.view(torch.int16))
    pkg.gemm_workspace_free(ws)
    pkg.awq_free(full)
    for w, _ in parts:
        pkg.awq_free(w)


@pytest.mark.parametrize("M", [1, 8])
def test_gather_free_mlp_two_emulated_ranks(pkg, oracle, synth, sharding, M):
    """gate|up row-sharded with the SwiGLU epilogue (no exchange) -> K-sharded down -> fp32 partials into every
    rank's buffer -> reduce in rank order + residual add; against the unsharded fused chain."""
    from gpu_util import rel_err
    H, I, R = 1024, 2048, 2
    gate, up = synth.make_weights(I, H, seed=101), synth.make_weights(I, H, seed=102)
    down = synth.make_weights(H, I, seed=103)
    h0 = synth.make_activations(M, H, seed=104)
    x = dev_bf16(synth.make_activations(M, H, seed=105, sigma=0.5))
    s = pkg.gemv_scratch_alloc(I, 2 * I, 128, 16)

    def dev(a, dt=np.int32):
        return torch.from_numpy(np.ascontiguousarray(a).view(dt)).cuda()

    def swiglu_container(g, u, inter):
        w = pkg.awq_alloc_fused(2 * inter, H)
        for off, (pk, sc, zp) in ((0, g), (inter, u)):
            pkg.awq_repack_into_swiglu(w, off, dev(pk), dev(sc, np.int16), dev(zp), inter)
        return w

    # one GPU, fused: two launches
    full = swiglu_container(gate, up, I)
    wd = pkg.weights_from_numpy(*down)
    act = torch.empty((M, I), dtype=torch.bfloat16, device="cuda")
    pkg.linear_fused(act, full, x, M, s, epilogue=pkg.EPILOGUE_SWIGLU)
    want = dev_bf16(h0).clone()
    pkg.linear_fused(want, wd, act, M, s, epilogue=pkg.EPILOGUE_RESIDUAL)
    # two emulated ranks
    flags, ptrs = _blocks(R)
    bufs = [torch.zeros((R, M, H), dtype=torch.float32, device="cuda") for _ in range(R)]
    hs = [dev_bf16(h0).clone() for _ in range(R)]
    torch.cuda.synchronize()
    comms = [pkg.make_comm(ptrs, r) for r in range(R)]
    keep = []
    for r in range(R):
        gs = sharding.shard_on_disk(*gate, R, r)[:3]
        us = sharding.shard_on_disk(*up, R, r)[:3]
        w_r = swiglu_container(gs, us, I // R)
        wd_r = pkg.weights_from_numpy(*sharding.shard_k_on_disk(*down, R, r)[:3])
        act_r = torch.empty((M, I // R), dtype=torch.bfloat16, device="cuda")
        pkg.linear_fused(act_r, w_r, x, M, s, epilogue=pkg.EPILOGUE_SWIGLU)
        pkg.gemm_skinny_partial([b.data_ptr() for b in bufs], comms[r], wd_r, act_r, M, s)
        keep += [w_r, wd_r, act_r]
    for r in range(R):
        pkg.reduce_partials(hs[r], bufs[r], comms[r], M, H, residual=True)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    assert torch.equal(hs[0].view(torch.int16), hs[1].view(torch.int16)), "the ranks disagree"
    got = hs[0].float().cpu().numpy().astype(np.float64)
    ref = want.float().cpu().numpy().astype(np.float64)
    assert rel_err(got, ref) <= 1e-2
    d = np.abs(host_bits(hs[0]).astype(np.int32) - host_bits(want).astype(np.int32))
    assert (d > 2).mean() < 0.01    # the same arithmetic up to the order of fp32 sums
    pkg.gemv_scratch_free(s)
    for w in (full, wd) + tuple(k for k in keep if hasattr(k, "qweight")):
        pkg.awq_free(w)
