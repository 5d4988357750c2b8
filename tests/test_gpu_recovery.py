"""Failure detection and recovery on the GPU, without any fault or hang.

Every device-side wait in the kernels is bounded: when one runs out, the kernel records
W4A16_ETIMEOUT in a status word and returns normally. Here a tiny self-test kernel makes exactly
such a wait run out (it waits on a barrier nobody arrives at, with a limit of a few dozen polls),
the host reads the status, clears it, resets the scratch counters and the next launches are bit
for bit what they were before. Also covered: weights allocated and repacked on a side stream."""
import numpy as np
import pytest
import torch

from gpu_util import dev_bf16, host_bits

pytestmark = pytest.mark.gpu


def test_bounded_wait_expires_and_the_library_recovers(pkg, synth):
    N, K = 5120, 2048
    packed, scale, zp = synth.make_weights(N, K, seed=31)
    w = pkg.weights_from_numpy(packed, scale, zp)
    s = pkg.gemv_scratch_alloc(K, N, 128, 1)
    x = dev_bf16(synth.make_activations(1, K, seed=31)[0])
    before = torch.empty(N, dtype=torch.bfloat16, device="cuda")
    pkg.gemv_w4a16(before, w, x, s)
    before_static = torch.empty(N, dtype=torch.bfloat16, device="cuda")
    pkg.gemv_w4a16_static(before_static, w, x)
    assert pkg.device_status() == 0

    pkg.selftest_wait_timeout(64)          # the wait gives up after 64 polls; nothing faults
    assert pkg.device_status() == -4       # W4A16_ETIMEOUT, and it is sticky:
    assert pkg.device_status() == -4
    assert "wait expired" in pkg.lib().w4a16_last_error().decode()

    # recovery: clear the word, reset the tickets of every scratch in use, carry on
    pkg.device_status_clear()
    pkg.gemv_scratch_reset(s)
    pkg.gemv_static_reset()
    assert pkg.device_status() == 0
    after = torch.empty(N, dtype=torch.bfloat16, device="cuda")
    pkg.gemv_w4a16(after, w, x, s)
    after_static = torch.empty(N, dtype=torch.bfloat16, device="cuda")
    pkg.gemv_w4a16_static(after_static, w, x)
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    assert torch.equal(after.view(torch.int16), before.view(torch.int16))
    assert torch.equal(after_static.view(torch.int16), before_static.view(torch.int16))
    assert torch.equal(after.view(torch.int16), after_static.view(torch.int16))
    pkg.gemv_scratch_free(s)
    pkg.awq_free(w)


def test_alloc_and_repack_on_a_side_stream(pkg, oracle, synth):
    """A ragged last tile (1040 rows) makes the allocation zero-fill the stream; that fill must be ordered
    with the repack on the caller's stream, whichever stream that is."""
    N, K = 1040, 1024
    packed, scale, zp = synth.make_weights(N, K, seed=41)
    want = oracle.dequant_bf16(packed, scale, zp)
    dp = torch.from_numpy(packed.view(np.int32)).cuda()
    ds = torch.from_numpy(scale.view(np.int16)).cuda()
    dz = torch.from_numpy(zp.view(np.int32)).cuda()
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    with torch.cuda.stream(st):
        for _ in range(3):
            w = pkg.awq_alloc_fused(N, K)          # uses the current stream = st
            pkg.awq_repack_into(w, 0, dp, ds, dz, stream=st)
            dst = torch.empty((N, K), dtype=torch.bfloat16, device="cuda")
            pkg.w4a16_dequant_rows(dst, w, 0, N, stream=st)
            st.synchronize()
            assert np.array_equal(host_bits(dst), want)
            pkg.awq_free(w)


def test_matmul_right_behind_a_repack_on_the_same_stream(pkg, oracle, synth):
    """The decode kernels fetch weights before they wait for the kernel in front of them, so the library
    enqueues the first matmul behind a weight write on its stream as a fully serialised launch. A repack
    followed at once by a GEMV, with no synchronisation in between, must give the bits of a GEMV on settled
    weights - for every one of a few rounds that overwrite the same container with new weights."""
    N, K = 4096, 2048
    st = torch.cuda.Stream()
    s = pkg.gemv_scratch_alloc(K, N, 128, 1)
    x = dev_bf16(synth.make_activations(1, K, seed=9)[0])
    torch.cuda.synchronize()
    with torch.cuda.stream(st):
        w = pkg.awq_alloc_fused(N, K)
        for rnd in range(4):
            packed, scale, zp = synth.make_weights(N, K, seed=50 + rnd)
            dp = torch.from_numpy(packed.view(np.int32)).cuda()
            ds = torch.from_numpy(scale.view(np.int16)).cuda()
            dz = torch.from_numpy(zp.view(np.int32)).cuda()
            torch.cuda.synchronize()  # the uploads above ran on this stream too; what is tested comes next
            early = torch.empty(N, dtype=torch.bfloat16, device="cuda")
            pkg.awq_repack_into(w, 0, dp, ds, dz, stream=st)
            pkg.gemv_w4a16(early, w, x, s, stream=st)   # no synchronisation since the repack
            st.synchronize()
            settled = torch.empty(N, dtype=torch.bfloat16, device="cuda")
            pkg.gemv_w4a16(settled, w, x, s, stream=st)
            st.synchronize()
            assert torch.equal(early.view(torch.int16), settled.view(torch.int16)), f"round {rnd}"
            ref = oracle.gemm_f64(packed, scale, zp, synth.make_activations(1, K, seed=9))[0]
            got = synth.bf16_bits_to_f32(host_bits(settled)).astype(np.float64)
            assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) <= 1e-2
        pkg.awq_free(w)
    assert pkg.device_status() == 0
    pkg.gemv_scratch_free(s)
