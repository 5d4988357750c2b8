"""The allocation-free GEMV entry point (collected last on purpose).

Some callers of this library cannot allocate device memory, and therefore cannot create the
scratch the regular launchers take: a server that has already given the rest of HBM to its KV
cache, or a latency-critical loop that cannot tolerate the device-wide synchronisation of an
allocation. For them `w4a16_gemv_static` keeps its scratch in a fixed device array inside the
library. It runs the same kernel on the same grid, so its output must equal the regular entry
point's bit for bit, on the first call and on a second call that reuses the array."""
import numpy as np
import pytest
import torch

from gpu_util import dev_bf16, rel_err

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K", [(5120, 17408), (17408, 5120)])
def test_static_scratch_gemv_equals_regular_gemv_twice(pkg, oracle, synth, N, K):
    packed, scale, zp = synth.make_weights(N, K, seed=21)
    w = pkg.weights_from_numpy(packed, scale, zp)
    s = pkg.gemv_scratch_alloc(K, N, 128, 1)
    ref64 = None
    for call in range(2):
        x = dev_bf16(synth.make_activations(1, K, seed=100 + call)[0])
        want = torch.empty(N, dtype=torch.bfloat16, device="cuda")
        pkg.gemv_w4a16(want, w, x, s)
        got = torch.full((N,), float("nan"), dtype=torch.bfloat16, device="cuda")
        pkg.gemv_w4a16_static(got, w, x)
        torch.cuda.synchronize()
        assert pkg.device_status() == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}: outputs differ"
        got32 = torch.empty(N, dtype=torch.float32, device="cuda")
        pkg.gemv_w4a16_static(got32, w, x, f32=True)
        if ref64 is None:  # and against the oracle once, with the GEMV tests' fp32 tolerance
            ref64 = oracle.gemm_f64(packed, scale, zp, synth.make_activations(1, K, seed=100))[0]
            assert rel_err(got32.cpu().numpy(), ref64) <= 1e-4
    pkg.gemv_scratch_free(s)
    pkg.awq_free(w)


def test_static_scratch_rejects_layers_beyond_its_limit(pkg, synth):
    N, K = 65536 + 128, 128
    packed, scale, zp = synth.make_weights(N, K, seed=1)
    w = pkg.weights_from_numpy(packed, scale, zp)
    x = torch.zeros(K, dtype=torch.bfloat16, device="cuda")
    y = torch.zeros(N, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(pkg.W4A16Error) as e:
        pkg.gemv_w4a16_static(y, w, x)
    assert e.value.code == -1 and "65536" in str(e.value)
    pkg.awq_free(w)


def test_static_scratch_entry_allocates_nothing_and_captures(pkg, synth):
    """After the first call on the device, further calls leave the free device memory where it was, and
    the entry can be captured into a CUDA graph whose replay gives the eager call's bits."""
    N, K = 4096, 2048
    packed, scale, zp = synth.make_weights(N, K, seed=5)
    w = pkg.weights_from_numpy(packed, scale, zp)
    x = dev_bf16(synth.make_activations(1, K, seed=6)[0])
    eager = torch.empty(N, dtype=torch.bfloat16, device="cuda")
    pkg.gemv_w4a16_static(eager, w, x)  # first call on this device: one-time kernel attribute, outside capture
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    for _ in range(3):
        pkg.gemv_w4a16_static(eager, w, x)
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, f"free device memory moved by {free0 - free1} bytes across three calls"
    replayed = torch.zeros(N, dtype=torch.bfloat16, device="cuda")
    side = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(g, stream=side):
            pkg.gemv_w4a16_static(replayed, w, x, stream=side)
        g.replay()
    torch.cuda.synchronize()
    assert pkg.device_status() == 0
    assert torch.equal(replayed.view(torch.int16), eager.view(torch.int16))
    pkg.awq_free(w)
