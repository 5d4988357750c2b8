"""The drop-in C++ headers (the reference's launcher names and signatures over the C ABI) must compile as
a caller would use them and link against the built library. No GPU is needed: nothing is executed."""
import os
import shutil
import subprocess
import tempfile

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CALLER = r'''
#include "kernels/gemv_w4a16.cuh"
#include "kernels/gemm_w4a16.cuh"
// the call sites of the reference server, in their own words (src/model/model.cu:103-128,634-660,796-815)
void caller(cudaStream_t st, const uint32_t* packed, const __nv_bfloat16* scale, const uint32_t* zp,
            const __nv_bfloat16* x, __nv_bfloat16* y, float* y32, int32_t* ids) {
  qwen::W4A16Weights w;
  qwen::awq_alloc_fused(w, 34816, 5120, 128, st);
  qwen::awq_repack_into(w, 0, packed, scale, zp, 17408, st);
  qwen::awq_repack_into(w, 17408, packed, scale, zp, 17408, st);
  qwen::GemvScratch s;
  qwen::gemv_scratch_alloc(s, 17408, 248320, 128, 16);
  qwen::gemv_partial_check(s, qwen::gemv_choose_splits(w.out_f, w.num_groups), w.out_f, 16);
  qwen::gemv_w4a16(y, w, x, s, st);
  qwen::gemv_w4a16_f32(y32, w, x, s, st);
  qwen::gemm_small_w4a16(y, w, x, 9, s, st);
  qwen::gemm_mma_w4a16(y, w, x, 16, s, st);
  qwen::lm_head_argmax_w4a16(ids, w, x, 1, s, nullptr, st);
  qwen::GemmWorkspace ws;
  qwen::gemm_workspace_alloc(ws, 1 << 20);
  qwen::gemm_w4a16(y, w, x, 4096, ws, st);
  qwen::w4a16_dequant_rows(y, w, 0, 64, st);
  qwen::gemm_workspace_free(ws);
  qwen::W8A16Weights w8;
  qwen::quantize_w8a16(w8, x, 248320, 5120, 128, st);
  qwen::gemv_w8a16(y, w8, x, s, st);
  qwen::gemm_small_w8a16(y, w8, x, 8, s, st);
  qwen::lm_head_argmax_w8a16(ids, w8, x, 9, s, nullptr, st);
  (void)w8.total_bytes();
  qwen::w8a16_free(w8);
  qwen::gemv_scratch_free(s);
  qwen::awq_free(w);
  (void)w.total_bytes();
  (void)qwen::gemv_scratch_bytes_for_m(s, 16);
}
int main() { return 0; }
'''


def test_dropin_headers_compile_and_link(pkg):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    pkg.lib()  # the library has to be there to link against
    pdir = os.path.dirname(pkg.LIB_PATH)
    with tempfile.TemporaryDirectory() as td:
        src = os.path.join(td, "caller.cu")
        with open(src, "w") as f:
            f.write(CALLER)
        cmd = [nvcc, "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a",
               "-I", os.path.join(pdir, "dropin"), "-I", os.path.join(ROOT, "include"),
               src, "-o", os.path.join(td, "caller"), "-L", pdir, "-lw4a16_b200", "-Xlinker", "-rpath," + pdir]
        out = subprocess.run(cmd, capture_output=True, text=True)
        assert out.returncode == 0, out.stdout + out.stderr


# The reference's own callers of the boundary, compiled unchanged against the drop-in headers.
REFERENCE = os.environ.get("W4A16_REFERENCE_DIR") or os.path.join(os.path.dirname(ROOT), "reference")
REFERENCE_CALLERS = ["src/model/model.cu", "src/draft/dflash.cu", "tests/gate_gemv.cu", "tests/gate_gemm.cu",
                     "bench/bench_decode_gemv.cu", "bench/bench_verify.cu"]


@pytest.mark.skipif(not os.path.isfile(os.path.join(REFERENCE, "src", "kernels", "gemv_w4a16.cuh")),
                    reason="reference checkout absent")
def test_reference_callers_compile_against_the_dropin_headers(pkg):
    """src/model, src/draft, the gates and the benches include the two kernel headers by relative path, so the
    drop-in replaces the files themselves: a mirror of the reference tree is made of symbolic links, with
    src/kernels/gemv_w4a16.cuh and gemm_w4a16.cuh pointing at the drop-in headers, and every caller is compiled
    (nvcc -c, nothing is run) exactly as it lies in the reference."""
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        pytest.skip("nvcc not found")
    pdir = os.path.dirname(pkg.LIB_PATH)
    dropin = os.path.join(pdir, "dropin", "kernels")
    with tempfile.TemporaryDirectory() as td:
        for top in ("src", "tests", "bench"):
            for d, _, files in os.walk(os.path.join(REFERENCE, top)):
                rel = os.path.relpath(d, REFERENCE)
                os.makedirs(os.path.join(td, rel), exist_ok=True)
                for f in files:
                    target = os.path.join(d, f)
                    if rel == os.path.join("src", "kernels") and f in ("gemv_w4a16.cuh", "gemm_w4a16.cuh"):
                        target = os.path.join(dropin, f)
                    os.symlink(target, os.path.join(td, rel, f))
        os.symlink(os.path.join(REFERENCE, "third_party"), os.path.join(td, "third_party"))
        procs = []
        for i, src in enumerate(REFERENCE_CALLERS):
            cmd = [nvcc, "-std=c++17", "--expt-relaxed-constexpr", "-gencode", "arch=compute_100a,code=sm_100a",
                   "-I", os.path.join(ROOT, "include"),
                   "-I", os.path.join(td, "src"), "-I", os.path.join(td, "third_party"), "-c", os.path.join(td, src),
                   "-o", os.path.join(td, f"caller{i}.o")]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        failures = []
        for src, p in procs:
            out, _ = p.communicate(timeout=900)
            if p.returncode != 0:
                failures.append(f"--- {src}\n{out[-3000:]}")
        assert not failures, "\n".join(failures)
