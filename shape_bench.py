#!/usr/bin/env python3
"""Per-shape timing of the W4A16 kernels on one GPU, cold cache.

    python shape_bench.py --case gemv:17408x5120:1 [--case skinny:34816x5120:9 ...]
                          [--iters 50] [--ring-mb 768] [--json out.json]

case = kind:NxK:M with kind in {gemv, skinny, lmhead, prefill} for the int4 weights and
{gemv8, skinny8, lmhead8} for the int8 lm_head variant. Each case cycles through a ring of
distinct weight copies whose total size exceeds `--ring-mb` (several times the 126 MB L2),
so every launch streams its weights from HBM. The launches are captured back to back into
one CUDA graph (as the decode step is) and timed with CUDA events; the figure is the mean
per launch. This is also the
small driver used for `ncu` captures of a single kernel (`--iters 1 --ring-mb 0`).
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
PKG = "qwen38-3090-cuda-server_b200"


def run_case(pkg, synth, torch, kind, N, K, M, iters, ring_mb, warmup=5, graph=True):
    G = K // 128
    w8 = kind.endswith("8")
    wbytes = (N * K + N * G * 2) if w8 else (N * K // 2 + N * G * 3)
    copies = max(1, min(64, -(-ring_mb * (1 << 20) // wbytes))) if ring_mb > 0 else 1
    if kind == "prefill" and M >= 1024:
        copies = 1  # compute bound: one weight copy (below that the weight stream matters: keep the ring)
    gen = torch.Generator(device="cuda").manual_seed(N * 31 + K)
    ws = []
    for _ in range(copies if not w8 else 0):
        packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (N, K // 8), dtype=torch.int32, device="cuda", generator=gen)
        scale = (torch.randn((N, G), device="cuda", generator=gen).abs() * 0.02 + 1e-4).to(torch.bfloat16)
        zp = torch.randint(-2 ** 31, 2 ** 31 - 1, (N // 8, G), dtype=torch.int32, device="cuda", generator=gen)
        ws.append(pkg.awq_repack(packed, scale, zp))
        del packed, scale, zp
    for _ in range(copies if w8 else 0):
        src = (torch.randn((N, K), device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
        ws.append(pkg.quantize_w8a16(src))
        torch.cuda.synchronize()
        del src
    x = torch.randn((M, K), device="cuda", generator=gen).to(torch.bfloat16)
    y = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    ids = torch.zeros(M, dtype=torch.int32, device="cuda")
    s = pkg.gemv_scratch_alloc(K, N, 128, 16)
    gws = pkg.gemm_workspace_alloc(4096) if kind == "prefill" else None

    def launch(i):
        w = ws[i % copies]
        if kind == "gemv":
            pkg.gemv_w4a16(y, w, x, s)
        elif kind == "skinny":
            pkg.gemm_mma_w4a16(y, w, x, M, s)
        elif kind == "lmhead":
            pkg.lm_head_argmax(ids, w, x, M, s)
        elif kind == "prefill":
            pkg.gemm_w4a16(y, w, x, M, gws)
        elif kind == "gemv8":
            pkg.gemv_w8a16(y, w, x, s)
        elif kind == "skinny8":
            pkg.gemm_small_w8a16(y, w, x, M, s)
        elif kind == "lmhead8":
            pkg.lm_head_argmax_w8(ids, w, x, M, s)
        else:
            raise SystemExit(f"unknown kind {kind}")

    for i in range(warmup if iters > 1 else 0):
        launch(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph and iters > 1:
        # one CUDA graph of `iters` back-to-back launches: no host launch cost in the timed region
        st = torch.cuda.Stream()
        st.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(st):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for i in range(iters):
                    launch(i)
            g.replay()
            torch.cuda.synchronize()
            e0.record(st)
            g.replay()
            e1.record(st)
        torch.cuda.synchronize()
    else:
        e0.record()
        for i in range(iters):
            launch(i)
        e1.record()
        torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    out_bytes = 4 * M if kind.startswith("lmhead") else 2 * M * N
    if w8:  # int8 codes + bf16 scales + activations in + output
        alg = N * K + 2 * N * G + 2 * M * K + out_bytes
    else:
        alg = synth.algorithmic_bytes(N, K, M, out_bytes=out_bytes)
    status = pkg.device_status()
    pkg.gemv_scratch_free(s)
    for w in ws:
        pkg.w8a16_free(w) if w8 else pkg.awq_free(w)
    if gws is not None:
        pkg.gemm_workspace_free(gws)
    return {"kind": kind, "N": N, "K": K, "M": M, "us": us, "algorithmic_bytes": alg,
            "tbps": alg / us / 1e6, "tflops": 2.0 * M * N * K / us / 1e6, "ring_copies": copies, "iters": iters,
            "device_status": status}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", action="append", required=True)
    ap.add_argument("--iters", type=int, default=50)
    ap.add_argument("--ring-mb", type=int, default=768)
    ap.add_argument("--json", default=None)
    ap.add_argument("--eager", action="store_true", help="time eager launches instead of one CUDA graph")
    a = ap.parse_args()
    import torch
    pkg = importlib.import_module(PKG)
    synth = importlib.import_module(PKG + ".synth")
    pkg.lib()
    peak, tf_peak = 6552.0, 1605.5
    try:
        mp = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        peak, tf_peak = float(mp["hbm_gbs"]), float(mp["bf16_tflops"])
    except Exception:
        pass
    rows = []
    for c in a.case:
        kind, shape, m = c.split(":")
        N, K = (int(v) for v in shape.split("x"))
        r = run_case(pkg, synth, torch, kind, N, K, int(m), a.iters, a.ring_mb, graph=not a.eager)
        r["frac_of_measured_hbm"] = r["tbps"] * 1e3 / peak
        rows.append(r)
        if kind == "prefill":
            r["frac_of_measured_bf16"] = r["tflops"] / tf_peak
            print(f"{kind:7s} {N:6d}x{K:<6d} M={int(m):4d}  {r['us']:9.2f} us  {r['tflops']:7.1f} TFLOP/s  "
                  f"{100 * r['frac_of_measured_bf16']:5.1f}% of {tf_peak:.0f} TFLOP/s  status {r['device_status']}",
                  flush=True)
            continue
        print(f"{kind:7s} {N:6d}x{K:<6d} M={int(m):2d}  {r['us']:9.2f} us  {r['tbps']:6.3f} TB/s  "
              f"{100 * r['frac_of_measured_hbm']:5.1f}% of {peak:.0f} GB/s  status {r['device_status']}", flush=True)
    if a.json:
        os.makedirs(os.path.dirname(os.path.abspath(a.json)), exist_ok=True)
        json.dump(rows, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
