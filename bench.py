#!/usr/bin/env python3
"""Benchmark of the W4A16 matmul path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

The headline "step" is one full decode token's weight pass: the 256 W4A16 GEMVs (M=1) of the
64-layer model, each on its own weight buffer (12.6 GB of packed int4 weights in total, far
larger than L2, so every step streams from HBM), replayed as one CUDA graph. Inputs are seeded
synthetic tensors with the checkpoint's shapes and the value distributions the benchmark
configuration states; the real checkpoint is not available here.

Prints ONE JSON line (rank 0). `value` is algorithmic TB/s over the whole job with everything
resident in HBM (median of several timed regions of exactly --steps steps; the spread is in
`regions_ms_per_step`); `e2e` is the same metric through the public C-ABI launchers with the
step's activations copied from pinned host memory and the result copied back inside the timed
region. `roofline` compares the GEMV kernel with the measured HBM copy bandwidth; `cpu_baseline`
times the CPU oracle on a bounded sample. `configs` carries the other benchmark configurations,
measured in the same run: the single GEMV (config 0), the 64-layer verify pass at M=9 and M=16
(config 2), the lm_head with fused argmax in int4 and int8 (config 3) and the prefill GEMM
(config 4).

With --gpus N > 1 (launched under torchrun, one rank per GPU) the layers are column-sharded over
the ranks; every sharded kernel stores its slice of the output straight into every rank's copy
over NVLink peer mappings and then raises a per-rank flag; the next layer's kernel waits for all
ranks' flags before it reads activations, so the timed pass carries one cross-rank
synchronisation per layer. The job is still one decode pass, so scaling is "strong".
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
PKG = "qwen38-3090-cuda-server_b200"

METRIC = "w4a16_gemv_hbm_tbps_full_decode_weight_pass"
UNIT = "TB/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0
WORKLOAD = "decode_weight_pass_256_gemv_M1"
REGIONS = 5            # timed regions of --steps steps each; the median is reported


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS}, "fallback"


def base_config(synth):
    """The `config` object both arms print: the workload the metric is quoted on."""
    shapes = synth.decode_pass_shapes()
    return {"workload": WORKLOAD, "layers": 64, "hidden": 5120, "gemvs_per_step": len(shapes),
            "algorithmic_bytes_per_step": sum(synth.algorithmic_bytes(N, K) for _, N, K in shapes),
            "cache": "inputs larger than L2 (12.6 GB of distinct weights per step)"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.rows, self.proc, self.gpu = [], None, gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for n, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            except Exception:
                pass
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------ reference arm
SAMPLE_LAYERS = 2
_CPU_CASES = None


def cpu_sample(repeats: int = 1):
    """Times the CPU oracle (dequant-then-fp32-matmul, all host threads) on the GEMVs of the first
    SAMPLE_LAYERS layers of the pass. Returns (TB/s, seconds per sample, description, threads)."""
    from oracle import oracle
    synth = importlib.import_module(PKG + ".synth")
    oracle.build()
    # every host core, whatever the launcher exported (torchrun sets OMP_NUM_THREADS=1 for its children)
    oracle.set_num_threads(os.cpu_count() or 1)
    global _CPU_CASES
    if _CPU_CASES is None:  # generated once; only the matmuls are timed
        _CPU_CASES = [(synth.make_weights(N, K, seed=i), synth.make_activations(1, K, seed=i), N, K)
                      for i, (_, N, K) in enumerate(synth.decode_pass_shapes()[: 4 * SAMPLE_LAYERS])]
    cases = _CPU_CASES
    nbytes = sum(synth.algorithmic_bytes(N, K) for _, _, N, K in cases)
    oracle.gemm_f32(*cases[0][0], cases[0][1])  # warm the thread pool
    t0 = time.perf_counter()
    for _ in range(repeats):
        for (w, x, N, K) in cases:
            oracle.gemm_f32(w[0], w[1], w[2], x)
    dt = (time.perf_counter() - t0) / repeats
    desc = (f"first {SAMPLE_LAYERS} of 64 layers ({len(cases)} of 256 GEMVs, {nbytes / 1e6:.0f} MB algorithmic), "
            f"oracle dequant-then-fp32-matmul, {repeats} repeat(s)")
    return nbytes / dt / 1e12, dt, desc, oracle.num_threads(), nbytes


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # The reference project has no CPU matmul of its own outside two test-embedded check loops, so its CPU
    # arm is the oracle port of that arithmetic, threaded over output rows. Each step times a bounded sample
    # of the pass (the first layers); ms_per_step is scaled to a whole pass by bytes.
    synth = importlib.import_module(PKG + ".synth")
    cfg = base_config(synth)
    times = []
    for i in range(args.warmup + args.steps):
        tb, dt, desc, threads, nbytes = cpu_sample(repeats=1)
        if i >= args.warmup:
            times.append(dt)
    dt = sum(times) / len(times)
    value = nbytes / dt / 1e12
    pass_ms = dt * 1e3 * cfg["algorithmic_bytes_per_step"] / nbytes
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": pass_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x int4 -> fp32", "data": "synthetic",
            "config": cfg,
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc,
                             "sample_ms": dt * 1e3},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------ our arm
def make_layer_weights(pkg, torch, gen, n_rows, K, seed):
    """Seeded on-device tensors in the on-disk layout, repacked into a weight container."""
    gen.manual_seed(seed)
    G = K // 128
    packed = torch.randint(-2 ** 31, 2 ** 31 - 1, (n_rows, K // 8), dtype=torch.int32, device="cuda", generator=gen)
    scale = (torch.randn((n_rows, G), device="cuda", generator=gen).abs() * 0.02 + 1e-4).to(torch.bfloat16)
    zp = torch.randint(-2 ** 31, 2 ** 31 - 1, (n_rows // 8, G), dtype=torch.int32, device="cuda", generator=gen)
    return pkg.awq_repack(packed, scale, zp)


def time_regions(torch, stream, step, steps, regions, barrier):
    """`regions` timed regions of exactly `steps` steps each, CUDA events on the launching stream."""
    out = []
    for _ in range(regions):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        barrier()
        out.append(e0.elapsed_time(e1) / steps)
    return out


def other_configs(pkg, synth, torch, layers, scratch, stream, peak_hbm, peak_tf, m1_ms, peak_tf_sustained=None):
    """Configs 0, 2, 3 and 4 of the benchmark on one GPU, after the headline measurement."""
    import shape_bench
    out = {}

    def shape(kind, N, K, M, iters):
        r = shape_bench.run_case(pkg, synth, torch, kind, N, K, M, iters, 768)
        d = {"us": round(r["us"], 2), "tbps": round(r["tbps"], 3), "frac_of_measured_hbm": round(r["tbps"] * 1e3 / peak_hbm, 3),
             "algorithmic_bytes": r["algorithmic_bytes"], "ring_copies": r["ring_copies"]}
        if kind == "prefill":
            # six back-to-back launches of about a millisecond: the burst peak is the denominator that applies
            d = {"us": round(r["us"], 1), "tflops": round(r["tflops"], 1), "frac_of_measured_bf16": round(r["tflops"] / peak_tf, 3)}
            if peak_tf_sustained:
                d["frac_of_measured_bf16_sustained"] = round(r["tflops"] / peak_tf_sustained, 3)
        return d

    out["config0_gemv_17408x5120_M1"] = shape("gemv", 17408, 5120, 1, 48)
    out["config3_lm_head_argmax_int4"] = {f"M{M}": shape("lmhead", 248320, 5120, M, 12) for M in (1, 9)}
    out["config3_lm_head_argmax_int8"] = {f"M{M}": shape("lmhead8", 248320, 5120, M, 12) for M in (1, 9)}

    # config 2: the 64-layer verify pass (skinny GEMM on every linear layer), same weight buffers as the M=1 pass
    verify = {}
    for M in (9, 16):
        xs = {L["K"]: None for L in layers}
        for K in xs:
            xs[K] = torch.randn((M, K), device="cuda").to(torch.bfloat16)
        ys = {}
        for L in layers:
            ys.setdefault(L["N"], torch.empty((M, L["N"]), dtype=torch.bfloat16, device="cuda"))

        def one():
            for L in layers:
                pkg.gemm_mma_w4a16(ys[L["N"]], L["w"], xs[L["K"]], M, scratch)

        with torch.cuda.stream(stream):
            one()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                one()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            ms = time_regions(torch, stream, g.replay, 5, 3, torch.cuda.synchronize)
        med = statistics.median(ms)
        alg = sum(synth.algorithmic_bytes(L["N"], L["K"], M) for L in layers)
        verify[f"M{M}"] = {"ms_per_pass": round(med, 4), "x_cost_vs_M1_pass": round(med / m1_ms, 3),
                           "tbps": round(alg / med / 1e9, 3), "frac_of_measured_hbm": round(alg / med / 1e6 / peak_hbm, 3),
                           "algorithmic_bytes": alg, "regions_ms": [round(v, 4) for v in ms]}
        del g, xs, ys
    out["config2_verify_pass_256_skinny_gemm"] = verify

    out["config4_prefill_M4096"] = {"gate_up_34816x5120": shape("prefill", 34816, 5120, 4096, 6),
                                    "down_5120x17408": shape("prefill", 5120, 17408, 4096, 6)}
    return out


def sharded_configs(pkg, synth, torch, dist, symm_mem, comm, rank, world, local, peak_hbm, peak_tf):
    """The sharded forms of configs 2, 3 and 4 on `world` GPUs: the MLP layers of the verify pass (gate|up and
    down column-sharded, fused all-gather, flag wait between them), the vocab-sharded lm_head with the pair
    exchange inside the kernel, and the column-sharded prefill GEMM. Times are the slowest rank's."""
    dev = torch.device("cuda", local)
    gen = torch.Generator(device="cuda")
    out = {}
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())

    def sym(numel, dtype):
        t = symm_mem.empty(numel, dtype=dtype, device=dev)
        t.zero_()
        h = symm_mem.rendezvous(t, dist.group.WORLD)
        return t, [int(b) for b in h.buffer_ptrs]

    def sync_all():
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, iters, regions=3):
        """CUDA graph of `iters` calls of fn(i), median over `regions` replays, max over ranks; us per call."""
        with torch.cuda.stream(stream):
            fn(0)
            torch.cuda.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                for i in range(iters):
                    fn(i)
            g.replay()
            torch.cuda.synchronize()
            ms = time_regions(torch, stream, g.replay, 1, regions, sync_all)
        t = torch.tensor(ms, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return statistics.median([float(v) for v in t]) * 1e3 / iters

    scratch = pkg.gemv_scratch_alloc(17408, 34816, 128, 16)
    # ---- config 2: the MLP of the verify pass, sharded (a ring of 8 distinct layers: 8 x 140 MB per pass) ----
    I, H, copies = 17408, 5120, 8
    gu, dn = [], []
    for c in range(copies):
        b, e = pkg.shard_rows(2 * I, world, rank)
        gu.append((make_layer_weights(pkg, torch, gen, e - b, H, 5000 + 10 * c + rank), b))
        b, e = pkg.shard_rows(H, world, rank)
        dn.append((make_layer_weights(pkg, torch, gen, e - b, I, 6000 + 10 * c + rank), b))
    verify = {}
    for M in (1, 9, 16):
        x0 = torch.randn((M, H), device="cuda").to(torch.bfloat16)
        x1 = torch.randn((M, I), device="cuda").to(torch.bfloat16)
        y_gu, p_gu = sym(M * 2 * I, torch.bfloat16)
        y_dn, p_dn = sym(M * H, torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier()

        def mlp(i):
            # gate|up, then down; each waits for every rank's flag of the layer before it. (down reads a
            # pre-filled activation buffer: the SwiGLU between the two is not part of this path.)
            w, b = gu[i % copies]
            pkg.gemm_skinny_gather(p_gu, comm, 2 * I, b, w, x0, M, scratch, wait_prev=True, stream=stream)
            w, b = dn[i % copies]
            pkg.gemm_skinny_gather(p_dn, comm, H, b, w, x1, M, scratch, wait_prev=True, stream=stream)

        us = timed(mlp, 4 * copies)  # long graphs: the ranks' launch skew is paid once per replay
        alg = synth.algorithmic_bytes(2 * I, H, M) + synth.algorithmic_bytes(H, I, M)
        verify[f"M{M}"] = {"us_per_mlp": round(us, 2), "aggregate_tbps": round(alg / us / 1e6, 3)}
        del y_gu, y_dn
    out["config2_sharded_mlp_gate_up_down"] = verify

    # ---- the same MLP without the gather: row-sharded gate|up with the SwiGLU epilogue (local), K-sharded down,
    #      fp32 partials of [M, 5120] into every rank's buffer, reduced in rank order (one exchange per MLP) ----
    dk = [make_layer_weights(pkg, torch, gen, H, I // world, 6500 + 10 * c + rank) for c in range(copies)]
    free_mlp = {}
    for M in (1, 9, 16):
        x0 = torch.randn((M, H), device="cuda").to(torch.bfloat16)
        act = torch.empty((M, I // world), dtype=torch.bfloat16, device="cuda")
        hres = torch.zeros((M, H), dtype=torch.bfloat16, device="cuda")
        pbuf, p_pbuf = sym(world * M * H, torch.float32)
        torch.cuda.synchronize()
        dist.barrier()

        def mlp2(i):
            w, _ = gu[i % copies]
            pkg.linear_fused(act, w, x0, M, scratch, epilogue=pkg.EPILOGUE_SWIGLU, stream=stream)
            pkg.gemm_skinny_partial(p_pbuf, comm, dk[i % copies], act, M, scratch, stream=stream)
            pkg.reduce_partials(hres, pbuf, comm, M, H, residual=True, stream=stream)

        us = timed(mlp2, 4 * copies)
        alg = synth.algorithmic_bytes(2 * I, H, M, out_bytes=2 * M * I) + synth.algorithmic_bytes(H, I, M)
        free_mlp[f"M{M}"] = {"us_per_mlp": round(us, 2), "aggregate_tbps": round(alg / us / 1e6, 3)}
        del pbuf
    out["config2_sharded_mlp_gather_free"] = free_mlp
    for w in dk:
        pkg.awq_free(w)

    # ---- config 3: vocab-sharded lm_head, one launch per call (ring of weight copies larger than L2) ----
    V = 248320
    b, e = pkg.shard_rows(V, world, rank)
    shard_bytes = (e - b) * H // 2 + (e - b) * (H // 128) * 3
    ncopy = max(2, min(16, -(-800 * (1 << 20) // shard_bytes)))
    heads = [make_layer_weights(pkg, torch, gen, e - b, H, 7000 + 10 * c + rank) for c in range(ncopy)]
    table, p_table = sym(world * 16 * 2, torch.int32)
    head = {}
    hscratch = pkg.gemv_scratch_alloc(H, e - b, 128, 16)
    for M in (1, 9):
        hx = torch.randn((M, H), device="cuda").to(torch.bfloat16)
        ids = torch.zeros(M, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        dist.barrier()
        us = timed(lambda i: pkg.lm_head_argmax_sharded(ids, p_table, comm, b, heads[i % ncopy], hx, M, hscratch,
                                                        stream=stream), 4 * ncopy)
        alg = synth.algorithmic_bytes(V, H, M, out_bytes=4 * M)
        head[f"M{M}"] = {"us": round(us, 2), "aggregate_tbps": round(alg / us / 1e6, 3), "ring_copies": ncopy}
    out["config3_sharded_lm_head_argmax_int4"] = head
    for w in heads:
        pkg.awq_free(w)
    pkg.gemv_scratch_free(hscratch)

    # ---- config 4: column-sharded prefill, M = 4096 ----
    pre = {}
    ws = pkg.gemm_workspace_alloc(4096)
    Mp = 4096
    for name, N, K, wl in (("gate_up_34816x5120", 2 * I, H, gu), ("down_5120x17408", H, I, dn)):
        A = torch.randn((Mp, K), device="cuda").to(torch.bfloat16)
        C, p_c = sym(Mp * N, torch.bfloat16)
        torch.cuda.synchronize()
        dist.barrier()

        def pf(i):
            w, b0 = wl[i % copies]
            pkg.gemm_w4a16_sharded(p_c, comm, N, b0, w, A, Mp, ws, stream=stream)
            pkg.wait_gather(comm, stream=stream)

        us = timed(pf, 8)
        tf = 2.0 * Mp * N * K / us / 1e6
        recv = (world - 1) / world * Mp * N * 2
        pre[name] = {"us": round(us, 1), "aggregate_tflops": round(tf, 1),
                     "frac_of_measured_bf16_x_gpus": round(tf / (peak_tf * world), 3),
                     "nvlink_bytes_received_per_rank": int(recv),
                     "nvlink_bound_us_at_770GBps": round(recv / 770e3, 1)}
        del C
    out["config4_sharded_prefill_M4096"] = pre
    pkg.gemm_workspace_free(ws)
    for w, _ in gu + dn:
        pkg.awq_free(w)
    pkg.gemv_scratch_free(scratch)
    return out


def run_ours(args):
    import torch
    import torch.distributed as dist

    pkg = importlib.import_module(PKG)
    synth = importlib.import_module(PKG + ".synth")
    pkg.lib()  # fail loudly if the CUDA library is missing

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    shapes = synth.decode_pass_shapes()
    # With more than one GPU every linear layer is column-sharded (all widths are multiples of 16 x 8);
    # W4A16_BENCH_SHARD=mlp shards only the two MLP layers and keeps the rest as replicas.
    if world == 1:
        sharded = set()
    elif os.environ.get("W4A16_BENCH_SHARD", "all") == "mlp":
        sharded = {"gate_up", "down"}
    else:
        sharded = {"gate_up", "down", "gdn_in", "gdn_out", "attn_qkv", "attn_o"}
    gen = torch.Generator(device="cuda")

    # ---- build the 256 weight containers (distinct buffers: 12.6 GB at N=1) ----
    layers = []
    for i, (name, N, K) in enumerate(shapes):
        kind = name.split(".")[1]
        n_local, row0 = N, 0
        if kind in sharded:
            row0, row1 = pkg.shard_rows(N, world, rank)
            n_local = row1 - row0
        w = make_layer_weights(pkg, torch, gen, n_local, K, 1000 * i + (rank if kind in sharded else 0))
        layers.append({"kind": kind, "N": N, "K": K, "n_local": n_local, "row0": row0, "w": w, "index": i})
    torch.cuda.synchronize()

    scratch = pkg.gemv_scratch_alloc(17408, 34816, 128, 16)

    # activations: one arena for all inputs, one for all outputs (16-byte aligned slices)
    x_off, y_off, xo, yo = [], [], 0, 0
    for L in layers:
        x_off.append(xo)
        y_off.append(yo)
        xo += L["K"]
        yo += L["N"]
    x_host = torch.randn(xo, generator=torch.Generator().manual_seed(7)).to(torch.bfloat16).pin_memory()
    x_dev = torch.empty(xo, dtype=torch.bfloat16, device="cuda")
    x_dev.copy_(x_host)
    # Outputs: one arena. With more than one GPU the arena lives in symmetric memory, so that the sharded
    # layers' kernels can store their column slice straight into every rank's copy (fused all-gather over
    # NVLink peer mappings, no collective call on the data path). W4A16_BENCH_COMM=nccl keeps the baseline:
    # a slice per rank + ncclAllGather, launched eagerly.
    comm = os.environ.get("W4A16_BENCH_COMM", "fused") if world > 1 else "none"
    peer_bases = None
    if comm == "fused":
        import torch.distributed._symmetric_memory as symm_mem
        y_dev = symm_mem.empty(yo, dtype=torch.bfloat16, device=torch.device("cuda", local))
        y_dev.zero_()
        hdl = symm_mem.rendezvous(y_dev, dist.group.WORLD)
        peer_bases = [int(b) for b in hdl.buffer_ptrs]
        # completion flags: one 256-byte block per rank
        flag_block = symm_mem.empty(64, dtype=torch.int32, device=torch.device("cuda", local))
        flag_block.zero_()
        fh = symm_mem.rendezvous(flag_block, dist.group.WORLD)
        comm_obj = pkg.make_comm([int(b) for b in fh.buffer_ptrs], rank)
        torch.cuda.synchronize()
        dist.barrier()
    else:
        y_dev = torch.zeros(yo, dtype=torch.bfloat16, device="cuda")
    y_host = torch.empty(layers[-1]["N"], dtype=torch.bfloat16).pin_memory()
    y_parts = [torch.empty(L["n_local"], dtype=torch.bfloat16, device="cuda")
               if (L["kind"] in sharded and comm == "nccl") else None for L in layers]

    def one_pass():
        for i, L in enumerate(layers):
            x = x_dev[x_off[i]: x_off[i] + L["K"]]
            y = y_dev[y_off[i]: y_off[i] + L["N"]]
            if L["kind"] in sharded and comm == "fused":
                # the slice goes to every rank's arena, then this rank's flag; the launch itself first waits for
                # every rank's flag of the previous layer (a real decode step consumes the gathered activations)
                pkg.gemm_skinny_gather([b + 2 * y_off[i] for b in peer_bases], comm_obj, L["N"], L["row0"], L["w"], x, 1,
                                       scratch, wait_prev=True)
            elif L["kind"] in sharded:
                pkg.gemv_w4a16(y_parts[i], L["w"], x, scratch)
                dist.all_gather_into_tensor(y, y_parts[i])
            else:
                pkg.gemv_w4a16(y, L["w"], x, scratch)

    # ---- capture the pass into a CUDA graph (the reference replays its decode step as a graph) ----
    graph, graphed = None, False
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        one_pass()  # eager warm-up: one-time function attributes, NCCL channels
        torch.cuda.synchronize()
        # Only the NCCL baseline is launched eagerly (its collectives are kept out of the graph).
        if comm != "nccl" and os.environ.get("W4A16_BENCH_GRAPH", "1") != "0":
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    one_pass()
                graphed = True
            except Exception as e:  # keep measuring eagerly, and say so
                print(f"[bench] graph capture failed ({type(e).__name__}: {e}); timing eager launches",
                      file=sys.stderr)
                graph = None
        torch.cuda.synchronize()

        def step():
            if graphed:
                graph.replay()
            else:
                one_pass()

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        alg_bytes = sum(synth.algorithmic_bytes(L["N"], L["K"]) for L in layers)
        # what THIS GPU streams per pass (its shards of the sharded layers, the replicated layers in full)
        alg_local = sum(synth.algorithmic_bytes(L["n_local"], L["K"]) for L in layers)
        n_launch = len(layers)

        # ---- device-resident timing: REGIONS regions of exactly --steps steps ----
        warm = max(args.warmup, 3)
        for _ in range(warm):
            step()
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        torch.cuda.profiler.start()  # a profiler started with --profile-from-start off sees only the timed steps
        regions = time_regions(torch, stream, step, args.steps, REGIONS, barrier)
        torch.cuda.profiler.stop()

        # ---- end to end: inputs from pinned host memory, result back to the host, every step ----
        def e2e_step():
            x_dev.copy_(x_host, non_blocking=True)
            step()
            y_host.copy_(y_dev[y_off[-1]:], non_blocking=True)

        for _ in range(2):
            e2e_step()
        e2e_regions = time_regions(torch, stream, e2e_step, args.steps, 3, barrier)
        clocks = sampler.stop() if rank == 0 else None

    if world > 1:
        t = torch.tensor(regions + e2e_regions, device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # every region: the slowest rank's time
        regions, e2e_regions = [float(v) for v in t[:REGIONS]], [float(v) for v in t[REGIONS:]]
    ms_step = statistics.median(regions)
    ms_e2e = statistics.median(e2e_regions)
    status = pkg.device_status()

    # ---- multi-GPU: is the gathered arena what the unsharded kernels give? (after the timed regions) ----
    parity_ok = None
    if world > 1:
        ok = True
        seen = set()
        for i, L in enumerate(layers):
            if L["kind"] not in sharded or L["kind"] in seen:
                continue
            seen.add(L["kind"])
            x = x_dev[x_off[i]: x_off[i] + L["K"]]
            per = L["N"] // world
            for r in range(world):  # every rank's shard, recomputed here from its seed, against the arena
                w_r = make_layer_weights(pkg, torch, gen, per, L["K"], 1000 * i + r)
                y_r = torch.empty(per, dtype=torch.bfloat16, device="cuda")
                pkg.gemv_w4a16(y_r, w_r, x, scratch)
                torch.cuda.synchronize()
                got = y_dev[y_off[i] + r * per: y_off[i] + (r + 1) * per]
                ok = ok and bool(torch.equal(got.view(torch.int16), y_r.view(torch.int16)))
                pkg.awq_free(w_r)
        t = torch.tensor([1 if ok else 0], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        parity_ok = bool(int(t[0]))

    peaks, which = measured_peaks()
    peak = float(peaks.get("hbm_gbs", FALLBACK_HBM_GBS))
    peak_tf = float(peaks.get("bf16_tflops", FALLBACK_BF16_TFLOPS))
    extras = None
    if os.environ.get("W4A16_BENCH_EXTRAS", "1") != "0":
        if world == 1:
            extras = other_configs(pkg, synth, torch, layers, scratch, stream, peak, peak_tf, ms_step,
                                    peaks.get("bf16_tflops_sustained"))
        elif comm == "fused":
            extras = sharded_configs(pkg, synth, torch, dist, symm_mem, comm_obj, rank, world, local, peak, peak_tf)
        status = status or pkg.device_status()

    if rank == 0:
        value = alg_bytes / (ms_step * 1e-3) / 1e12
        e2e_value = alg_bytes / (ms_e2e * 1e-3) / 1e12
        # dominant kernel: the persistent W4A16 GEMV kernel, all 256 launches of a step.
        per_launch_bytes = alg_local / n_launch  # roofline of one GPU's kernel: that GPU's bytes
        per_launch_s = ms_step * 1e-3 / n_launch
        achieved = per_launch_bytes / per_launch_s / 1e9
        # DRAM bytes per launch of the dominant kernel: ncu measured 97.39 MB (read + write) for the
        # 93.68 MB (algorithmic) launch on out 34816 x in 5120 (ncu summary under profiles/);
        # the weight stream is read exactly once for every shape, so traffic scales with the bytes.
        traffic = per_launch_bytes * (97.39 / 93.68)
        cpu = None
        if world == 1 and not args.no_cpu:
            tb, dt, desc, threads, _ = cpu_sample(repeats=3)
            cpu = {"value": tb, "unit": UNIT, "cores": threads, "kind": "port", "sample": desc, "sample_ms": dt * 1e3}
        cfg = base_config(synth)
        run = {"launch": "cuda_graph" if graphed else "eager",
               "parallelism": "single" if world == 1 else
               (f"column_shard_x{world}({len(sharded)}_of_6_layer_kinds)+fused_peer_store_all_gather+flag_wait_per_layer"
                if comm == "fused" else f"column_shard_x{world}+nccl_all_gather")}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16 x int4 -> fp32", "data": "synthetic",
            "config": cfg,
            "run": run,
            "us_per_weight_pass": ms_step * 1e3,
            "regions_ms_per_step": [round(v, 4) for v in regions],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic, "peak_source": which,
                         "kernel": "k_skinny<MT=1> (persistent W4A16 GEMV, tcgen05 kind::i8)",
                         "frac_of_nominal_8TBps": achieved / 8000.0},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(x_host.numel() * 2),
                    "d2h_bytes_per_step": int(y_host.numel() * 2), "ms_per_step": ms_e2e,
                    "regions_ms_per_step": [round(v, 4) for v in e2e_regions]},
            "gpu_launches": n_launch * args.steps * REGIONS,
            "clocks": clocks,
            "device_status": status,
        }
        if parity_ok is not None:
            line["parity_ok"] = parity_ok
        if extras is not None:
            line["configs"] = extras
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
