"""One rank of the 2+ GPU parity check (launched by torch.distributed.run from test_multi_gpu.py).

Checks, on real GPUs: (1) the skinny GEMM whose epilogue stores its column slice into every
rank's output over NVLink peer mappings (the fused all-gather) against the unsharded kernel and the
CPU oracle; (2) the vocab-sharded lm_head: per-rank (max, global index) pairs, 8*M-byte all-gather,
pair reduction, against the unsharded fused argmax; (3) the completion flags: two chained sharded
layers with no host barrier between them; (4) the one-launch sharded lm_head with the pair exchange
and reduction inside the kernel; (5) the column-sharded prefill GEMM."""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
PKG = "qwen38-3090-cuda-server_b200"


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    import torch.distributed._symmetric_memory as symm_mem
    pkg = importlib.import_module(PKG)
    synth = importlib.import_module(PKG + ".synth")
    sharding = importlib.import_module(PKG + ".sharding")
    from oracle import oracle
    from gpu_util import dev_bf16, host_bits, rel_err

    N, K, M = 4096, 1024, 9
    packed, scale, zp = synth.make_weights(N, K, seed=11)
    x = synth.make_activations(M, K, seed=11)
    dx = dev_bf16(x)
    s = pkg.gemv_scratch_alloc(K, N, 128, 16)
    w_full = pkg.weights_from_numpy(packed, scale, zp)
    sp, ss, sz, row0 = sharding.shard_on_disk(packed, scale, zp, world, rank)
    w_shard = pkg.weights_from_numpy(sp, ss, sz)

    # ---- fused all-gather: peer stores from the epilogue ----
    y = symm_mem.empty(M * N, dtype=torch.bfloat16, device=torch.device("cuda", local))
    y.zero_()
    hdl = symm_mem.rendezvous(y, dist.group.WORLD)
    ptrs = [int(p) for p in hdl.buffer_ptrs]
    torch.cuda.synchronize()
    dist.barrier()
    pkg.gemm_skinny_sharded(ptrs, rank, N, row0, w_shard, dx, M, s)
    torch.cuda.synchronize()
    dist.barrier()  # every rank's stores have landed everywhere
    got = synth.bf16_bits_to_f32(host_bits(y.view(M, N))).astype(np.float64)
    ref = oracle.gemm_f64(packed, scale, zp, x)
    e = rel_err(got, ref)
    assert e <= 1e-2, f"rank {rank}: fused all-gather relative error {e}"
    y1 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w4a16(y1, w_full, dx, M, s)
    one = synth.bf16_bits_to_f32(host_bits(y1)).astype(np.float64)
    assert np.max(np.abs(got - one)) <= 2 * np.max(np.abs(ref)) * 2.0 ** -8, "sharded and unsharded results differ"

    # ---- baseline: NCCL all-gather of the slices ----
    ys = torch.empty((M, N // world), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_small_w4a16(ys, w_shard, dx, M, s)
    parts = [torch.empty_like(ys) for _ in range(world)]
    dist.all_gather(parts, ys)
    yg = torch.cat(parts, dim=1)
    assert torch.equal(yg.view(torch.int16), y.view(M, N).view(torch.int16)), "NCCL gather != fused peer stores"

    # ---- sharded lm_head: pairs + reduce ----
    pairs = torch.zeros((M, 2), dtype=torch.int32, device="cuda")
    pkg.lm_head_argmax(None, w_shard, dx, M, s, pairs=pairs, row_offset=row0)
    allp = torch.empty((world, M, 2), dtype=torch.int32, device="cuda")
    dist.all_gather_into_tensor(allp, pairs)
    ids = torch.zeros(M, dtype=torch.int32, device="cuda")
    pkg.argmax_pairs_reduce(ids, allp, world, M)
    ids1 = torch.zeros(M, dtype=torch.int32, device="cuda")
    pkg.lm_head_argmax(ids1, w_full, dx, M, s)
    want, gaps, _ = oracle.lm_head_argmax(packed, scale, zp, x)
    torch.cuda.synchronize()
    a, b = ids.cpu().numpy(), ids1.cpu().numpy()
    assert all(p == q or g == 0 for p, q, g in zip(a, want, gaps)), (a, want)
    assert all(p == q or g == 0 for p, q, g in zip(a, b, gaps)), (a, b)
    assert pkg.device_status() == 0

    # ---- completion flags: two chained sharded layers with no host barrier in between ----
    blocks = symm_mem.empty(64, dtype=torch.int32, device=torch.device("cuda", local))
    blocks.zero_()
    bh = symm_mem.rendezvous(blocks, dist.group.WORLD)
    comm = pkg.make_comm([int(p) for p in bh.buffer_ptrs], rank)
    N2 = 2048
    p2, s2, z2 = synth.make_weights(N2, N, seed=12)            # layer 2 consumes the gathered [M, N] of layer 1
    sp2, ss2, sz2, row2 = sharding.shard_on_disk(p2, s2, z2, world, rank)
    w2_shard = pkg.weights_from_numpy(sp2, ss2, sz2)
    w2_full = pkg.weights_from_numpy(p2, s2, z2)
    s_big = pkg.gemv_scratch_alloc(N, N, 128, 16)
    ya = symm_mem.empty(M * N, dtype=torch.bfloat16, device=torch.device("cuda", local))
    yb = symm_mem.empty(M * N2, dtype=torch.bfloat16, device=torch.device("cuda", local))
    ya.zero_()
    yb.zero_()
    ha, hb = symm_mem.rendezvous(ya, dist.group.WORLD), symm_mem.rendezvous(yb, dist.group.WORLD)
    xs = dev_bf16(synth.make_activations(M, K, seed=13, sigma=0.05))
    torch.cuda.synchronize()
    dist.barrier()
    for rep in range(3):
        pkg.gemm_skinny_gather([int(p) for p in ha.buffer_ptrs], comm, N, row0, w_shard, xs, M, s_big)
        pkg.gemm_skinny_gather([int(p) for p in hb.buffer_ptrs], comm, N2, row2, w2_shard, ya.view(M, N), M, s_big,
                               wait_prev=True)
        pkg.wait_gather(comm)
        torch.cuda.synchronize()
        r1 = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
        r2 = torch.empty((M, N2), dtype=torch.bfloat16, device="cuda")
        pkg.gemm_small_w4a16(r1, w_full, xs, M, s_big)
        pkg.gemm_small_w4a16(r2, w2_full, r1, M, s_big)
        torch.cuda.synchronize()
        # sharded and unsharded runs split the K range differently across CTAs: equal up to fp32 summation order,
        # i.e. at most one bf16 ulp per element
        d1 = (ya.view(M, N).float() - r1.float()).abs().max().item()
        d2 = (yb.view(M, N2).float() - r2.float()).abs().max().item()
        assert d1 <= r1.float().abs().max().item() * 2.0 ** -7, (rep, d1)
        assert d2 <= r2.float().abs().max().item() * 2.0 ** -6, (rep, d2)
        dist.barrier()
    assert pkg.device_status() == 0

    # ---- vocab-sharded lm_head in one launch: pairs exchanged by peer stores + flag, reduced in the kernel ----
    table = symm_mem.empty(world * 16 * 2, dtype=torch.int32, device=torch.device("cuda", local))
    table.zero_()
    ht = symm_mem.rendezvous(table, dist.group.WORLD)
    torch.cuda.synchronize()
    dist.barrier()
    for Mh in (1, M):
        ids_s = torch.full((Mh,), -1, dtype=torch.int32, device="cuda")
        pkg.lm_head_argmax_sharded(ids_s, [int(p) for p in ht.buffer_ptrs], comm, row0, w_shard, dx[:Mh], Mh, s_big)
        torch.cuda.synchronize()
        got = ids_s.cpu().numpy()
        assert all(p == q or g == 0 for p, q, g in zip(got, want[:Mh], gaps[:Mh])), (Mh, got, want[:Mh])
        dist.barrier()
    assert pkg.device_status() == 0

    # ---- gather-free MLP: row-sharded gate|up + SwiGLU (local), K-sharded down, partials reduced in rank order ----
    Hm, Im, Mm = 1024, 2048, 8
    gate, up = synth.make_weights(Im, Hm, seed=21), synth.make_weights(Im, Hm, seed=22)
    down = synth.make_weights(Hm, Im, seed=23)

    def dev(a, dt=np.int32):
        return torch.from_numpy(np.ascontiguousarray(a).view(dt)).cuda()

    def swiglu_container(g, u, inter):
        wq = pkg.awq_alloc_fused(2 * inter, Hm)
        for off, (pk, sc, zz) in ((0, g), (inter, u)):
            pkg.awq_repack_into_swiglu(wq, off, dev(pk), dev(sc, np.int16), dev(zz), inter)
        return wq

    xm = dev_bf16(synth.make_activations(Mm, Hm, seed=24, sigma=0.5))
    h0 = synth.make_activations(Mm, Hm, seed=25)
    sm = pkg.gemv_scratch_alloc(Im, 2 * Im, 128, 16)
    full_gu, full_dn = swiglu_container(gate, up, Im), pkg.weights_from_numpy(*down)
    act = torch.empty((Mm, Im), dtype=torch.bfloat16, device="cuda")
    pkg.linear_fused(act, full_gu, xm, Mm, sm, epilogue=pkg.EPILOGUE_SWIGLU)
    h_ref = dev_bf16(h0).clone()
    pkg.linear_fused(h_ref, full_dn, act, Mm, sm, epilogue=pkg.EPILOGUE_RESIDUAL)
    w_gu = swiglu_container(sharding.shard_on_disk(*gate, world, rank)[:3], sharding.shard_on_disk(*up, world, rank)[:3],
                            Im // world)
    w_dn = pkg.weights_from_numpy(*sharding.shard_k_on_disk(*down, world, rank)[:3])
    pbuf = symm_mem.empty(world * Mm * Hm, dtype=torch.float32, device=torch.device("cuda", local))
    pbuf.zero_()
    hp = symm_mem.rendezvous(pbuf, dist.group.WORLD)
    torch.cuda.synchronize()
    dist.barrier()
    for rep in range(2):
        h_r = dev_bf16(h0).clone()
        act_r = torch.empty((Mm, Im // world), dtype=torch.bfloat16, device="cuda")
        pkg.linear_fused(act_r, w_gu, xm, Mm, sm, epilogue=pkg.EPILOGUE_SWIGLU)
        pkg.gemm_skinny_partial([int(p) for p in hp.buffer_ptrs], comm, w_dn, act_r, Mm, sm)
        pkg.reduce_partials(h_r, pbuf, comm, Mm, Hm, residual=True)
        torch.cuda.synchronize()
        assert rel_err(h_r.float().cpu().numpy().astype(np.float64), h_ref.float().cpu().numpy().astype(np.float64)) <= 1e-2
        allh = [torch.empty_like(h_r) for _ in range(world)]
        dist.all_gather(allh, h_r)
        assert all(torch.equal(a.view(torch.int16), allh[0].view(torch.int16)) for a in allh), "ranks disagree"
        dist.barrier()
    assert pkg.device_status() == 0

    # ---- column-sharded prefill: tiles stored into every rank's C, then the flag ----
    Mp = 300
    ws = pkg.gemm_workspace_alloc(4096)
    xp = dev_bf16(synth.make_activations(Mp, K, seed=14))
    cp = symm_mem.empty(Mp * N, dtype=torch.bfloat16, device=torch.device("cuda", local))
    cp.zero_()
    hc = symm_mem.rendezvous(cp, dist.group.WORLD)
    torch.cuda.synchronize()
    dist.barrier()
    pkg.gemm_w4a16_sharded([int(p) for p in hc.buffer_ptrs], comm, N, row0, w_shard, xp, Mp, ws)
    pkg.wait_gather(comm)
    torch.cuda.synchronize()
    cfull = torch.empty((Mp, N), dtype=torch.bfloat16, device="cuda")
    pkg.gemm_w4a16(cfull, w_full, xp, Mp, ws)
    torch.cuda.synchronize()
    assert torch.equal(cp.view(Mp, N).view(torch.int16), cfull.view(torch.int16)), "sharded prefill != unsharded"
    assert pkg.device_status() == 0
    dist.barrier()
    if rank == 0:
        print(f"MULTI_GPU_OK world={world} fused-gather rel {e:.2e}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
