"""One rank of the 2+ GPU parity check (launched by torch.distributed.run from test_multi_gpu.py).

Checks, on real GPUs: (1) the skinny GEMM whose epilogue stores its column slice into every
rank's output over NVLink peer mappings (the fused all-gather) against the unsharded kernel and the
CPU oracle; (2) the vocab-sharded lm_head: per-rank (max, global index) pairs, 8*M-byte all-gather,
pair reduction, against the unsharded fused argmax."""
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
    dist.barrier()
    if rank == 0:
        print(f"MULTI_GPU_OK world={world} fused-gather rel {e:.2e}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
