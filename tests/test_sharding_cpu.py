"""Multi-rank host logic on CPU: 2 gloo ranks, the oracle standing in for the GPU kernels."""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = "qwen38-3090-cuda-server_b200"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import importlib
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle import oracle
    synth = importlib.import_module(PKG + ".synth")
    sharding = importlib.import_module(PKG + ".sharding")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        N, K, M = 256, 512, 9
        packed, scale, zp = synth.make_weights(N, K, seed=3)
        x = synth.make_activations(M, K, seed=3)
        sp, ss, sz, row0 = sharding.shard_on_disk(packed, scale, zp, world, rank)
        # MLP-style layer: local slice, then all-gather into column blocks
        y_local = oracle.f32_to_bf16(oracle.gemm_f64(sp, ss, sz, x).astype(np.float32))
        slices = [torch.empty(M, N // world, dtype=torch.int32) for _ in range(world)]  # gloo has no 16-bit ints
        dist.all_gather(slices, torch.from_numpy(y_local.astype(np.int32)))
        y = np.zeros((M, N), np.uint16)
        for r, sl in enumerate(slices):
            b, _ = sharding.shard_rows(N, world, r)
            sharding.place_slice(y, sl.numpy().astype(np.uint16), b)
        want = oracle.f32_to_bf16(oracle.gemm_f64(packed, scale, zp, x).astype(np.float32))
        ok_gather = bool(np.array_equal(y, want))
        # lm_head: per-shard (max, global index) pairs, 8*M bytes per rank, then the pair reduction
        ids_local, _, logits = oracle.lm_head_argmax(sp, ss, sz, x, want_logits=True)
        vals = synth.bf16_bits_to_f32(logits[np.arange(M), ids_local])
        pair = torch.stack([torch.from_numpy(vals.view(np.int32).copy()), torch.from_numpy((ids_local + row0).astype(np.int32))])
        pairs = [torch.empty_like(pair) for _ in range(world)]
        dist.all_gather(pairs, pair)
        v = np.stack([p[0].numpy().view(np.float32) for p in pairs])
        i = np.stack([p[1].numpy() for p in pairs])
        ids = sharding.reduce_pairs(v, i)
        want_ids, _, _ = oracle.lm_head_argmax(packed, scale, zp, x)
        q.put((rank, ok_gather, bool(np.array_equal(ids, want_ids))))
    except Exception as e:  # surface the failure instead of letting the parent time out
        q.put((rank, False, False, repr(e)))
        raise
    finally:
        dist.destroy_process_group()


def test_two_rank_gather_and_pair_reduce():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(len(r) == 3 for r in res), res
    assert sorted(r[0] for r in res) == [0, 1]
    assert all(r[1] for r in res), "gathered column blocks differ from the unsharded result"
    assert all(r[2] for r in res), "pair-reduced argmax ids differ from the unsharded result"


def _flag_worker(rank, world, port, q):
    """Each rank keeps a FlagBlock; 'peer stores' of the flag value travel as gloo all-gathers. Rank 1 leaves
    after the second launch: rank 0's third wait must not pass (on the device it would run out and report)."""
    import importlib
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    sharding = importlib.import_module(PKG + ".sharding")
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        blk = sharding.FlagBlock(world)
        blk.seq = sharding.np.uint32(0xFFFF)              # next launch wraps the 32-bit counters
        blk.flags[:] = (0xFFFF << 16) & 0xFFFFFFFF
        seen = []
        for launch in range(2):
            amount = blk.launch()                           # this rank's launch is done: its CTAs add their shares
            vals = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
            dist.all_gather(vals, torch.tensor([amount], dtype=torch.int64))
            before = blk.arrived()                          # own seq moved on, the adds have not landed yet
            blk.add(rank, amount - 1)                       # all but one CTA of the own launch: still not enough
            partial = blk.arrived()
            blk.add(rank, 1)
            for r, t in enumerate(vals):
                if r != rank:
                    blk.add(r, int(t.item()))
            seen.append((before or partial, blk.arrived()))
        # third launch: only rank 0 takes part
        stuck = None
        if rank == 0:
            blk.add(0, blk.launch())
            stuck = not blk.arrived()
        q.put((rank, seen, stuck))
    except Exception as e:
        q.put((rank, repr(e), None))
        raise
    finally:
        dist.destroy_process_group()


def test_flag_protocol_two_ranks():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_flag_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=180) for _ in procs], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, seen, stuck in res:
        assert isinstance(seen, list), seen
        # before the peers' values land the wait does not pass; after, it does - across the 32-bit wrap too
        assert seen == [(False, True), (False, True)], (rank, seen)
    assert res[0][2] is True      # a rank that never signals keeps the others' wait from passing
    assert res[1][2] is None


def test_shard_planner_matches_c_abi(pkg):
    import importlib
    sharding = importlib.import_module(PKG + ".sharding")
    for out_f, g in [(34816, 8), (5120, 8), (248320, 8), (34816, 2), (5120, 4)]:
        for r in range(g):
            assert sharding.shard_rows(out_f, g, r) == pkg.shard_rows(out_f, g, r)
    with pytest.raises(ValueError):
        sharding.shard_rows(5136, 8, 0)
    with pytest.raises(pkg.W4A16Error):
        pkg.shard_rows(5136, 8, 0)


def test_pair_reduce_ties_and_empty():
    import importlib
    sharding = importlib.import_module(PKG + ".sharding")
    v = np.array([[1.0, -3.0, 5.0], [1.0, -2.0, 5.0]], np.float32)
    i = np.array([[7, 1, 9], [3, 2, 11]], np.int32)
    assert list(sharding.reduce_pairs(v, i)) == [3, 2, 9]
    big = np.iinfo(np.int32).max
    v = np.full((2, 1), -np.finfo(np.float32).max, np.float32)
    i = np.full((2, 1), big, np.int32)
    assert list(sharding.reduce_pairs(v, i)) == [0]
