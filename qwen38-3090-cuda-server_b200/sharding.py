"""Column (output-row) sharding of W4A16 layers over the GPUs of one node: host-side helpers.

The reference server is single-GPU (README.md:123 of the reference project); this is the plan the
sharded entry points of the C ABI implement. Output rows are independent, so rank r of g owns rows
[r*N/g, (r+1)*N/g) of a layer together with their scales and zero points, every rank holds the full
activations, and one exchange step follows:
  * MLP layers: all-gather of the [M, N/g] output slices into Y[M, N] (slices are column blocks);
  * lm_head: all-gather of M (max, global index) pairs per rank, then "larger value, else lower
    index" - no logits cross the link.
"""
from __future__ import annotations

import numpy as np


def shard_rows(out_f: int, nranks: int, rank: int):
    """Row range of `rank`; mirrors w4a16_shard_rows (whole 16-row blocks per rank)."""
    if not (0 <= rank < nranks):
        raise ValueError(f"rank {rank} of {nranks}")
    if out_f <= 0 or out_f % (16 * nranks) != 0:
        raise ValueError(f"out_f {out_f} does not split into {nranks} shards of whole 16-row blocks")
    per = out_f // nranks
    return rank * per, (rank + 1) * per


def shard_on_disk(packed, scale, zp, nranks: int, rank: int):
    """Slice the checkpoint's on-disk tensors to a rank's rows (zero points are packed 8 rows per word)."""
    b, e = shard_rows(packed.shape[0], nranks, rank)
    return packed[b:e], scale[b:e], zp[b // 8:e // 8], b


def shard_fused_gate_up(gate, up, nranks: int, rank: int):
    """gate|up are fused along N in the reference; shard each half by rows so a rank holds matching rows,
    and the gathered [M, 2*I] keeps the [gate | up] column order swiglu expects."""
    g = shard_on_disk(*gate, nranks, rank)
    u = shard_on_disk(*up, nranks, rank)
    return g, u


def shard_k_on_disk(packed, scale, zp, nranks: int, rank: int):
    """Slice the on-disk tensors along K (whole groups of 128) for a K-sharded layer: every output row, this
    rank's share of the input features. Returns (packed, scale, zp, k_begin)."""
    K = packed.shape[1] * 8
    if K % (128 * nranks) != 0:
        raise ValueError(f"in_f {K} does not split into {nranks} shards of whole 128-k groups")
    per = K // nranks
    k0, k1 = rank * per, (rank + 1) * per
    return (np.ascontiguousarray(packed[:, k0 // 8:k1 // 8]), np.ascontiguousarray(scale[:, k0 // 128:k1 // 128]),
            np.ascontiguousarray(zp[:, k0 // 128:k1 // 128]), k0)


def place_slice(y_full: np.ndarray, y_slice: np.ndarray, row_begin: int):
    """What the fused epilogue / the all-gather does: slice -> columns [row_begin, row_begin + n)."""
    y_full[:, row_begin:row_begin + y_slice.shape[1]] = y_slice
    return y_full


def reduce_pairs(values: np.ndarray, indices: np.ndarray) -> np.ndarray:
    """values float32 [ranks, M], indices int32 [ranks, M] -> ids [M]: larger value wins, then lower
    index; INT32_MAX marks 'no finite candidate' and yields 0 (w4a16_argmax_pairs_reduce)."""
    R, M = values.shape
    out = np.zeros(M, np.int32)
    for m in range(M):
        bv, bi = -np.finfo(np.float32).max, np.iinfo(np.int32).max
        for r in range(R):
            v, i = values[r, m], indices[r, m]
            if v > bv or (v == bv and i < bi):
                bv, bi = v, i
        out[m] = 0 if bi == np.iinfo(np.int32).max else bi
    return out


class FlagBlock:
    """Host model of one rank's completion-flag block (w4a16_comm_t): `flags[r]` is a counter written by rank r,
    `seq` counts this rank's own signalling launches. The device kernels implement exactly this:
      signal  (every CTA of a sharded launch, after its last store): its share of UNIT = 65536 is added to
              flags[this rank] on every rank; the launch as a whole adds UNIT and bumps `seq` once
      wait    (prologue of the consumer): passes once flags[r] - seq * UNIT >= 0 (as signed 32-bit) for every r
    All ranks issue the same sequence of signalling launches, so a rank's own `seq` names the launch whose
    slices it is waiting for; counters only grow, a peer that is already one launch ahead does not matter, and
    a launch of which only some CTAs have arrived does not reach the target."""
    UNIT = 1 << 16

    def __init__(self, nranks: int):
        self.flags = np.zeros(nranks, np.uint32)
        self.seq = np.uint32(0)

    def launch(self) -> int:
        """This rank signals one launch: returns what the launch adds to its counter on every rank."""
        self.seq = np.uint32((int(self.seq) + 1) & 0xFFFFFFFF)
        return self.UNIT

    def add(self, rank: int, amount: int):
        self.flags[rank] = np.uint32((int(self.flags[rank]) + amount) & 0xFFFFFFFF)

    def arrived(self) -> bool:
        target = (int(self.seq) * self.UNIT) & 0xFFFFFFFF
        d = (self.flags.astype(np.int64) - target) & 0xFFFFFFFF
        return bool(np.all(d < 0x80000000))
