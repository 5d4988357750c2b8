#!/usr/bin/env python3
"""Derive on-disk-format known-answer vectors from the reference's dequant fixtures.

The reference pins its int4 unpack with tests/fixtures/dequant/{manifest.json,
*.q8, *.f32}: for 7 real checkpoint tensors, a 64-row x 512-column block of the
signed codes q and of the dequantised fp32 values, both produced by
compressed_tensors' own unpack_from_int32 (tools/dump_dequant_ref.py:71-84 of
the reference project). The checkpoint itself is not needed to use them: for
every (row, group) the pair (zero point, bf16 scale) is the unique solution of
deq == float(q - zp) * scale, so the packed tensors can be rebuilt exactly.

This script solves for (zp, scale), re-packs q / zp with compressed_tensors'
pack_to_int32 (the library that defines the format) and writes
dequant_golden.npz next to itself:
  <stem>/packed  uint32 [64, 64]   weight_packed block   (packed along K)
  <stem>/scale   uint16 [64, 4]    bf16 bits
  <stem>/zp      uint32 [8, 4]     weight_zero_point block (packed along rows)
  <stem>/q       int8   [64, 512]  expected codes
  <stem>/deq     float32 [64, 512] expected dequantised values

Usage: python tests/golden/make_dequant_golden.py [reference_root]
"""
import json
import os
import sys

import numpy as np
import torch
from compressed_tensors.compressors.pack_quantized.helpers import pack_to_int32, unpack_from_int32


def bf16_round(a):
    u = a.astype(np.float32).view(np.uint32)
    r = (u >> 16) & 1
    return (((u + 0x7FFF + r) >> 16) << 16).astype(np.uint32).view(np.float32)


def solve_cell(q, deq):
    """q int [128], deq fp32 [128] -> (zp, scale_f32) with deq == float(q-zp)*scale exactly."""
    sols = []
    for zp in range(-8, 8):
        d = (q - zp).astype(np.float32)
        nz = d != 0
        if not nz.any():
            continue
        if np.any(deq[~nz] != 0):
            continue
        s = bf16_round(np.array([np.median(deq[nz].astype(np.float64) / d[nz])], np.float32))[0]
        if np.array_equal((d * s).astype(np.float32).view(np.uint32), deq.view(np.uint32)):
            sols.append((zp, s))
    assert len(sols) == 1, f"expected one solution, found {len(sols)}"
    return sols[0]


def main():
    here = os.path.dirname(os.path.abspath(__file__))
    default = os.environ.get("W4A16_REFERENCE_DIR") or os.path.join(here, "..", "..", "..", "reference")
    ref = sys.argv[1] if len(sys.argv) > 1 else default
    fx = os.path.join(ref, "tests", "fixtures", "dequant")
    man = json.load(open(os.path.join(fx, "manifest.json")))
    gs = man["group_size"]
    out = {}
    for t in man["tensors"]:
        rows, cols = t["rows"], t["cols"]
        stem = t["deq_file"][:-4]
        q = np.fromfile(os.path.join(fx, t["q_file"]), np.int8).reshape(rows, cols)
        deq = np.fromfile(os.path.join(fx, t["deq_file"]), np.float32).reshape(rows, cols)
        G = cols // gs
        zp = np.zeros((rows, G), np.int8)
        sc = np.zeros((rows, G), np.float32)
        for r in range(rows):
            for g in range(G):
                zp[r, g], sc[r, g] = solve_cell(q[r, g * gs:(g + 1) * gs].astype(np.int32),
                                                deq[r, g * gs:(g + 1) * gs])
        packed = pack_to_int32(torch.from_numpy(q), 4, packed_dim=1)
        zpp = pack_to_int32(torch.from_numpy(zp), 4, packed_dim=0)
        # the library must round-trip its own packing
        assert torch.equal(unpack_from_int32(packed, 4, torch.Size([rows, cols]), packed_dim=1),
                           torch.from_numpy(q))
        assert torch.equal(unpack_from_int32(zpp, 4, torch.Size([rows, G]), packed_dim=0),
                           torch.from_numpy(zp))
        out[stem + "/packed"] = packed.numpy().view(np.uint32)
        out[stem + "/scale"] = (sc.view(np.uint32) >> 16).astype(np.uint16)
        out[stem + "/zp"] = zpp.numpy().view(np.uint32)
        out[stem + "/q"] = q
        out[stem + "/deq"] = deq
        print(f"{stem}: zp in [{zp.min()},{zp.max()}], scale in [{sc.min():.3e},{sc.max():.3e}]")
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "dequant_golden.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
