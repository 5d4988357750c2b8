"""Seeded synthetic tensors in the checkpoint's on-disk layout.

The reference server measures on its real AWQ checkpoint, which is not
available here; these tensors have the checkpoint's shapes, dtypes and packing
and the value distributions the benchmark configuration states:
  weights  int4 nibbles uniform 0..15, 8 per uint32 along K
           (element i -> bits [4(i%8), 4(i%8)+4) of word i/8)
  scales   bf16( |N(0, 0.02)| + 1e-4 ), one per (row, group of 128 along K)
  zeros    int4 nibbles uniform 0..15, 8 ROWS per uint32 (row o -> nibble o%8 of word [o/8][g])
  x        bf16( N(0, 1) )
Packing follows src/loader/w4a16_unpack.h:6-24 of the reference project.
"""
from __future__ import annotations

import numpy as np


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit pattern (uint16)."""
    u = np.ascontiguousarray(a, np.float32).view(np.uint32)
    r = (u >> np.uint32(16)) & np.uint32(1)
    return ((u + np.uint32(0x7FFF) + r) >> np.uint32(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def pack_weight(nib: np.ndarray) -> np.ndarray:
    """uint8 nibbles [N, K] (0..15) -> uint32 [N, K/8], packed along K."""
    N, K = nib.shape
    v = nib.astype(np.uint32).reshape(N, K // 8, 8)
    sh = (np.arange(8, dtype=np.uint32) * np.uint32(4))[None, None, :]
    return np.bitwise_or.reduce(v << sh, axis=2).astype(np.uint32)


def pack_zero_point(nib: np.ndarray) -> np.ndarray:
    """uint8 nibbles [N, G] (0..15) -> uint32 [N/8, G], packed down the output axis."""
    N, G = nib.shape
    v = nib.astype(np.uint32).reshape(N // 8, 8, G)
    sh = (np.arange(8, dtype=np.uint32) * np.uint32(4))[None, :, None]
    return np.bitwise_or.reduce(v << sh, axis=1).astype(np.uint32)


def make_weights(N: int, K: int, group: int = 128, seed: int = 0, scale_sigma: float = 0.02):
    """Returns (packed uint32 [N,K/8], scale uint16 [N,G], zp uint32 [N/8,G])."""
    rng = np.random.Generator(np.random.PCG64(seed))
    G = K // group
    packed = rng.integers(0, 2 ** 32, size=(N, K // 8), dtype=np.uint64).astype(np.uint32)
    scale = f32_to_bf16_bits((np.abs(rng.standard_normal((N, G))) * scale_sigma + 1e-4)
                             .astype(np.float32))
    zp = rng.integers(0, 2 ** 32, size=(N // 8, G), dtype=np.uint64).astype(np.uint32)
    return packed, scale, zp


def make_activations(M: int, K: int, seed: int = 0, sigma: float = 1.0) -> np.ndarray:
    """bf16 bits [M, K] ~ N(0, sigma)."""
    rng = np.random.Generator(np.random.PCG64(seed + 7919))
    return f32_to_bf16_bits((rng.standard_normal((M, K)) * sigma).astype(np.float32))


# Per-layer linear shapes (K -> N) of one decode token's weight pass:
# 64 layers in a 16 x (GDN, GDN, GDN, Attn) pattern, hidden 5120.
def decode_pass_shapes():
    """List of (name, N, K) for the 256 GEMVs of one token, in execution order."""
    mlp = [("gate_up", 34816, 5120), ("down", 5120, 17408)]
    gdn = [("gdn_in", 16384, 5120), ("gdn_out", 5120, 8192)]
    att = [("attn_qkv", 8192, 5120), ("attn_o", 5120, 6144)]
    out = []
    for layer in range(64):
        mix = att if layer % 4 == 3 else gdn
        for name, N, K in (mix[0], mix[1], mlp[0], mlp[1]):
            out.append((f"L{layer}.{name}", N, K))
    return out


def algorithmic_bytes(N: int, K: int, M: int = 1, group: int = 128, out_bytes=None) -> int:
    """Minimum bytes one GEMV/GEMM must move: int4 weights + bf16 scales +
    4-bit zero points + bf16 activations in + output."""
    G = K // group
    if out_bytes is None:
        out_bytes = 2 * M * N
    return N * K // 2 + N * G * 2 + N * G // 2 + 2 * M * K + out_bytes
