"""Seeded synthetic inputs with the shapes and value distributions of the benchmark
configurations (weights, per-group scales, activations).  numpy only."""
from __future__ import annotations

import numpy as np

from .format import SaltV2Tensor


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    rounded = u + 0x7FFF + ((u >> 16) & 1)
    return (rounded >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << 16).view(np.float32)


def make_planes(n: int, k: int, planes: int, seed: int = 0,
                densities=(0.66, 0.10, 0.03), scale_mults=(1.0, 0.3, 0.1), group: int = 128):
    """trits[P,N,K] int8 and scales[P,N,K//group] fp32.

    Plane 1 is dense (P(-1)=P(+1)=0.33, P(0)=0.34); residual planes have nonzero density 10% / 3%
    with equiprobable signs.  Scales are 0.02*|N(0,1)|+1e-3 per (row, group); residual planes take
    0.3x / 0.1x the plane-1 scale."""
    rng = np.random.default_rng(seed)
    trits = np.zeros((planes, n, k), np.int8)
    for p in range(planes):
        u = rng.random((n, k), dtype=np.float32)
        d = densities[p]
        trits[p] = np.where(u < d / 2, -1, np.where(u < d, 1, 0)).astype(np.int8)
    base = (0.02 * np.abs(rng.standard_normal((n, k // group), dtype=np.float32)) + 1e-3).astype(np.float32)
    scales = np.stack([base * np.float32(scale_mults[p]) for p in range(planes)]).astype(np.float32)
    return trits, scales


def make_tensor(name: str, n: int, k: int, planes: int, seed: int = 0, **kw) -> SaltV2Tensor:
    trits, scales = make_planes(n, k, planes, seed, **kw)
    return SaltV2Tensor.from_matrix_planes(name, trits, scales)


def make_shard_tensor(name: str, n: int, k: int, planes: int, mode: str, rank: int, world: int, seed: int = 0, **kw) -> SaltV2Tensor:
    """One rank's shard of a synthetic [n, k] tensor, generated directly (the full tensor is never
    built): column-parallel -> [n / world, k]; row-parallel -> [n, k / world] padded with zero
    trits and zero scales to whole 256-wide tiles.  Distribution as `make_planes`."""
    if mode == "column":
        return make_tensor(name, n // world, k, planes, seed=seed * 1009 + rank, **kw)
    kv = k // world
    kp = (kv + 255) // 256 * 256
    trits, scales = make_planes(n, kv, planes, seed=seed * 1009 + rank, **kw)
    if kp != kv:
        tp_ = np.zeros((planes, n, kp), np.int8)
        tp_[:, :, :kv] = trits
        sp_ = np.zeros((planes, n, kp // 128), np.float32)
        sp_[:, :, : kv // 128] = scales
        trits, scales = tp_, sp_
    return SaltV2Tensor.from_matrix_planes(name, trits, scales)


def make_activations(m: int, k: int, seed: int = 0, outlier_fraction: float = 0.001, outlier_gain: float = 20.0,
                     bf16: bool = False) -> np.ndarray:
    """N(0,1) activations [m,k]; `outlier_fraction` of the channels (the same for every token) are
    scaled by `outlier_gain`.  With bf16=True the values are rounded to bfloat16 (returned as fp32)."""
    rng = np.random.default_rng(seed + 7919)
    x = rng.standard_normal((m, k), dtype=np.float32)
    n_out = int(round(outlier_fraction * k))
    if n_out:
        ch = rng.choice(k, n_out, replace=False)
        x[:, ch] *= np.float32(outlier_gain)
    if bf16:
        x = bf16_bits_to_f32(f32_to_bf16_bits(x))
    return x


def algorithmic_bytes(n: int, k: int, planes: int, codec_bytes_per_plane: int, m: int, x_size: int, y_size: int,
                      group: int = 128) -> int:
    """Bytes one linear call has to move: resident arenas read once, activations in, outputs out."""
    tiles = n * k // 256
    payload = tiles * planes * codec_bytes_per_plane
    scales = tiles * planes * (256 // group) * 2
    index = (2 * tiles) // 8 + 4 * ((tiles - 1) // 256)
    return payload + scales + index + m * k * x_size + m * n * y_size
