"""Seeded synthetic inputs for the benchmark and parity workloads.

Uniform values come from the SplitMix64 stream the reference uses for weight
initialisation (crates/katsu-core/src/conv2d.rs:49-56): element i is a pure
function of seed + (i + 1) * 0x9e3779b97f4a7c15, so the stream vectorises.
Normal values are Box-Muller in f64 over two such uniforms, cast to f32.
No dataset is involved anywhere: the reference itself runs on a synthetic ramp
image (crates/katsu-core/examples/conv2d/main.rs:5-7).
"""
from __future__ import annotations

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix_u24(seed: int, count: int, offset: int = 0) -> np.ndarray:
    """Top 24 bits of SplitMix64 outputs offset+1 .. offset+count of `seed`, as uint64."""
    with np.errstate(over="ignore"):
        idx = np.arange(offset + 1, offset + count + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + idx * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        z ^= z >> np.uint64(31)
    return z >> np.uint64(40)


def uniform(seed: int, count: int, lo: float, hi: float) -> np.ndarray:
    """f32 values in [lo, hi): lo + (hi - lo) * u with u = bits / 2^24 (exact in f32)."""
    u = splitmix_u24(seed, count).astype(np.float32) / np.float32(16777216.0)
    return (np.float32(lo) + np.float32(hi - lo) * u).astype(np.float32)


def normal(seed: int, count: int, std: float) -> np.ndarray:
    """f32 N(0, std^2) by Box-Muller on consecutive pairs of the uniform stream."""
    bits = splitmix_u24(seed, 2 * count).astype(np.float64) / 16777216.0
    u1, u2 = bits[0::2], bits[1::2]
    z = np.sqrt(-2.0 * np.log1p(-u1)) * np.cos(2.0 * np.pi * u2)
    return (z * std).astype(np.float32)


def reference_weights(seed: int, count: int, fan_in: int) -> np.ndarray:
    """Conv2D::new_seeded's initialiser, conv2d.rs:46-58."""
    u = splitmix_u24(seed, count).astype(np.float32) / np.float32(16777216.0)
    bound = np.float32(1.0) / np.sqrt(np.float32(fan_in))
    return ((np.float32(2.0) * u - np.float32(1.0)) * bound).astype(np.float32)
