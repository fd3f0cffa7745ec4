"""Seeded synthetic inputs for the benchmark and parity workloads.

Uniform values come from the SplitMix64 stream the reference uses for weight
initialisation (crates/katsu-core/src/conv2d.rs:49-56): element i is a pure
function of seed + (i + 1) * 0x9e3779b97f4a7c15, so the stream vectorises.
Normal values are Box-Muller in f64 over two such uniforms, cast to f32.
No dataset is involved anywhere: the reference itself runs on a synthetic ramp
image (crates/katsu-core/examples/conv2d/main.rs:5-7).
"""
from __future__ import annotations

import concurrent.futures
import os

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


_CHUNK = 1 << 16  # elements per work item: every temporary of a chunk stays in the core's cache


def _threads() -> int:
    return max(1, min(16, os.cpu_count() or 1))


def _in_chunks(count: int, fill) -> None:
    """Runs fill(first, n) over [0, count) in cache-sized chunks on a few threads (numpy's
    element-wise loops release the interpreter lock).  Whole-array passes over 1e8-element
    temporaries are bound by host memory bandwidth and took minutes for the wide workloads."""
    starts = range(0, count, _CHUNK)
    if count <= _CHUNK:
        for first in starts:
            fill(first, min(_CHUNK, count - first))
        return
    with concurrent.futures.ThreadPoolExecutor(_threads()) as pool:
        list(pool.map(lambda first: fill(first, min(_CHUNK, count - first)), starts))


def _splitmix_block(seed: int, count: int, offset: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = np.arange(offset + 1, offset + count + 1, dtype=np.uint64)
        z *= _GAMMA
        z += np.uint64(seed & 0xFFFFFFFFFFFFFFFF)
        t = z >> np.uint64(30)
        z ^= t
        z *= _M1
        np.right_shift(z, np.uint64(27), out=t)
        z ^= t
        z *= _M2
        np.right_shift(z, np.uint64(31), out=t)
        z ^= t
        z >>= np.uint64(40)
    return z


def splitmix_u24(seed: int, count: int, offset: int = 0) -> np.ndarray:
    """Top 24 bits of SplitMix64 outputs offset+1 .. offset+count of `seed`, as uint64."""
    out = np.empty(count, dtype=np.uint64)

    def fill(first, n):
        out[first:first + n] = _splitmix_block(seed, n, offset + first)

    _in_chunks(count, fill)
    return out


def uniform(seed: int, count: int, lo: float, hi: float, offset: int = 0) -> np.ndarray:
    """f32 values in [lo, hi): lo + (hi - lo) * u with u = bits / 2^24 (exact in f32), for stream
    positions offset .. offset+count-1."""
    out = np.empty(count, dtype=np.float32)

    def fill(first, n):
        u = _splitmix_block(seed, n, offset + first).astype(np.float32) / np.float32(16777216.0)
        out[first:first + n] = np.float32(lo) + np.float32(hi - lo) * u

    _in_chunks(count, fill)
    return out


def normal(seed: int, count: int, std: float, offset: int = 0) -> np.ndarray:
    """f32 N(0, std^2) by Box-Muller on consecutive pairs of the uniform stream: value i uses
    stream positions 2i and 2i+1, so any slice offset .. offset+count-1 is generated on its own."""
    out = np.empty(count, dtype=np.float32)

    def fill(first, n):
        bits = _splitmix_block(seed, 2 * n, 2 * (offset + first)).astype(np.float64)
        bits /= 16777216.0
        u1, u2 = bits[0::2], bits[1::2]
        z = np.sqrt(-2.0 * np.log1p(-u1)) * np.cos(2.0 * np.pi * u2)
        out[first:first + n] = (z * std).astype(np.float32)

    _in_chunks(count, fill)
    return out


def reference_weights(seed: int, count: int, fan_in: int) -> np.ndarray:
    """Conv2D::new_seeded's initialiser, conv2d.rs:46-58."""
    u = splitmix_u24(seed, count).astype(np.float32) / np.float32(16777216.0)
    bound = np.float32(1.0) / np.sqrt(np.float32(fan_in))
    return ((np.float32(2.0) * u - np.float32(1.0)) * bound).astype(np.float32)
