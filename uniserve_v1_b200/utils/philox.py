"""Philox4x32-10 addressed by (seed, position, stage, draw) in pure Python.

Bit-for-bit the same function as ``csrc/include/us_philox.h`` so the CPU
reference sampler, the scheduler and the CUDA kernels agree on every draw.
A draw depends on (seed, position) only: not on the batch, the rank, a graph
replay or a migration (reference behaviour:
crates/engine/src/batch/philox.rs:18-35, reference project path).
"""
from __future__ import annotations

import math

M32 = 0xFFFFFFFF
M64 = 0xFFFFFFFFFFFFFFFF


def splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & M64
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M64
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M64
    return x ^ (x >> 31)


def philox4x32_10(seed: int, position: int, stage: int = 0, draw: int = 0):
    k = splitmix64(seed & M64)
    k0, k1 = k & M32, (k >> 32) & M32
    c0, c1, c2, c3 = position & M32, (position >> 32) & M32, stage & M32, draw & M32
    for _ in range(10):
        p0 = 0xD2511F53 * c0
        p1 = 0xCD9E8D57 * c2
        hi0, lo0 = (p0 >> 32) & M32, p0 & M32
        hi1, lo1 = (p1 >> 32) & M32, p1 & M32
        c0, c1, c2, c3 = hi1 ^ c1 ^ k0, lo1, hi0 ^ c3 ^ k1, lo0
        k0 = (k0 + 0x9E3779B9) & M32
        k1 = (k1 + 0xBB67AE85) & M32
    return c0, c1, c2, c3


def philox_uniform(seed: int, position: int, stage: int = 0, draw: int = 0) -> float:
    """One uniform in [0, 1): the top 24 bits of word 0."""
    return (philox4x32_10(seed, position, stage, draw)[0] >> 8) / 16777216.0


def philox_normal2(seed: int, position: int, stage: int = 0, draw: int = 0):
    """Two standard normals by Box-Muller from words 0 and 1."""
    w = philox4x32_10(seed, position, stage, draw)
    u0 = ((w[0] >> 8) + 0.5) / 16777216.0
    u1 = ((w[1] >> 8) + 0.5) / 16777216.0
    r = math.sqrt(-2.0 * math.log(u0))
    return r * math.cos(2 * math.pi * u1), r * math.sin(2 * math.pi * u1)
