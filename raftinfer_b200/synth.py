"""Deterministic synthetic operands for the parity tests and the benchmark.

Element i of tensor k under seed s is  z(splitmix64(s ^ (k << 40) ^ i)):  the two 32-bit halves of
the hash feed one Box-Muller draw, giving N(0,1) as float32.  The same routine runs wherever the
operands are needed (host side of the tests, fixture generation), so every party sees identical bits.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        x = ((x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        x = ((x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return x ^ (x >> np.uint64(31))


def normal(seed: int, tensor_id: int, shape, chunk: int = 1 << 22) -> np.ndarray:
    """N(0,1) float32 tensor of `shape`, reproducible from (seed, tensor_id)."""
    n = int(np.prod(shape))
    out = np.empty(n, dtype=np.float32)
    key = np.uint64((seed ^ (tensor_id << 40)) & 0xFFFFFFFFFFFFFFFF)
    for start in range(0, n, chunk):
        stop = min(n, start + chunk)
        idx = np.arange(start, stop, dtype=np.uint64) ^ key
        h = _splitmix64(idx)
        hi = (h >> np.uint64(32)).astype(np.float64)
        lo = (h & np.uint64(0xFFFFFFFF)).astype(np.float64)
        u1 = (hi + 1.0) / 4294967296.0
        u2 = lo / 4294967296.0
        out[start:stop] = (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)).astype(np.float32)
    return out.reshape(shape)


def round_bf16(a: np.ndarray) -> np.ndarray:
    """float32 -> nearest-even bfloat16 -> float32 (finite inputs)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    rounded = (bits + np.uint32(0x7FFF) + lsb) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32)


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns (uint16), nearest even (finite inputs)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    lsb = (bits >> np.uint32(16)) & np.uint32(1)
    return ((bits + np.uint32(0x7FFF) + lsb) >> np.uint32(16)).astype(np.uint16)


def softplus(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, dtype=np.float64)
    return np.where(x > 20.0, x, np.log1p(np.exp(np.minimum(x, 20.0)))).astype(np.float32)


def sigmoid(x: np.ndarray) -> np.ndarray:
    return (1.0 / (1.0 + np.exp(-np.asarray(x, dtype=np.float64)))).astype(np.float32)
