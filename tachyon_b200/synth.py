"""Seeded synthetic tensors for the Granite-MoE workloads.

Counter-based, so any slice of any tensor can be regenerated on any machine:
``z = splitmix64(seed * 2**32 + stream + 16 * layer)``; element ``i`` draws
``r = splitmix64(z + i)``, splits it into two 32-bit uniforms and applies
Box-Muller in float64, rounded to float32. Streams: 1 hidden states, 2 router,
3 gate_up, 4 down, 5 token ids, 6 the routing-skew permutation.
"""
from __future__ import annotations

import numpy as np

STREAM_HIDDEN, STREAM_ROUTER, STREAM_GATE_UP, STREAM_DOWN, STREAM_IDS, STREAM_SKEW = 1, 2, 3, 4, 5, 6

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(z):
    """One splitmix64 output per input word (numpy uint64, wrapping)."""
    z = np.asarray(z, dtype=np.uint64)
    with np.errstate(over="ignore"):
        z = z + np.uint64(0x9E3779B97F4A7C15)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def _base(seed: int, stream: int, layer: int) -> np.uint64:
    word = (seed * (1 << 32) + stream + 16 * layer) & 0xFFFFFFFFFFFFFFFF
    return splitmix64(np.uint64(word))


def raw_words(seed: int, stream: int, n: int, layer: int = 0, start: int = 0) -> np.ndarray:
    base = _base(seed, stream, layer)
    with np.errstate(over="ignore"):
        return splitmix64(base + np.arange(start, start + n, dtype=np.uint64))


def normal(seed: int, stream: int, n: int, layer: int = 0, scale: float = 1.0, start: int = 0,
           chunk: int = 1 << 22) -> np.ndarray:
    """n draws of N(0, scale^2) as float32."""
    out = np.empty(n, np.float32)
    for lo in range(0, n, chunk):
        hi = min(n, lo + chunk)
        r = raw_words(seed, stream, hi - lo, layer, start + lo)
        u1 = ((r >> np.uint64(32)).astype(np.float64) + 1.0) * (1.0 / 4294967296.0)
        u2 = (r & np.uint64(0xFFFFFFFF)).astype(np.float64) * (1.0 / 4294967296.0)
        z = np.sqrt(-2.0 * np.log(u1)) * np.cos((2.0 * np.pi) * u2)
        if scale != 1.0:
            z *= scale
        out[lo:hi] = z.astype(np.float32)
    return out


def token_ids(seed: int, n: int, vocab: int) -> np.ndarray:
    """Token ids uniform over the vocabulary."""
    return (raw_words(seed, STREAM_IDS, n) % np.uint64(vocab)).astype(np.uint32)


def zipf_router_bias(seed: int, experts: int, s: float = 1.2) -> np.ndarray:
    """log of a Zipf(s) popularity over a seeded permutation of the experts."""
    order = np.argsort(raw_words(seed, STREAM_SKEW, experts), kind="stable")
    p = np.empty(experts, np.float64)
    p[order] = np.arange(1, experts + 1, dtype=np.float64) ** (-s)
    p /= p.sum()
    return np.log(p).astype(np.float32)
