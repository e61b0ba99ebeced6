"""The deterministic generators Tachyon's own unit tests draw their inputs from."""
import numpy as np


def lcg_data(n: int, seed: int) -> np.ndarray:
    """src/kernels.rs:1513-1521: s = s*1664525 + 1013904223; (s>>8)/2^24*2-1."""
    out = np.empty(n, np.float32)
    s = seed & 0xFFFFFFFF
    for i in range(n):
        s = (s * 1664525 + 1013904223) & 0xFFFFFFFF
        out[i] = np.float32(np.float32(s >> 8) / np.float32(1 << 24) * np.float32(2.0) - np.float32(1.0))
    return out


def xorshift_data(n: int, seed: int) -> np.ndarray:
    """src/weights.rs:670-680: xorshift64, (s>>40)/2^23 - 1."""
    m = (1 << 64) - 1
    s = ((seed * 0x9E3779B97F4A7C15) & m) | 1
    out = np.empty(n, np.float32)
    for i in range(n):
        s ^= (s << 13) & m
        s ^= s >> 7
        s ^= (s << 17) & m
        out[i] = np.float32(np.float32(s >> 40) / np.float32(1 << 23) - np.float32(1.0))
    return out
