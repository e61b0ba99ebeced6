"""Host-side mirror of Tachyon's ``Matrix`` (src/weights.rs:58-126): the three
storage formats, built from float32 data with numpy, in the byte layout the
CUDA backend uploads unchanged.

  bf16: u16[rows*cols], round to nearest even          (src/kernels.rs:21-28)
  q8:   f16 scale per 32 weights + int8 values         (src/kernels.rs:135-149)
  q4:   packed 4-bit with per-block scale and offset   (src/kernels.rs:180-242)
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

QK = 32
SUPER = 8
SUPER_WORDS = 5
KIND_BF16, KIND_Q8, KIND_Q4 = 0, 1, 2
KIND_NAMES = {KIND_BF16: "bf16", KIND_Q8: "q8", KIND_Q4: "q4"}


def q4_words(cols: int) -> int:
    """Words of packed 4-bit scales per row (src/weights.rs:276-278)."""
    return -(-(cols // QK) // SUPER) * SUPER_WORDS


def f32_to_bf16(data: np.ndarray) -> np.ndarray:
    data = np.ascontiguousarray(data, np.float32)
    bits = data.view(np.uint32)
    rnd = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
    with np.errstate(over="ignore"):
        out = ((bits + rnd) >> np.uint32(16)).astype(np.uint16)
    out[np.isnan(data)] = 0x7FC0
    return out


def bf16_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def round_half_away(v: np.ndarray) -> np.ndarray:
    """f32::round: halfway cases away from zero (numpy's rint rounds them to even)."""
    return np.copysign(np.floor(np.abs(v) + np.float32(0.5)), v).astype(np.float32)


def _round_away_exact(v: np.ndarray) -> np.ndarray:
    # floor(|v| + 0.5) is wrong when |v| + 0.5 rounds up in float32 (|v| just
    # below a half); truncation plus a comparison of the exact remainder is not.
    a = np.abs(v)
    t = np.trunc(a)
    t = t + ((a - t) >= np.float32(0.5)).astype(np.float32)
    return np.copysign(t, v).astype(np.float32)


def f16_finite(h: np.ndarray) -> np.ndarray:
    """src/kernels.rs:127-130: half bits shifted into place, times 2^112. Equal
    to the IEEE conversion on every finite half; on inf/NaN bits it gives the
    finite value the reference computes, which the 8-bit quantizer then uses."""
    h = np.asarray(h, np.uint16).astype(np.uint32)
    bits = ((h & np.uint32(0x8000)) << np.uint32(16)) | ((h & np.uint32(0x7FFF)) << np.uint32(13))
    return (bits.view(np.float32) * np.float32(2.0 ** 112)).astype(np.float32)


def quantize_q8_weights(data: np.ndarray):
    """(f16 scales as u16, int8 values) of ``quantize_q8_weights``."""
    x = np.ascontiguousarray(data, np.float32).reshape(-1, QK)
    amax = np.max(np.abs(x), axis=1)
    with np.errstate(over="ignore"):
        h = (amax / np.float32(127.0)).astype(np.float16)
    d = f16_finite(h.view(np.uint16))
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    with np.errstate(over="ignore"):
        q = _round_away_exact(x * inv[:, None])
    q = np.clip(q, -127.0, 127.0).astype(np.int8)
    return h.view(np.uint16).copy(), q.reshape(-1)


def quantize_q8_activations(data: np.ndarray):
    """(f32 scales, int8 values) of ``quantize_q8`` (src/kernels.rs:84-98)."""
    x = np.ascontiguousarray(data, np.float32).reshape(-1, QK)
    amax = np.max(np.abs(x), axis=1)
    d = (amax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0, np.float32(1.0) / d, np.float32(0.0)).astype(np.float32)
    q = np.clip(_round_away_exact(x * inv[:, None]), -128.0, 127.0).astype(np.int8)
    return d, q.reshape(-1)


@dataclass
class Matrix:
    kind: int
    rows: int
    cols: int
    scales: np.ndarray | None
    data: np.ndarray

    @staticmethod
    def from_f32(data, rows: int, cols: int, fmt: str) -> "Matrix":
        """``Matrix::from_f32`` (src/weights.rs:82-105)."""
        data = np.ascontiguousarray(data, np.float32).reshape(rows * cols)
        fmt = fmt.lower()
        if cols % QK != 0:
            fmt = "bf16"  # quantized blocks must not straddle rows
        if fmt == "bf16":
            return Matrix(KIND_BF16, rows, cols, None, f32_to_bf16(data))
        if fmt in ("q8", "int8"):
            s, q = quantize_q8_weights(data)
            return Matrix(KIND_Q8, rows, cols, s, q)
        if fmt in ("q4", "int4"):
            from .q4 import quantize_q4_matrix

            s, q = quantize_q4_matrix(data, rows, cols)
            return Matrix(KIND_Q4, rows, cols, s, q)
        raise ValueError(f"unknown format {fmt!r}")

    def nbytes(self) -> int:
        """``Matrix::bytes`` (src/weights.rs:166-172)."""
        return self.data.nbytes + (0 if self.scales is None else self.scales.nbytes)
