"""ctypes binding of the CPU oracle (``liboracle.so``): TEST INFRASTRUCTURE ONLY.

Only the tests, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs
may import this module. It wraps ``oracle/tachyon_oracle.cpp``, a restatement of
Tachyon's x86-64 CPU path for the Granite MoE block, behind numpy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")

KIND_BF16, KIND_Q8, KIND_Q4 = 0, 1, 2


def build(force: bool = False) -> str:
    """Compiles the oracle with the recipe in ``oracle/Makefile``."""
    src = os.path.join(_HERE, "tachyon_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = C.CDLL(_LIB_PATH)
        _declare(_lib)
    return _lib


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _declare(L: C.CDLL) -> None:
    f32, u16, sz, vp, i32 = C.c_float, C.c_uint16, C.c_size_t, C.c_void_p, C.c_int
    sig = {
        "to_f32_to_bf16": (u16, [f32]),
        "to_f32_to_f16": (u16, [f32]),
        "to_f16_to_f32": (f32, [u16]),
        "to_f16_finite": (f32, [u16]),
        "to_bf16_to_f32": (f32, [u16]),
        "to_exp_scalar": (f32, [f32]),
        "to_exp_many": (None, [vp, sz, vp]),
        "to_libm_exp_many": (None, [vp, sz, vp]),
        "to_quantize_q8": (None, [vp, sz, vp, vp]),
        "to_quantize_q4": (None, [vp, sz, vp, vp]),
        "to_quantize_q8_weights": (None, [vp, sz, vp, vp]),
        "to_q4_words": (sz, [sz]),
        "to_quantize_q4_matrix": (None, [vp, sz, sz, vp, vp, vp, i32]),
        "to_unpack_q4": (None, [vp, sz, vp, vp]),
        "to_dequantize_q8": (None, [vp, vp, sz, vp]),
        "to_dequantize_q4": (None, [vp, vp, sz, vp]),
        "to_dot_f32": (f32, [vp, vp, sz]),
        "to_dot_bf16": (f32, [vp, vp, sz]),
        "to_dot_bf16_scalar": (f32, [vp, vp, sz]),
        "to_dot_q8": (f32, [vp, sz, vp, vp, vp]),
        "to_dot_q8_half": (f32, [vp, sz, vp, vp, vp]),
        "to_dot_q4": (f32, [vp, sz, vp, vp, vp]),
        "to_dot_q4_packed": (f32, [vp, sz, vp, vp, vp]),
        "to_dot_q8_x4": (None, [vp, sz, vp, vp, vp, sz, vp]),
        "to_dot_q4_x4": (None, [vp, sz, vp, vp, vp, sz, vp]),
        "to_dot_q8_scalar": (f32, [vp, sz, vp, vp, vp]),
        "to_dot_q4_scalar": (f32, [vp, sz, vp, vp, vp]),
        "to_dot_offsets": (f32, [vp, vp, sz]),
        "to_dot_offsets_expanded": (f32, [vp, vp, sz]),
        "to_silu_mul": (None, [vp, vp, sz, vp]),
        "to_rmsnorm": (None, [vp, vp, vp, sz, f32]),
        "to_rmsnorm_rows": (None, [vp, vp, vp, sz, sz, f32]),
        "to_axpy": (None, [vp, f32, vp, sz]),
        "to_route": (None, [vp, sz, sz, vp, vp]),
        "to_row_into": (None, [i32, sz, sz, vp, vp, sz, vp]),
        "to_matmul_rows": (None, [i32, sz, sz, vp, vp, vp, sz, vp, sz, sz, i32]),
        "to_quantize_input": (None, [vp, sz, sz, vp, vp]),
        "to_moe": (None, [sz, sz, sz, sz, vp, i32, vp, vp, i32, vp, vp, vp, sz, vp, vp, vp, vp, vp, vp, i32]),
        "to_add_inplace": (None, [vp, vp, sz]),
        "to_default_threads": (i32, []),
        "to_set_arith": (None, [i32]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


# ------------------------------------------------------------------ scalars

def f32_to_bf16(v: float) -> int:
    return lib().to_f32_to_bf16(v)


def f32_to_f16(v: float) -> int:
    return lib().to_f32_to_f16(v)


def f16_to_f32(h: int) -> float:
    return lib().to_f16_to_f32(h)


def f16_finite(h: int) -> float:
    return lib().to_f16_finite(h)


def bf16_to_f32(h: int) -> float:
    return lib().to_bf16_to_f32(h)


def exp_many(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().to_exp_many(_p(x), x.size, _p(out))
    return out


def libm_exp_many(x) -> np.ndarray:
    x = _f32(x)
    out = np.empty_like(x)
    lib().to_libm_exp_many(_p(x), x.size, _p(out))
    return out


# ------------------------------------------------------------------ quantizers

def quantize_q8(x):
    """Activations: (f32 scales per 32-block, int8 values)."""
    x = _f32(x).ravel()
    s = np.empty(x.size // 32, np.float32)
    q = np.empty(x.size, np.int8)
    lib().to_quantize_q8(_p(x), x.size, _p(s), _p(q))
    return s, q


def quantize_q4_symmetric(x):
    x = _f32(x).ravel()
    s = np.empty(x.size // 32, np.float32)
    q = np.empty(x.size // 2, np.uint8)
    lib().to_quantize_q4(_p(x), x.size, _p(s), _p(q))
    return s, q


def quantize_q8_weights(x):
    x = _f32(x).ravel()
    s = np.empty(x.size // 32, np.uint16)
    q = np.empty(x.size, np.int8)
    lib().to_quantize_q8_weights(_p(x), x.size, _p(s), _p(q))
    return s, q


def q4_words(cols: int) -> int:
    return lib().to_q4_words(cols)


def quantize_q4_matrix(data, rows: int, cols: int, importance=None, threads: int = 0):
    data = _f32(data).ravel()
    words = q4_words(cols)
    s = np.zeros(rows * words, np.uint32)
    q = np.zeros(rows * cols // 2, np.uint8)
    imp = None if importance is None else _f32(importance)
    lib().to_quantize_q4_matrix(_p(data), rows, cols, _p(imp), _p(s), _p(q), threads or default_threads())
    return s, q


def unpack_q4(packed, nb: int):
    packed = np.ascontiguousarray(packed, np.uint32)
    d = np.zeros(nb, np.float32)
    c = np.zeros(nb, np.float32)
    lib().to_unpack_q4(_p(packed), nb, _p(d), _p(c))
    return d, c


def dequantize_q8(scales, qs) -> np.ndarray:
    scales, qs = _f32(scales), np.ascontiguousarray(qs, np.int8)
    out = np.empty(qs.size, np.float32)
    lib().to_dequantize_q8(_p(scales), _p(qs), qs.size, _p(out))
    return out


def dequantize_q4(scales, qs) -> np.ndarray:
    scales, qs = _f32(scales), np.ascontiguousarray(qs, np.uint8)
    out = np.empty(qs.size * 2, np.float32)
    lib().to_dequantize_q4(_p(scales), _p(qs), qs.size * 2, _p(out))
    return out


# ------------------------------------------------------------------ dots

def dot_f32(a, b) -> float:
    a, b = _f32(a), _f32(b)
    return lib().to_dot_f32(_p(a), _p(b), min(a.size, b.size))


def dot_bf16(w, x, scalar: bool = False) -> float:
    w, x = np.ascontiguousarray(w, np.uint16), _f32(x)
    fn = lib().to_dot_bf16_scalar if scalar else lib().to_dot_bf16
    return fn(_p(w), _p(x), min(w.size, x.size))


def dot_q8(ws, wq, xs, xq, scalar: bool = False) -> float:
    wq, xs, xq = np.ascontiguousarray(wq, np.int8), _f32(xs), np.ascontiguousarray(xq, np.int8)
    if np.asarray(ws).dtype == np.uint16:
        ws = np.ascontiguousarray(ws, np.uint16)
        return lib().to_dot_q8_half(_p(ws), ws.size, _p(wq), _p(xs), _p(xq))
    ws = _f32(ws)
    fn = lib().to_dot_q8_scalar if scalar else lib().to_dot_q8
    return fn(_p(ws), ws.size, _p(wq), _p(xs), _p(xq))


def dot_q4(ws, wq, xs, xq, scalar: bool = False) -> float:
    ws, wq = _f32(ws), np.ascontiguousarray(wq, np.uint8)
    xs, xq = _f32(xs), np.ascontiguousarray(xq, np.int8)
    fn = lib().to_dot_q4_scalar if scalar else lib().to_dot_q4
    return fn(_p(ws), ws.size, _p(wq), _p(xs), _p(xq))


def dot_q4_packed(words, nb, wq, xs, xq) -> float:
    words, wq = np.ascontiguousarray(words, np.uint32), np.ascontiguousarray(wq, np.uint8)
    xs, xq = _f32(xs), np.ascontiguousarray(xq, np.int8)
    return lib().to_dot_q4_packed(_p(words), nb, _p(wq), _p(xs), _p(xq))


def dot_q8_x4(ws, wq, xs4, xq4) -> np.ndarray:
    ws, wq = _f32(ws), np.ascontiguousarray(wq, np.int8)
    xs4, xq4 = _f32(xs4), np.ascontiguousarray(xq4, np.int8)
    out = np.empty(4, np.float32)
    lib().to_dot_q8_x4(_p(ws), ws.size, _p(wq), _p(xs4), _p(xq4), ws.size * 32, _p(out))
    return out


def dot_q4_x4(ws, wq, xs4, xq4) -> np.ndarray:
    ws, wq = _f32(ws), np.ascontiguousarray(wq, np.uint8)
    xs4, xq4 = _f32(xs4), np.ascontiguousarray(xq4, np.int8)
    out = np.empty(4, np.float32)
    lib().to_dot_q4_x4(_p(ws), ws.size, _p(wq), _p(xs4), _p(xq4), ws.size * 32, _p(out))
    return out


def dot_offsets(words, sums) -> float:
    words, sums = np.ascontiguousarray(words, np.uint32), _f32(sums)
    return lib().to_dot_offsets(_p(words), _p(sums), sums.size)


def dot_offsets_expanded(c, sums) -> float:
    c, sums = _f32(c), _f32(sums)
    return lib().to_dot_offsets_expanded(_p(c), _p(sums), sums.size)


# ------------------------------------------------------------------ elementwise

def silu_mul(g, u) -> np.ndarray:
    g, u = _f32(g), _f32(u)
    out = np.empty_like(g)
    lib().to_silu_mul(_p(g), _p(u), g.size, _p(out))
    return out


def rmsnorm_rows(x, w, eps: float) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    t, n = x.shape
    out = np.empty_like(x)
    lib().to_rmsnorm_rows(_p(out), _p(x), _p(w), t, n, eps)
    return out


def route(scores, k: int):
    scores = _f32(scores)
    k = min(k, scores.size)
    ids = np.empty(k, np.uint32)
    gates = np.empty(k, np.float32)
    lib().to_route(_p(scores), scores.size, k, _p(ids), _p(gates))
    return ids, gates


class fast_arithmetic_model:
    """Context manager: inside it, quantized matmuls (and so ``moe``) use the
    single-fma-chain order of the CUDA backend's fast kernels instead of the
    reference's eight-lane order. A model of the GPU, not of Tachyon."""

    def __enter__(self):
        lib().to_set_arith(1)

    def __exit__(self, *exc):
        lib().to_set_arith(0)


def default_threads() -> int:
    return lib().to_default_threads()


# ------------------------------------------------------------------ matrices

@dataclass
class OracleMatrix:
    """The buffers of Tachyon's ``Matrix`` enum (src/weights.rs:58-79)."""

    kind: int
    rows: int
    cols: int
    scales: np.ndarray | None  # Q8: u16[rows*cols/32]; Q4: u32[rows*q4_words]; BF16: None
    data: np.ndarray  # BF16: u16; Q8: i8; Q4: u8 (two values per byte)

    @staticmethod
    def from_f32(data, rows: int, cols: int, fmt: str, threads: int = 0) -> "OracleMatrix":
        """``Matrix::from_f32`` (src/weights.rs:82-105); fmt is bf16, q8 or q4."""
        data = _f32(data).reshape(rows * cols)
        if cols % 32 != 0:
            fmt = "bf16"
        if fmt == "bf16":
            # Round to nearest even on the bit pattern (src/kernels.rs:21-28).
            bits = data.view(np.uint32)
            rnd = np.uint32(0x7FFF) + ((bits >> np.uint32(16)) & np.uint32(1))
            out = ((bits + rnd) >> np.uint32(16)).astype(np.uint16)
            out[np.isnan(data)] = 0x7FC0
            return OracleMatrix(KIND_BF16, rows, cols, None, out)
        if fmt == "q8":
            s, q = quantize_q8_weights(data)
            return OracleMatrix(KIND_Q8, rows, cols, s, q)
        if fmt == "q4":
            s, q = quantize_q4_matrix(data, rows, cols, None, threads)
            return OracleMatrix(KIND_Q4, rows, cols, s, q)
        raise ValueError(fmt)

    def row(self, r: int) -> np.ndarray:
        out = np.empty(self.cols, np.float32)
        lib().to_row_into(self.kind, self.rows, self.cols, _p(self.scales), _p(self.data), r, _p(out))
        return out

    def matmul_rows(self, x, row0: int = 0, rows: int | None = None, threads: int = 1) -> np.ndarray:
        """``Matrix::matmul_rows``: x is [t, cols]; returns [t, rows]."""
        x = _f32(x).reshape(-1, self.cols)
        rows = self.rows - row0 if rows is None else rows
        out = np.zeros((x.shape[0], rows), np.float32)
        lib().to_matmul_rows(self.kind, self.rows, self.cols, _p(self.scales), _p(self.data), _p(x),
                             x.shape[0], _p(out), row0, rows, threads)
        return out


def quantize_input(x, cols: int):
    x = _f32(x).reshape(-1, cols)
    t = x.shape[0]
    xs = np.empty((t, cols // 32), np.float32)
    xq = np.empty((t, cols), np.int8)
    lib().to_quantize_input(_p(x), t, cols, _p(xs), _p(xq))
    return xs, xq


@dataclass
class MoeResult:
    proj: np.ndarray  # [t, hidden], what the block adds to the residual
    logits: np.ndarray  # [t, experts] (after the optional bias)
    ids: np.ndarray  # [t, k] descending score order
    gates: np.ndarray  # [t, k]
    counts: np.ndarray  # [experts]


def moe(router: OracleMatrix, gate_up: OracleMatrix, down: OracleMatrix, xb, k: int,
        router_bias=None, threads: int = 1) -> MoeResult:
    """The MoE block (src/model.rs:462-521) over normed inputs ``xb[t, hidden]``."""
    hidden, experts = router.cols, router.rows
    inter = down.cols
    assert router.kind == KIND_BF16
    assert gate_up.rows == experts * 2 * inter and gate_up.cols == hidden
    assert down.rows == experts * hidden
    xb = _f32(xb).reshape(-1, hidden)
    t = xb.shape[0]
    bias = None if router_bias is None else _f32(router_bias)
    proj = np.zeros((t, hidden), np.float32)
    logits = np.zeros((t, experts), np.float32)
    ids = np.zeros((t, k), np.uint32)
    gates = np.zeros((t, k), np.float32)
    counts = np.zeros(experts, np.uint32)
    lib().to_moe(hidden, experts, k, inter, _p(router.data), gate_up.kind, _p(gate_up.scales),
                 _p(gate_up.data), down.kind, _p(down.scales), _p(down.data), _p(xb), t, _p(bias),
                 _p(proj), _p(logits), _p(ids), _p(gates), _p(counts), threads)
    return MoeResult(proj, logits, ids, gates, counts)
