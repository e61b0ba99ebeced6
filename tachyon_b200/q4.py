"""Tachyon's packed 4-bit quantizer (src/kernels.rs:180-242, 438-495) in numpy,
vectorized over the blocks of a matrix. Produces the same bytes as the
reference's per-row loop; importance is None (as in every workload here)."""
from __future__ import annotations

import numpy as np

from .weights import QK, SUPER, SUPER_WORDS, _round_away_exact, f16_finite, q4_words

F = np.float32


def _seq_sum(a: np.ndarray) -> np.ndarray:
    """Left-to-right float32 sum over the last axis (an iterator `.sum()`)."""
    acc = np.zeros(a.shape[:-1], F)
    for j in range(a.shape[-1]):
        acc = (acc + a[..., j]).astype(F)
    return acc


def _fit_blocks(x: np.ndarray, w: np.ndarray):
    """fit_q4_offset over blocks: x, w are [n, 32]. Returns (d, c) per block."""
    n = x.shape[0]
    lo = x.min(axis=1)
    hi = x.max(axis=1)
    const = hi <= lo
    rng = np.where(const, F(1.0), hi - lo).astype(F)

    def levels_for(iscale):
        l = _round_away_exact(((x - lo[:, None]).astype(F) * iscale[:, None]).astype(F))
        return np.clip(l, 0.0, 15.0).astype(F)

    def err(a, m, l):
        r = ((x - (a[:, None] * l).astype(F)).astype(F) - m[:, None]).astype(F)
        return _seq_sum((w * (r * r).astype(F)).astype(F))

    plain = levels_for((F(15.0) / rng).astype(F))
    best_a = (rng / F(15.0)).astype(F)
    best_m = lo.copy()
    best_e = err(best_a, best_m, plain)
    for step in range(-10, 11):
        l = levels_for(((F(15.0) + F(F(0.1) * F(step))) / rng).astype(F))
        sw = _seq_sum(w)
        sl = _seq_sum((w * l).astype(F))
        sll = _seq_sum(((w * l).astype(F) * l).astype(F))
        sx = _seq_sum((w * x).astype(F))
        slx = _seq_sum(((w * l).astype(F) * x).astype(F))
        det = ((sw * sll).astype(F) - (sl * sl).astype(F)).astype(F)
        ok = det > 0
        safe = np.where(ok, det, F(1.0)).astype(F)
        a = (((sw * slx).astype(F) - (sl * sx).astype(F)).astype(F) / safe).astype(F)
        m = (((sll * sx).astype(F) - (sl * slx).astype(F)).astype(F) / safe).astype(F)
        e = err(a, m, l)
        better = ok & (e < best_e)
        best_a = np.where(better, a, best_a).astype(F)
        best_m = np.where(better, m, best_m).astype(F)
        best_e = np.where(better, e, best_e).astype(F)
    d = np.where(const, F(0.0), best_a).astype(F)
    c = np.where(const, lo, (best_m + (F(8.0) * best_a).astype(F)).astype(F)).astype(F)
    return d, c


def quantize_q4_matrix(data: np.ndarray, rows: int, cols: int):
    """Returns (u32 packed scales [rows*q4_words(cols)], u8 nibbles [rows*cols/2])."""
    x = np.ascontiguousarray(data, F).reshape(rows, cols)
    nb = cols // QK
    supers = -(-nb // SUPER)
    words = q4_words(cols)
    sigma2 = (_seq_sum((x * x).astype(F)) / F(cols)).astype(F)  # per row
    xb = x.reshape(rows, nb, QK)
    w = np.sqrt((sigma2[:, None, None] + (xb * xb).astype(F)).astype(F)).astype(F)
    d, c = _fit_blocks(xb.reshape(-1, QK), w.reshape(-1, QK))
    d = np.maximum(d, F(0.0)).reshape(rows, nb)
    c = c.reshape(rows, nb)
    pad = supers * SUPER - nb
    dpad = np.pad(d, ((0, 0), (0, pad))).reshape(rows, supers, SUPER)
    cpad = np.pad(np.abs(c), ((0, 0), (0, pad))).reshape(rows, supers, SUPER)
    with np.errstate(over="ignore"):
        dh = (dpad.max(axis=2) / F(255.0)).astype(np.float16)
        mh = (cpad.max(axis=2) / F(127.0)).astype(np.float16)
    step_d = np.repeat(f16_finite(dh.view(np.uint16)), SUPER, axis=1)[:, :nb]
    step_c = np.repeat(f16_finite(mh.view(np.uint16)), SUPER, axis=1)[:, :nb]

    def near(v, step, lo, hi):
        safe = np.where(step > 0, step, F(1.0)).astype(F)
        f = np.where(step > 0, np.floor((v / safe).astype(F)), F(0.0)).astype(F)
        return np.clip(f, lo, hi).astype(F), np.clip(f + F(1.0), lo, hi).astype(F)

    s_opts = near(d, step_d, 0.0, 255.0)
    o_opts = near(c, step_c, -128.0, 127.0)
    best_err = np.full((rows, nb), np.inf, F)
    best_s = np.zeros((rows, nb), np.uint32)
    best_o = np.zeros((rows, nb), np.uint32)
    best_l = np.full((rows, nb, QK), 8, np.uint8)
    for s in s_opts:
        for o in o_opts:
            dq = (step_d * s).astype(F)
            cq = (step_c * o).astype(F)
            with np.errstate(divide="ignore"):
                inv = np.where(dq > 0, F(1.0) / np.where(dq > 0, dq, F(1.0)), F(0.0)).astype(F)
            l = _round_away_exact((((xb - cq[..., None]).astype(F) * inv[..., None]).astype(F) + F(8.0)).astype(F))
            l = np.clip(l, 0.0, 15.0).astype(F)
            r = ((xb - (dq[..., None] * (l - F(8.0)).astype(F)).astype(F)).astype(F) - cq[..., None]).astype(F)
            e = _seq_sum((w * (r * r).astype(F)).astype(F))
            better = e < best_err
            best_err = np.where(better, e, best_err)
            best_s = np.where(better, s.astype(np.uint32), best_s)
            best_o = np.where(better, o.astype(np.int32).astype(np.int8).view(np.uint8).astype(np.uint32), best_o)
            best_l = np.where(better[..., None], l.astype(np.uint8), best_l)
    packed = np.zeros((rows, supers, SUPER_WORDS), np.uint32)
    packed[:, :, 0] = dh.view(np.uint16).astype(np.uint32) | (mh.view(np.uint16).astype(np.uint32) << np.uint32(16))
    sp = np.pad(best_s, ((0, 0), (0, pad))).reshape(rows, supers, SUPER)
    op = np.pad(best_o, ((0, 0), (0, pad))).reshape(rows, supers, SUPER)
    for j in range(SUPER):
        packed[:, :, 1 + j // 4] |= sp[:, :, j] << np.uint32(8 * (j % 4))
        packed[:, :, 3 + j // 4] |= op[:, :, j] << np.uint32(8 * (j % 4))
    qs = (best_l[..., : QK // 2] | (best_l[..., QK // 2:] << np.uint8(4))).astype(np.uint8)
    assert packed.reshape(rows, -1).shape[1] == words
    return packed.reshape(-1).copy(), qs.reshape(-1).copy()
