"""Pins the CPU oracle to the known-answer and property tests Tachyon keeps
beside the code the oracle restates. Each test names the reference test it
restates (paths relative to the Tachyon project root)."""
import math

import numpy as np
import pytest

from refgen import lcg_data, xorshift_data

QK = 32


def test_route_known_answer(oracle):
    # src/model.rs:790-798
    ids, gates = oracle.route([0.5, 3.0, -1.0, 3.0, 2.0], 3)
    assert ids.tolist() == [1, 3, 4]  # ties go to the lower expert
    assert abs(float(gates.sum()) - 1.0) < 1e-6
    assert abs(gates[0] / gates[2] - math.exp(1.0)) < 1e-5


def test_route_orders_like_total_cmp(oracle):
    # total_cmp: -NaN < -inf < ... < -0 < +0 < ... < +inf < +NaN
    scores = np.array([0.0, -0.0, np.inf, -np.inf, 1.0, 1.0], np.float32)
    ids, _ = oracle.route(scores, 6)
    assert ids.tolist() == [2, 4, 5, 0, 1, 3]


def test_half_floats(oracle):
    # src/kernels.rs:1788-1810
    assert oracle.bf16_to_f32(oracle.f32_to_bf16(1.5)) == 1.5
    assert oracle.f16_to_f32(0x3C00) == 1.0
    assert oracle.f16_to_f32(0xC000) == -2.0
    assert oracle.f16_to_f32(0x0001) == 2.0 ** -24
    for v, h in [
        (1.0, 0x3C00),
        (-2.0, 0xC000),
        (65504.0, 0x7BFF),
        (65520.0, 0x7C00),
        (2.0 ** -24, 0x0001),
        (2.0 ** -14, 0x0400),
        (1.0 + 2.0 ** -11, 0x3C00),
        (1.0 + 3.0 * 2.0 ** -11, 0x3C02),
    ]:
        assert oracle.f32_to_f16(v) == h, v
    x = lcg_data(1000, 3)
    for v in x:
        v100 = float(np.float32(v) * np.float32(100.0))
        assert abs(oracle.f16_to_f32(oracle.f32_to_f16(v100)) - v100) <= 0.05


def test_f16_finite_equals_f16_to_f32_on_every_finite_half(oracle):
    # src/kernels.rs:1734-1742
    for h in range(0x7C00):
        a, b = oracle.f16_finite(h), oracle.f16_to_f32(h)
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32)
        a, b = oracle.f16_finite(h | 0x8000), oracle.f16_to_f32(h | 0x8000)
        assert np.float32(a).view(np.uint32) == np.float32(b).view(np.uint32)


def test_f16_matches_numpy_half(oracle):
    # numpy's float16 is IEEE binary16 with round-to-nearest-even: an
    # independent statement of the same conversion.
    x = (lcg_data(4000, 77).astype(np.float64) * 10.0 ** np.linspace(-9, 5, 4000)).astype(np.float32)
    got = np.array([oracle.f32_to_f16(float(v)) for v in x], np.uint16)
    assert np.array_equal(got, x.astype(np.float16).view(np.uint16))


def test_simd_matches_scalar(oracle):
    # src/kernels.rs:1523-1552
    a, b = lcg_data(896, 1), lcg_data(896, 2)
    exact = np.float32(0)
    for x, y in zip(a, b):
        exact = np.float32(exact + np.float32(x * y))
    assert abs(oracle.dot_f32(a, b) - exact) < 1e-3
    wb = np.array([oracle.f32_to_bf16(float(v)) for v in a], np.uint16)
    assert abs(oracle.dot_bf16(wb, b) - oracle.dot_bf16(wb, b, scalar=True)) < 1e-3
    ws, wq = oracle.quantize_q8(a)
    xs, xq = oracle.quantize_q8(b)
    q8 = oracle.dot_q8(ws, wq, xs, xq)
    assert abs(q8 - oracle.dot_q8(ws, wq, xs, xq, scalar=True)) < 1e-3
    assert abs(q8 - exact) < 0.05 * max(abs(exact), 1.0)
    ws4, w4 = oracle.quantize_q4_symmetric(a)
    q4 = oracle.dot_q4(ws4, w4, xs, xq)
    assert abs(q4 - oracle.dot_q4(ws4, w4, xs, xq, scalar=True)) < 1e-3


def test_four_token_dots_match_single_dots_bit_for_bit(oracle):
    # src/kernels.rs:1554-1581
    cols = 896
    w = lcg_data(cols, 21)
    ws, wq8 = oracle.quantize_q8(w)
    ws4, wq4 = oracle.quantize_q4_symmetric(w)
    xs4 = np.empty((4, cols // QK), np.float32)
    xq4 = np.empty((4, cols), np.int8)
    for j in range(4):
        xs4[j], xq4[j] = oracle.quantize_q8(lcg_data(cols, 30 + j))
    q8 = oracle.dot_q8_x4(ws, wq8, xs4, xq4)
    q4 = oracle.dot_q4_x4(ws4, wq4, xs4, xq4)
    for j in range(4):
        assert q8[j] == np.float32(oracle.dot_q8(ws, wq8, xs4[j], xq4[j]))
        assert q4[j] == np.float32(oracle.dot_q4(ws4, wq4, xs4[j], xq4[j]))
        assert abs(q8[j] - oracle.dot_q8(ws, wq8, xs4[j], xq4[j], scalar=True)) < 1e-3
        assert abs(q4[j] - oracle.dot_q4(ws4, wq4, xs4[j], xq4[j], scalar=True)) < 1e-3


def test_quantizers_round_trip(oracle):
    # src/kernels.rs:1651-1668
    x = lcg_data(256, 7)
    s, q8 = oracle.quantize_q8(x)
    assert np.all(np.abs(x - oracle.dequantize_q8(s, q8)) <= 1.0 / 127.0)
    s, q4 = oracle.quantize_q4_symmetric(x)
    assert np.all(np.abs(x - oracle.dequantize_q4(s, q4)) <= 1.0 / 8.0 + 1e-6)


def test_exp_is_within_two_ulp(oracle):
    # src/kernels.rs:1722-1732
    xs = (np.float32(-87.0) + np.arange(200_000, dtype=np.float32) * np.float32(0.000875)).astype(np.float32)
    xs = np.concatenate([xs, np.array([0.0, -0.0, 1.0, -1e-30, -50.5, -87.3], np.float32)])
    want = oracle.libm_exp_many(xs)
    got = oracle.exp_many(xs)
    ulps = np.abs(got.view(np.int32).astype(np.int64) - want.view(np.int32).astype(np.int64))
    assert ulps.max() <= 2


def _packed_dequant(oracle, x):
    nb = x.size // QK
    s, q = oracle.quantize_q4_matrix(x, 1, x.size)
    d, c = oracle.unpack_q4(s, nb)
    out = oracle.dequantize_q4(d, q)
    return out + np.repeat(c, QK), d, c, s, q


def test_packed_q4_round_trip_partial_super_block_and_constant_blocks(oracle):
    # src/kernels.rs:1743-1786
    x = lcg_data(11 * QK, 5)
    x[3 * QK:4 * QK] = 0.25
    x[9 * QK:10 * QK] = 0.0
    out, d, c, s, q = _packed_dequant(oracle, x)
    assert s.size == 2 * 5
    assert np.all(out[9 * QK:10 * QK] == 0.0)
    assert np.all(np.abs(out[3 * QK:4 * QK] - 0.25) < 0.01)
    rms = math.sqrt(float(np.mean(x.astype(np.float64) ** 2)))
    err = math.sqrt(float(np.mean((x.astype(np.float64) - out) ** 2)))
    assert err < rms * 0.12
    s8, q8 = oracle.quantize_q8_weights(x)
    ds = np.array([oracle.f16_finite(int(h)) for h in s8], np.float32)
    assert np.all(np.abs(x - oracle.dequantize_q8(ds, q8)) <= 0.5 / 127.0 + 1e-3)


def test_offset_q4_beats_symmetric_q4_on_its_own_measure(oracle):
    # src/kernels.rs:1670-1720 (the importance=None arm, which the workloads use)
    x = lcg_data(64 * QK, 11)
    sigma2 = np.float32(np.sum(x * x, dtype=np.float32) / np.float32(x.size))
    w = np.sqrt(sigma2 + x * x)

    def werr(out):
        return float(np.sum(w * (x - out) ** 2))

    s, q = oracle.quantize_q4_symmetric(x)
    sym = oracle.dequantize_q4(s, q)
    out, *_ = _packed_dequant(oracle, x)
    assert werr(out) < werr(sym) * 0.8


@pytest.mark.parametrize("fmt", ["q8", "q4"])
def test_matmul_matches_dequantized_rows_and_is_batch_invariant(oracle, fmt):
    # src/weights.rs:685-731: every path through the integer matmul (fours,
    # leftovers, single token, row chunks) gives the dequantized row times the
    # token's 8-bit activations, and a token alone gives exactly its result in
    # a batch.
    rows, cols = 37, 11 * QK
    w = xorshift_data(rows * cols, 1)
    m = oracle.OracleMatrix.from_f32(w, rows, cols, fmt)
    deq = np.stack([m.row(r) for r in range(rows)])
    for t in [1, 2, 3, 5, 8, 9]:
        x = xorshift_data(t * cols, t + 7).reshape(t, cols)
        out = m.matmul_rows(x, threads=3)
        xs, xq = oracle.quantize_input(x, cols)
        xd = oracle.dequantize_q8(xs.ravel(), xq.ravel()).reshape(t, cols)
        for i in range(t):
            alone = m.matmul_rows(x[i:i + 1], threads=3)
            assert np.array_equal(alone[0], out[i]), (fmt, t, i)
        for i in range(t):
            for r in range(rows):
                want = np.float32(0)
                for a, b in zip(deq[r], xd[i]):
                    want = np.float32(want + np.float32(a * b))
                assert abs(out[i, r] - want) < 1e-4, (fmt, t, i, r)


def test_matmul_rows_subrange_equals_full(oracle):
    # Matrix::matmul_rows over an expert's row range (src/weights.rs:214-225)
    rows, cols = 48, 4 * QK
    w = xorshift_data(rows * cols, 3)
    x = xorshift_data(5 * cols, 4).reshape(5, cols)
    for fmt in ["q8", "q4", "bf16"]:
        m = oracle.OracleMatrix.from_f32(w, rows, cols, fmt)
        full = m.matmul_rows(x, threads=2)
        part = m.matmul_rows(x, row0=16, rows=16, threads=2)
        assert np.array_equal(full[:, 16:32], part)


def test_threads_do_not_change_results(oracle):
    rows, cols = 64, 8 * QK
    w = xorshift_data(rows * cols, 5)
    x = xorshift_data(7 * cols, 6).reshape(7, cols)
    for fmt in ["q8", "q4"]:
        m = oracle.OracleMatrix.from_f32(w, rows, cols, fmt)
        assert np.array_equal(m.matmul_rows(x, threads=1), m.matmul_rows(x, threads=6))
