"""The synthetic Granite-MoE workloads: shapes, seeded weights and inputs.

Weights are N(0, 0.02^2) draws (``synth.normal``) put through the host mirror
of Tachyon's quantizers; the router stays bf16 (src/model.rs:189-195). Hidden
states are N(0, 1) and, where a workload says "after RMSNorm", normed by the
device kernel or the oracle, not here.
"""
from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass

import numpy as np

from . import synth
from .weights import Matrix


@dataclass(frozen=True)
class MoeShape:
    name: str
    hidden: int
    experts: int
    topk: int
    inter: int
    layers: int = 1
    fmt: str = "q8"


# Shapes of the five workloads (hidden, experts, top-k, expert intermediate).
GRANITE_1B = MoeShape("granite-1b-a400m", 1024, 32, 8, 512, layers=24, fmt="q8")
GRANITE_3B = MoeShape("granite-3b-a800m", 1536, 40, 8, 512, layers=32, fmt="q4")
GRANITE_3B_Q8 = MoeShape("granite-3b-a800m-q8", 1536, 40, 8, 512, layers=32, fmt="q8")
SKEW = MoeShape("skew-h2048-e64", 2048, 64, 8, 1024, layers=1, fmt="q8")


@dataclass
class LayerWeights:
    router: Matrix
    gate_up: Matrix
    down: Matrix


def _normal_matrix(seed, stream, layer, rows, cols, fmt, threads=1):
    n = rows * cols
    if threads <= 1 or n < (1 << 22):
        data = synth.normal(seed, stream, n, layer, scale=0.02)
    else:
        data = np.empty(n, np.float32)
        step = -(-n // threads)
        step = -(-step // 4096) * 4096

        def part(lo):
            hi = min(n, lo + step)
            data[lo:hi] = synth.normal(seed, stream, hi - lo, layer, scale=0.02, start=lo)

        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(part, range(0, n, step)))
    if fmt == "q8" and threads > 1 and n >= (1 << 22):
        # Blocks are independent: quantize row ranges on the thread pool.
        from .weights import KIND_Q8, quantize_q8_weights

        scales = np.empty(n // 32, np.uint16)
        qs = np.empty(n, np.int8)
        step = -(-rows // threads) * cols

        def quant(lo):
            hi = min(n, lo + step)
            s, q = quantize_q8_weights(data[lo:hi])
            scales[lo // 32:hi // 32] = s
            qs[lo:hi] = q

        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(quant, range(0, n, step)))
        return Matrix(KIND_Q8, rows, cols, scales, qs)
    return Matrix.from_f32(data, rows, cols, fmt)


def layer_weights(shape: MoeShape, seed: int = 0, layer: int = 0, fmt: str | None = None,
                  threads: int = 1) -> LayerWeights:
    fmt = fmt or shape.fmt
    h, e, i = shape.hidden, shape.experts, shape.inter
    return LayerWeights(
        router=_normal_matrix(seed, synth.STREAM_ROUTER, layer, e, h, "bf16"),
        gate_up=_normal_matrix(seed, synth.STREAM_GATE_UP, layer, e * 2 * i, h, fmt, threads),
        down=_normal_matrix(seed, synth.STREAM_DOWN, layer, e * h, i, fmt, threads),
    )


def layer_weights_local(shape: MoeShape, first: int, count: int, seed: int = 0, layer: int = 0,
                        fmt: str | None = None, threads: int = 1) -> LayerWeights:
    """The full router and experts [first, first+count) of a layer: the same values
    ``layer_weights`` gives for those rows (the generator is counter-based)."""
    fmt = fmt or shape.fmt
    h, e, i = shape.hidden, shape.experts, shape.inter

    def rows(stream, rows_per_expert, cols):
        n = count * rows_per_expert * cols
        start = first * rows_per_expert * cols
        data = np.empty(n, np.float32)
        step = max(1 << 20, -(-n // max(1, threads)))
        step = -(-step // 4096) * 4096

        def part(lo):
            hi = min(n, lo + step)
            data[lo:hi] = synth.normal(seed, stream, hi - lo, layer, scale=0.02, start=start + lo)

        if threads > 1:
            with ThreadPoolExecutor(threads) as ex:
                list(ex.map(part, range(0, n, step)))
        else:
            for lo in range(0, n, step):
                part(lo)
        return Matrix.from_f32(data, count * rows_per_expert, cols, fmt)

    return LayerWeights(router=_normal_matrix(seed, synth.STREAM_ROUTER, layer, e, h, "bf16"),
                        gate_up=rows(synth.STREAM_GATE_UP, 2 * i, h), down=rows(synth.STREAM_DOWN, h, i))


def hidden_states(shape: MoeShape, tokens: int, seed: int = 0, layer: int = 0) -> np.ndarray:
    return synth.normal(seed, synth.STREAM_HIDDEN, tokens * shape.hidden, layer).reshape(tokens, shape.hidden)


def expert_bytes(shape: MoeShape, fmt: str | None = None) -> int:
    """Stored bytes of one expert's gate_up + down rows."""
    fmt = fmt or shape.fmt
    h, i = shape.hidden, shape.inter
    if fmt == "q8":
        return 3 * i * h + 3 * i * h // 32 * 2
    if fmt == "q4":
        from .weights import q4_words

        return 3 * i * h // 2 + (2 * i * q4_words(h) + h * q4_words(i)) * 4
    raise ValueError(fmt)


def decode_algorithmic_bytes(shape: MoeShape, tokens: int, distinct_experts: int, fmt: str | None = None) -> int:
    """Bytes one MoE block must move for a decode-size batch: the weights of
    every expert that was selected, the router, and the activations in and out."""
    return (distinct_experts * expert_bytes(shape, fmt) + shape.experts * shape.hidden * 2
            + tokens * shape.hidden * 4 * 2)
