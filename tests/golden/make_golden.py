"""Generates tests/golden/moe_block_*.npz: the CPU oracle's answers for small seeded
MoE blocks, committed so that a change in the oracle (or in the synthetic
generator or the quantizers feeding it) shows up as a diff instead of moving
the target the CUDA kernels are held to.

Tachyon itself is Rust and cannot be built or run in this environment, so
these are outputs of the C++ restatement (oracle/tachyon_oracle.cpp), which is
pinned separately by Tachyon's own known-answer tests (tests/test_oracle_kats.py).

    python tests/golden/make_golden.py        # rewrites the fixtures

Each file holds the inputs' checksums, the routing (ids, gates, counts, logits)
and the block's output in both arithmetic orders the library offers: the CPU
path's eight-lane order ("proj") and the single-chain order of the default
kernels ("proj_chain", the oracle's model of it).
"""
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import binding as oracle  # noqa: E402
from tachyon_b200 import synth, weights, workloads  # noqa: E402
from tachyon_b200.workloads import MoeShape  # noqa: E402

CASES = {
    # name: (shape, tokens, seed)
    "q8": (MoeShape("golden-q8", 256, 8, 2, 64, fmt="q8"), 7, 21),
    "q4": (MoeShape("golden-q4", 512, 10, 4, 96, fmt="q4"), 5, 22),
}


def case_inputs(shape: MoeShape, tokens: int, seed: int):
    """Weights and input rows of a case; 4-bit matrices through the oracle's quantizer."""
    if shape.fmt == "q4":
        h, e, i = shape.hidden, shape.experts, shape.inter
        router = workloads._normal_matrix(seed, synth.STREAM_ROUTER, 0, e, h, "bf16")

        def q4(stream, rows, cols):
            data = synth.normal(seed, stream, rows * cols, 0, scale=0.02)
            s, q = oracle.quantize_q4_matrix(data, rows, cols, None, 2)
            return weights.Matrix(weights.KIND_Q4, rows, cols, s, q)

        lw = workloads.LayerWeights(router, q4(synth.STREAM_GATE_UP, e * 2 * i, h), q4(synth.STREAM_DOWN, e * h, i))
    else:
        lw = workloads.layer_weights(shape, seed=seed, threads=2)
    x = workloads.hidden_states(shape, tokens, seed=seed)
    return lw, x


def digest(*arrays) -> str:
    h = hashlib.sha256()
    for a in arrays:
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def run_case(name: str):
    shape, tokens, seed = CASES[name]
    lw, x = case_inputs(shape, tokens, seed)

    def om(m):
        return oracle.OracleMatrix(m.kind, m.rows, m.cols, m.scales, m.data)

    ref = oracle.moe(om(lw.router), om(lw.gate_up), om(lw.down), x, shape.topk, threads=2)
    with oracle.fast_arithmetic_model():
        chain = oracle.moe(om(lw.router), om(lw.gate_up), om(lw.down), x, shape.topk, threads=2)
    return {
        "inputs_sha256": np.array(digest(lw.router.data, lw.gate_up.scales, lw.gate_up.data, lw.down.scales,
                                         lw.down.data, x)),
        "ids": ref.ids, "gates": ref.gates, "counts": ref.counts, "logits": ref.logits,
        "proj": ref.proj, "proj_chain": chain.proj,
    }


def main():
    oracle.build()
    here = os.path.dirname(os.path.abspath(__file__))
    for name in CASES:
        out = run_case(name)
        np.savez_compressed(os.path.join(here, f"moe_block_{name}.npz"), **out)
        print(name, {k: getattr(v, "shape", None) for k, v in out.items()})


if __name__ == "__main__":
    main()
