"""The committed golden fixtures (tests/golden/moe_block_*.npz, made by
tests/golden/make_golden.py): the oracle must still reproduce them, and the CUDA
path must reproduce them through the C ABI in both arithmetic modes."""
import importlib.util
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
_spec = importlib.util.spec_from_file_location("make_golden", os.path.join(HERE, "golden", "make_golden.py"))
make_golden = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(make_golden)


def load(name):
    return np.load(os.path.join(HERE, "golden", f"moe_block_{name}.npz"))


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_oracle_reproduces_the_golden_fixture(oracle, name):
    want = load(name)
    got = make_golden.run_case(name)
    assert str(got["inputs_sha256"]) == str(want["inputs_sha256"]), "the seeded inputs changed"
    for key in ["ids", "gates", "counts", "logits", "proj", "proj_chain"]:
        assert np.array_equal(got[key], want[key]), key


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_cuda_path_reproduces_the_golden_fixture(oracle, name):
    from tachyon_b200 import build, cuda

    build.build()
    want = load(name)
    shape, tokens, seed = make_golden.CASES[name]
    lw, x = make_golden.case_inputs(shape, tokens, seed)
    ctx = cuda.Context(0)
    try:
        for mode, key in [(ctx.ARITH_CPU_LANES, "proj"), (ctx.ARITH_FAST, "proj_chain")]:
            ctx.set_arithmetic(mode)
            layer = cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.topk, tokens)
            xd, yd = ctx.to_device(x), ctx.to_device(np.zeros_like(x))
            layer.forward(xd, yd)
            ctx.sync()
            ids, gates, counts, logits = layer.last_routing(tokens)
            assert np.array_equal(logits, want["logits"])
            assert np.array_equal(ids, want["ids"]) and np.array_equal(counts, want["counts"])
            assert np.max(np.abs(gates - want["gates"])) <= 1e-5
            same = np.all(gates == want["gates"], axis=1)
            assert same.any()
            y = yd.get()
            assert np.array_equal(y[same], (np.zeros_like(x) + want[key])[same]), key
            assert np.max(np.abs(y - want[key])) <= 2e-3
            for d in (xd, yd):
                d.free()
            layer.free()
    finally:
        ctx.set_arithmetic(ctx.ARITH_FAST)
        ctx.close()
