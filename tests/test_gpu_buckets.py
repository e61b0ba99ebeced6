"""A CUDA graph per batch-size bucket: a step padded to its bucket gives the real rows the
bits of an eager call on exactly those rows, and a bucket is captured once."""
import numpy as np
import pytest

from tachyon_b200 import synth, workloads
from tachyon_b200.buckets import GraphBuckets
from tachyon_b200.workloads import MoeShape
from test_gpu_parity import ctx, layer_weights, make_layer  # noqa: F401

pytestmark = pytest.mark.gpu


def test_bucketed_graphs_equal_eager_blocks(oracle, ctx):
    shape = MoeShape("buckets", 256, 8, 2, 64, fmt="q8")
    ctx.set_arithmetic(ctx.ARITH_FAST)
    lws = [layer_weights(oracle, shape, 40 + i) for i in range(2)]
    layers = [make_layer(ctx, lw, shape.topk, 64) for lw in lws]
    norms = [ctx.to_device((1.0 + synth.normal(7, 2, shape.hidden, layer=i, scale=0.1)).astype(np.float32))
             for i in range(2)]
    gb = GraphBuckets(ctx, layers, norms, 1e-6, shape.hidden, buckets=(1, 2, 4, 8, 16, 32, 64))
    try:
        for t in [3, 1, 8, 20, 3, 33, 64]:
            x = workloads.hidden_states(shape, t, seed=300 + t)
            got = gb.step(x)
            yd = ctx.to_device(x)
            for layer, w in zip(layers, norms):
                layer.block(w, 1e-6, yd, t=t)
            ctx.sync()
            want = yd.get()
            yd.free()
            assert got.shape == want.shape
            assert np.array_equal(got, want), (t, np.abs(got - want).max())
        assert sorted(gb.graphs) == [1, 4, 8, 32, 64]
        assert gb.launches[4] == 2
    finally:
        gb.free()
        for d in norms:
            d.free()
        for layer in layers:
            layer.free()
