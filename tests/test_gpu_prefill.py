"""The tcgen05 (tensor memory) expert kernels against the oracle and against the
bandwidth-oriented kernels: same fma chain per output, so the same bits.

The library picks the tensor-core kernels from an average of 32 tokens per
expert; the tests force either path with the threshold."""
import numpy as np
import pytest

from tachyon_b200 import synth, workloads
from tachyon_b200.workloads import MoeShape
from test_gpu_parity import check_block, ctx, layer_weights, make_layer  # noqa: F401

pytestmark = pytest.mark.gpu

NEVER = 1 << 30


def forward(ctx, layer, x, y0):
    xd, yd = ctx.to_device(x), ctx.to_device(y0)
    layer.forward(xd, yd)
    ctx.sync()
    y = yd.get()
    xd.free()
    yd.free()
    return y


@pytest.fixture
def always_prefill(ctx):
    ctx.set_prefill_threshold(0)
    yield ctx
    ctx.set_prefill_threshold(32)


@pytest.mark.parametrize("shape,t", [
    (MoeShape("small-q8", 256, 8, 2, 96, fmt="q8"), 300),    # ragged row tile (96 rows of 128), one chunk
    (MoeShape("small-q4", 512, 16, 4, 192, fmt="q4"), 333),  # 4-bit offsets, ragged token tiles
    (MoeShape("1b-q8", 1024, 32, 8, 512, fmt="q8"), 512),    # operand ring and TMEM ring wrap
    (MoeShape("3b-q4", 1536, 40, 8, 512, fmt="q4"), 200),
])
def test_prefill_kernels_meet_the_oracle_bars(oracle, always_prefill, shape, t):
    lw = layer_weights(oracle, shape, 11)
    x = workloads.hidden_states(shape, t, seed=11)
    check_block(oracle, always_prefill, shape, lw, x, arith="fast")


@pytest.mark.parametrize("fmt", ["q8", "q4"])
def test_both_kernel_families_give_the_same_bits(oracle, ctx, fmt):
    """Also with a skewed router: experts with no token, one token, several 64-token tiles."""
    shape = MoeShape("skew-small", 256, 64, 8, 64, fmt=fmt)
    lw = layer_weights(oracle, shape, 5)
    bias = synth.zipf_router_bias(5, 64)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    for t in [1, 7, 64, 65, 700, 2048]:
        x = workloads.hidden_states(shape, t, seed=5)
        y0 = synth.normal(9, synth.STREAM_HIDDEN, x.size, layer=1).reshape(x.shape)
        layer = make_layer(ctx, lw, shape.topk, t)
        layer.set_router_bias(bias)
        try:
            ctx.set_prefill_threshold(NEVER)
            a = forward(ctx, layer, x, y0)
            ctx.set_prefill_threshold(0)
            b = forward(ctx, layer, x, y0)
            b2 = forward(ctx, layer, x, y0)
        finally:
            ctx.set_prefill_threshold(32)
            layer.free()
        assert np.array_equal(a, b)
        assert np.array_equal(b, b2)


def test_default_threshold_switches_by_batch_size(oracle, ctx):
    """Crossing the threshold must not change a token's output."""
    shape = MoeShape("small-q8", 256, 8, 2, 96, fmt="q8")
    lw = layer_weights(oracle, shape, 11)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    ctx.set_prefill_threshold(32)
    x = workloads.hidden_states(shape, 256, seed=3)  # 256 * 2 / 8 = 64 per expert: tensor-core path
    y0 = np.zeros_like(x)
    layer = make_layer(ctx, lw, shape.topk, 256)
    big = forward(ctx, layer, x, y0)
    small = forward(ctx, layer, x[:40], y0[:40])     # 10 per expert: bandwidth path
    layer.free()
    assert np.array_equal(big[:40], small)


def test_scratch_shared_by_layers_only_grows(oracle, ctx):
    """Two layers in one context share the token-tile scratch of the tensor-core path. A
    wide layer is created first, then a narrow one that needs more tiles but fewer bytes
    per tile; the wide layer's next prefill-size block must still fit (and be right)."""
    wide = MoeShape("wide", 1024, 8, 2, 256, fmt="q8")
    narrow = MoeShape("narrow", 256, 16, 4, 64, fmt="q8")
    lw_w, lw_n = layer_weights(oracle, wide, 21), layer_weights(oracle, narrow, 22)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    la = make_layer(ctx, lw_w, wide.topk, 600)
    lb = make_layer(ctx, lw_n, narrow.topk, 1200)
    ctx.set_prefill_threshold(0)
    try:
        for layer, shape, lw, t in [(la, wide, lw_w, 600), (lb, narrow, lw_n, 1200), (la, wide, lw_w, 600)]:
            x = workloads.hidden_states(shape, t, seed=23)
            y0 = np.zeros_like(x)
            got = forward(ctx, layer, x, y0)
            with oracle.fast_arithmetic_model():
                from test_gpu_parity import oracle_moe

                want = oracle_moe(oracle, lw, x, shape.topk).proj
            assert np.abs(got - want).max() <= 2e-3
            assert np.mean(np.all(got == want, axis=1)) > 0.5
    finally:
        ctx.set_prefill_threshold(32)
        la.free()
        lb.free()
