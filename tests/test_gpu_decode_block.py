"""The one-kernel decode block (up to 32 tokens: router, experts and combine in one
persistent kernel whose CTAs meet at grid-wide counters) against the oracle and
against the four-kernel path: same arithmetic, so the same bits."""
import numpy as np
import pytest

from tachyon_b200 import synth, workloads
from tachyon_b200.workloads import MoeShape
from test_gpu_parity import check_block, ctx, layer_weights, make_layer, oracle_moe  # noqa: F401

pytestmark = pytest.mark.gpu

SHAPES = [
    MoeShape("1b", 1024, 32, 8, 512, fmt="q8"),
    MoeShape("1b-q4", 1024, 32, 8, 512, fmt="q4"),
    MoeShape("3b-q4", 1536, 40, 8, 512, fmt="q4"),
    MoeShape("skew", 2048, 64, 8, 1024, fmt="q8"),
    MoeShape("tiny", 256, 8, 2, 64, fmt="q8"),       # fewer 16-row units than CTAs
    MoeShape("many", 256, 200, 4, 32, fmt="q8"),     # a CTA's range spans many experts
]


def both_paths(ctx, layer, x, y0, norm_w=None):
    outs = []
    for on in (True, False):
        ctx.set_decode_block(on)
        yd = ctx.to_device(y0)
        if norm_w is None:
            xd = ctx.to_device(x)
            layer.forward(xd, yd)
            xd.free()
        else:
            layer.block(norm_w, 1e-6, yd)
        ctx.sync()
        outs.append(yd.get())
        yd.free()
    ctx.set_decode_block(True)
    return outs


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: s.name)
def test_one_kernel_block_equals_the_four_kernel_path(oracle, ctx, shape):
    """Every batch size the kernel takes that changes its walk: one token, the sparse walk
    (only the picked experts), the dense walk, a full batch, with and without a router
    bias that piles the tokens onto a few experts."""
    lw = layer_weights(oracle, shape, 13)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    layer = make_layer(ctx, lw, shape.topk, 32)
    bias = synth.zipf_router_bias(13, shape.experts)
    try:
        for t in [1, 2, 7, 8, 9, 16, 25, 32]:
            for b in (None, bias):
                layer.set_router_bias(b)
                x = workloads.hidden_states(shape, t, seed=40 + t)
                y0 = workloads.hidden_states(shape, t, seed=80 + t)
                one, four = both_paths(ctx, layer, x, y0)
                assert np.array_equal(one, four), (shape.name, t, b is not None, np.abs(one - four).max())
                ids1, gates1, counts1, logits1 = layer.last_routing(t)  # the taps of the four-kernel run
                ctx.set_decode_block(True)
                xd, yd = ctx.to_device(x), ctx.to_device(y0)
                layer.forward(xd, yd)
                ids2, gates2, counts2, logits2 = layer.last_routing(t)  # built on demand after the one-kernel run
                offsets, perm = layer.last_dispatch(t)
                assert np.array_equal(ids1, ids2) and np.array_equal(gates1, gates2)
                assert np.array_equal(counts1, counts2) and np.array_equal(logits1, logits2)
                assert np.array_equal(np.diff(offsets), counts2)
                assert np.array_equal(np.sort(perm), np.arange(t * shape.topk, dtype=np.uint32))
                xd.free()
                yd.free()
    finally:
        layer.free()


@pytest.mark.parametrize("fmt", ["q8", "q4"])
@pytest.mark.parametrize("t", [1, 8, 32])
def test_one_kernel_block_meets_the_oracle_bars(oracle, ctx, fmt, t):
    """The decode batch sizes of the 1b-a400m shape against the CPU path (tolerances of the
    workload; bit for bit against the oracle's model of the single-chain order)."""
    shape = MoeShape("1b", 1024, 32, 8, 512, fmt=fmt)
    lw = layer_weights(oracle, shape, 0)
    x = workloads.hidden_states(shape, t, seed=3)
    ctx.set_decode_block(True)
    check_block(oracle, ctx, shape, lw, x, arith="fast")


@pytest.mark.parametrize("shape", SHAPES[:4] + SHAPES[5:], ids=lambda s: s.name)
def test_one_kernel_block_from_33_to_128_tokens(oracle, ctx, shape):
    """Above 32 tokens the one-kernel block runs in its expert-parallel form with the GPU as the
    only rank (an expert's tokens in runs of up to 32, rows and outputs through a local window):
    same bits as the four-kernel path, whatever the batch before it was."""
    lw = layer_weights(oracle, shape, 17)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    ctx.set_prefill_threshold(1 << 30)  # the comparison path stays on the bandwidth kernels
    layer = make_layer(ctx, lw, shape.topk, 128)
    bias = synth.zipf_router_bias(17, shape.experts)
    try:
        for t in [33, 64, 5, 100, 128, 47]:
            for b in (None, bias):
                layer.set_router_bias(b)
                x = workloads.hidden_states(shape, t, seed=140 + t)
                y0 = workloads.hidden_states(shape, t, seed=180 + t)
                one, four = both_paths(ctx, layer, x, y0)
                assert np.array_equal(one, four), (shape.name, t, b is not None, np.abs(one - four).max())
    finally:
        ctx.set_prefill_threshold(32)
        layer.free()


def test_64_token_block_meets_the_oracle_bars_and_replays_from_a_graph(oracle, ctx):
    shape = MoeShape("1b", 1024, 32, 8, 512, fmt="q8")
    lw = layer_weights(oracle, shape, 0)
    x = workloads.hidden_states(shape, 64, seed=3)
    ctx.set_decode_block(True)
    check_block(oracle, ctx, shape, lw, x, arith="fast")
    layer = make_layer(ctx, lw, shape.topk, 64)
    y0 = workloads.hidden_states(shape, 64, seed=4)
    xd, yd = ctx.to_device(x), ctx.to_device(y0)
    layer.forward(xd, yd)
    ctx.sync()
    want = yd.get()
    ctx.capture_begin()
    layer.forward(xd, yd)
    g = ctx.capture_end()
    for _ in range(3):
        ctx.upload(yd.ptr, y0)
        g.launch()
        ctx.sync()
        assert np.array_equal(yd.get(), want)
    g.free()
    layer.free()


def test_blocks_chained_in_a_graph_with_the_norm_fused(oracle, ctx):
    """Six blocks back to back on the residual stream, captured and replayed: each kernel
    starts under the previous one's tail, and the grid-wide counters must be back at
    zero every time."""
    shape = MoeShape("chain", 512, 16, 4, 128, fmt="q8")
    ctx.set_arithmetic(ctx.ARITH_FAST)
    lws = [layer_weights(oracle, shape, 30 + i) for i in range(3)]
    layers = [make_layer(ctx, lw, shape.topk, 32) for lw in lws]
    w = (1.0 + synth.normal(4, 2, shape.hidden, scale=0.1)).astype(np.float32)
    wd = ctx.to_device(w)
    for t in [3, 32]:
        y0 = workloads.hidden_states(shape, t, seed=5)
        results = []
        for on in (True, False):
            ctx.set_decode_block(on)
            yd = ctx.to_device(y0)
            ctx.capture_begin()
            for _ in range(2):
                for layer in layers:
                    layer.block(wd, 1e-6, yd, t=t)
            g = ctx.capture_end()
            for rep in range(3):
                ctx.upload(yd.ptr, y0)
                g.launch()
                ctx.sync()
                results.append(yd.get())
            g.free()
            yd.free()
        ctx.set_decode_block(True)
        for r in results[1:]:
            assert np.array_equal(results[0], r)
        # and the CPU path, block by block
        want = y0.copy()
        with oracle.fast_arithmetic_model():
            for _ in range(2):
                for lw in lws:
                    want = want + oracle_moe(oracle, lw, oracle.rmsnorm_rows(want, w, 1e-6), shape.topk).proj
        assert np.abs(results[0] - want).max() <= 2e-3 * max(1.0, np.abs(want).max())
    for layer in layers:
        layer.free()


def test_phase_stamps_are_ordered(oracle, ctx):
    shape = MoeShape("1b", 1024, 32, 8, 512, fmt="q8")
    lw = layer_weights(oracle, shape, 0)
    layer = make_layer(ctx, lw, shape.topk, 32)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    ctx.set_decode_block(True)
    ctx.profile_phases(True)
    x = workloads.hidden_states(shape, 32, seed=3)
    xd, yd = ctx.to_device(x), ctx.to_device(np.zeros_like(x))
    layer.forward(xd, yd)
    phases = ctx.read_phases()
    ctx.profile_phases(False)
    assert all(v >= 0 for v in phases.values()), phases
    assert 0 < sum(phases.values()) < 1e5, phases  # microseconds
    layer.free()
