"""Parity at the sizes the workloads name, not only at toy token counts: the
routing-skew shape at 256, 4096 and 16384 tokens, the 3b-a800m shape in 4 bits at a
prefill of 4 x 1024 tokens, and the 1b-a400m shape at the batch where the library
switches kernel families. Both families (the bandwidth-oriented kernels and the
tcgen05 ones) against the oracle, and against each other bit for bit."""
import numpy as np
import pytest

from tachyon_b200 import synth, workloads
from tachyon_b200.workloads import MoeShape
from test_gpu_parity import check_block, ctx, layer_weights, make_layer, oracle_moe  # noqa: F401

pytestmark = pytest.mark.gpu

NEVER = 1 << 30
SKEW = MoeShape("skew", 2048, 64, 8, 1024, fmt="q8")


@pytest.fixture
def thresholds(ctx):
    yield ctx
    ctx.set_prefill_threshold(32)
    ctx.set_arithmetic(ctx.ARITH_FAST)


def forward(ctx, layer, x, y0):
    xd, yd = ctx.to_device(x), ctx.to_device(y0)
    layer.forward(xd, yd)
    ctx.sync()
    y = yd.get()
    xd.free()
    yd.free()
    return y


@pytest.mark.parametrize("t", [256, 4096])
@pytest.mark.parametrize("family", ["bandwidth", "tcgen05"])
def test_skew_shape_with_zipf_bias(oracle, thresholds, t, family):
    """hidden 2048, 64 experts, intermediate 1024, int8, Zipf(1.2) router bias: loads span far
    more than 20x; each kernel family forced in turn, against the CPU path."""
    ctx = thresholds
    lw = layer_weights(oracle, SKEW, 1)
    bias = synth.zipf_router_bias(1, SKEW.experts)
    x = workloads.hidden_states(SKEW, t, seed=21)
    ctx.set_prefill_threshold(NEVER if family == "bandwidth" else 0)
    check_block(oracle, ctx, SKEW, lw, x, bias=bias, arith="fast")
    ref = oracle_moe(oracle, lw, x, SKEW.topk, bias)
    assert ref.counts.max() > 20 * max(1, ref.counts[ref.counts > 0].min())


def test_skew_shape_16384_tokens(oracle, thresholds):
    """The largest token count of the workload: the two kernel families bit for bit against each
    other on all 16384 tokens, and 512 of the tokens against the CPU path (a token's output
    does not depend on its batch, so the sample runs through the oracle on its own)."""
    ctx = thresholds
    t = 16384
    lw = layer_weights(oracle, SKEW, 1)
    bias = synth.zipf_router_bias(1, SKEW.experts)
    x = workloads.hidden_states(SKEW, t, seed=22)
    y0 = np.zeros_like(x)
    layer = make_layer(ctx, lw, SKEW.topk, t)
    layer.set_router_bias(bias)
    try:
        ctx.set_prefill_threshold(0)
        tc = forward(ctx, layer, x, y0)
        ids, gates, counts, _ = layer.last_routing(t)
        ctx.set_prefill_threshold(NEVER)
        bw = forward(ctx, layer, x, y0)
    finally:
        layer.free()
    assert np.array_equal(tc, bw)
    assert counts.sum() == t * SKEW.topk and counts.max() > 20 * max(1, counts[counts > 0].min())
    pick = np.arange(0, t, 32)  # 512 tokens spread over the batch
    ref = oracle_moe(oracle, lw, x[pick], SKEW.topk, bias)
    assert np.array_equal(ids[pick], ref.ids)
    assert np.abs(gates[pick] - ref.gates).max() <= 1e-5
    err = np.abs(tc[pick] - ref.proj)
    assert err.max() <= 2e-3 and err.max() <= 1e-3 * np.abs(ref.proj).max()
    with oracle.fast_arithmetic_model():
        model = oracle_moe(oracle, lw, x[pick], SKEW.topk, bias)
    same = np.all(gates[pick] == model.gates, axis=1)
    assert same.mean() > 0.5
    assert np.array_equal(tc[pick][same], model.proj[same])


def test_granite_3b_shape_4bit_prefill_of_4096_tokens(oracle, thresholds):
    """hidden 1536, 40 experts, intermediate 512, Tachyon's 4-bit group quantizer, 4 x 1024 tokens."""
    ctx = thresholds
    shape = MoeShape("3b-q4", 1536, 40, 8, 512, fmt="q4")
    lw = layer_weights(oracle, shape, 1)
    x = workloads.hidden_states(shape, 4096, seed=23)
    ctx.set_prefill_threshold(32)  # the library's own choice at this size: the tcgen05 kernels
    check_block(oracle, ctx, shape, lw, x, arith="fast")


@pytest.mark.parametrize("fmt", ["q8", "q4"])
def test_granite_1b_shape_at_the_switch_between_kernel_families(oracle, thresholds, fmt):
    """Batch 128 of the 1b-a400m shape averages exactly 32 tokens per expert, the default
    threshold; 127 tokens stay on the other side. Both against the CPU path, and the shared
    tokens bit for bit against each other."""
    ctx = thresholds
    shape = MoeShape("1b", 1024, 32, 8, 512, fmt=fmt)
    lw = layer_weights(oracle, shape, 0)
    x = workloads.hidden_states(shape, 128, seed=24)
    ctx.set_prefill_threshold(32)
    a = check_block(oracle, ctx, shape, lw, x, arith="fast")
    b = check_block(oracle, ctx, shape, lw, x[:127], arith="fast")
    assert np.array_equal(a[:127], b)
