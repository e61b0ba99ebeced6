"""Parity of the CUDA MoE block with the CPU oracle, through the C ABI.

Bars (the ones the workload states): expert indices and per-expert counts equal
wherever the router-logit gap at the k-th position exceeds 1e-5; gates within
1e-5; block outputs within 2e-3 max-abs and 1e-3 relative. Where the kernels
reproduce the CPU path's operation order, the tests also ask for bit equality.
"""
import numpy as np
import pytest

from refgen import xorshift_data
from tachyon_b200 import synth, weights, workloads
from tachyon_b200.workloads import MoeShape

pytestmark = pytest.mark.gpu

GATE_TOL = 1e-5
OUT_ABS, OUT_REL = 2e-3, 1e-3
GAP = 1e-5


@pytest.fixture(scope="module")
def ctx():
    from tachyon_b200 import build, cuda

    build.build()
    c = cuda.Context(0)
    yield c
    c.close()


_WEIGHTS = {}


def layer_weights(oracle, shape: MoeShape, seed: int):
    """Seeded weights of a shape, cached across tests. 4-bit matrices go through
    the oracle's multi-threaded quantizer: it produces the same bytes as the
    numpy mirror (tests/test_host_mirror.py) in a fraction of the time."""
    key = (shape.hidden, shape.experts, shape.inter, shape.fmt, seed)
    if key not in _WEIGHTS:
        if shape.fmt == "q4":
            h, e, i = shape.hidden, shape.experts, shape.inter
            router = workloads._normal_matrix(seed, synth.STREAM_ROUTER, 0, e, h, "bf16")

            def q4(stream, rows, cols):
                data = synth.normal(seed, stream, rows * cols, 0, scale=0.02)
                s, q = oracle.quantize_q4_matrix(data, rows, cols, None, 8)
                return weights.Matrix(weights.KIND_Q4, rows, cols, s, q)

            _WEIGHTS[key] = workloads.LayerWeights(router, q4(synth.STREAM_GATE_UP, e * 2 * i, h),
                                                   q4(synth.STREAM_DOWN, e * h, i))
        else:
            _WEIGHTS[key] = workloads.layer_weights(shape, seed=seed, threads=6)
    return _WEIGHTS[key]


def to_oracle(oracle, m: weights.Matrix):
    return oracle.OracleMatrix(m.kind, m.rows, m.cols, m.scales, m.data)


def make_layer(ctx, lw, topk, max_tokens):
    from tachyon_b200 import cuda

    return cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, topk, max_tokens)


def oracle_moe(oracle, lw, x, topk, bias=None, threads=6):
    return oracle.moe(to_oracle(oracle, lw.router), to_oracle(oracle, lw.gate_up), to_oracle(oracle, lw.down),
                      x, topk, router_bias=bias, threads=threads)


def run_gpu(ctx, layer, x, y0):
    xd, yd = ctx.to_device(x), ctx.to_device(y0)
    layer.forward(xd, yd)
    ctx.sync()
    y = yd.get()
    t = x.shape[0]
    ids, gates, counts, logits = layer.last_routing(t)
    xd.free()
    yd.free()
    return y, ids, gates, counts, logits


ARITH = ["fast", "lanes"]


def check_block(oracle, ctx, shape: MoeShape, lw, x, bias=None, arith="lanes"):
    """Runs both sides on x[t, hidden] and applies the bars. Returns the GPU output.

    arith="lanes": the kernels that keep the CPU path's eight-lane order; they
    must match the oracle bit for bit. arith="fast" (the default mode of the
    library): one fma chain per output; held to the stated tolerances against
    the oracle, and bit for bit against the oracle's model of that order."""
    t = x.shape[0]
    ctx.set_arithmetic(ctx.ARITH_CPU_LANES if arith == "lanes" else ctx.ARITH_FAST)
    layer = make_layer(ctx, lw, shape.topk, t)
    if bias is not None:
        layer.set_router_bias(bias)
    y0 = synth.normal(7, synth.STREAM_HIDDEN, x.size, layer=3).reshape(x.shape)
    y, ids, gates, counts, logits = run_gpu(ctx, layer, x, y0)
    ref = oracle_moe(oracle, lw, x, shape.topk, bias)
    want = y0 + ref.proj  # src/model.rs:681

    # Router logits follow the AVX2 summation order: bit equality.
    assert np.array_equal(logits, ref.logits)
    # Indices wherever the gap between the k-th and (k+1)-th logit is above 1e-5.
    srt = -np.sort(-ref.logits, axis=1)
    gap = srt[:, shape.topk - 1] - srt[:, shape.topk] if shape.experts > shape.topk else np.full(t, 1.0)
    clear = gap > GAP
    assert np.array_equal(ids[clear], ref.ids[clear])
    if clear.all():
        assert np.array_equal(counts, ref.counts)
        assert np.array_equal(counts, np.bincount(ids.ravel(), minlength=shape.experts))
    assert np.max(np.abs(gates[clear] - ref.gates[clear])) <= GATE_TOL
    # Block output.
    err = np.abs(y - want)
    assert err.max() <= OUT_ABS, err.max()
    assert err.max() <= OUT_REL * np.abs(want).max()
    assert np.linalg.norm(y - want) <= OUT_REL * np.linalg.norm(want)
    # Tokens whose gates came out bit-equal must match bit for bit: SwiGLU,
    # re-quantization and the combine order are the CPU path's own, and the
    # expert products are either the CPU path's ("lanes") or the stated chain
    # order, which the oracle models ("fast").
    same = clear & np.all(gates == ref.gates, axis=1)
    assert same.mean() > 0.5
    if arith == "lanes":
        assert np.array_equal(y[same], want[same])
    else:
        with oracle.fast_arithmetic_model():
            model = oracle_moe(oracle, lw, x, shape.topk, bias)
        assert np.array_equal(y[same], (y0 + model.proj)[same])
    # Dispatch: expert-contiguous, ascending tokens within each expert.
    offsets, perm = layer.last_dispatch(t)
    assert offsets[0] == 0 and offsets[-1] == t * shape.topk
    assert np.array_equal(np.diff(offsets), counts)
    assert np.array_equal(np.sort(perm), np.arange(t * shape.topk, dtype=np.uint32))
    flat = ids.ravel()
    for e in range(shape.experts):
        seg = perm[offsets[e]:offsets[e + 1]]
        assert np.all(flat[seg] == e)
        assert np.all(np.diff(seg // shape.topk) > 0)
    layer.free()
    return y


def test_rmsnorm_matches_cpu_bit_for_bit(oracle, ctx):
    for t, n in [(64, 1024), (3, 352), (5, 40), (2, 1536)]:
        x = synth.normal(0, 1, t * n).reshape(t, n)
        w = (1.0 + synth.normal(0, 2, n, scale=0.1)).astype(np.float32)
        xd, wd, od = ctx.to_device(x), ctx.to_device(w), ctx.empty((t, n))
        ctx.rmsnorm(xd, wd, 1e-6, od)
        ctx.sync()
        assert np.array_equal(od.get(), oracle.rmsnorm_rows(x, w, 1e-6)), (t, n)
        ctx.rmsnorm(xd, wd, 1e-6, xd)  # in place
        ctx.sync()
        assert np.array_equal(xd.get(), oracle.rmsnorm_rows(x, w, 1e-6))


@pytest.mark.parametrize("arith", ARITH)
@pytest.mark.parametrize("fmt", ["q8", "q4"])
def test_single_block_64_tokens(oracle, ctx, fmt, arith):
    """64 tokens, hidden 1024, 32 experts, top-8, intermediate 512, inputs
    N(0,1) after RMSNorm (weight 1, eps 1e-6), seed 0."""
    shape = MoeShape("block", 1024, 32, 8, 512, fmt=fmt)
    lw = layer_weights(oracle, shape, 0)
    h = workloads.hidden_states(shape, 64, seed=0)
    hd, wd = ctx.to_device(h), ctx.to_device(np.ones(1024, np.float32))
    ctx.rmsnorm(hd, wd, 1e-6, hd)
    ctx.sync()
    x = hd.get()
    assert np.array_equal(x, oracle.rmsnorm_rows(h, np.ones(1024, np.float32), 1e-6))
    check_block(oracle, ctx, shape, lw, x, arith=arith)


@pytest.mark.parametrize("arith", ARITH)
@pytest.mark.parametrize("fmt", ["q8", "q4"])
@pytest.mark.parametrize("t", [1, 2, 3, 5, 8, 9, 17, 40])
def test_ragged_shapes(oracle, ctx, fmt, t, arith):
    """A partial last super-block (11 blocks per row), row counts that do not
    fill a warp's tile, and the token counts Tachyon's own matmul test walks
    (src/weights.rs:696)."""
    shape = MoeShape("ragged", 352, 5, 3, 96, fmt=fmt)
    rng_w = lambda n, s: xorshift_data(n, s) * np.float32(0.05)
    router = weights.Matrix.from_f32(rng_w(5 * 352, 11), 5, 352, "bf16")
    gate_up = weights.Matrix.from_f32(rng_w(5 * 192 * 352, 12), 5 * 192, 352, fmt)
    down = weights.Matrix.from_f32(rng_w(5 * 352 * 96, 13), 5 * 352, 96, fmt)
    lw = workloads.LayerWeights(router, gate_up, down)
    x = xorshift_data(t * 352, t + 7).reshape(t, 352)
    check_block(oracle, ctx, shape, lw, x, arith=arith)


@pytest.mark.parametrize("arith", ARITH)
@pytest.mark.parametrize("fmt", ["q8", "q4"])
def test_batching_never_changes_a_token(oracle, ctx, fmt, arith):
    """Each token alone gives exactly its result in the batch (the property
    src/weights.rs:704-713 asserts for the CPU matmul), in both arithmetic modes."""
    shape = MoeShape("inv", 512, 8, 2, 128, fmt=fmt)
    lw = layer_weights(oracle, shape, 3)
    x = workloads.hidden_states(shape, 85, seed=3)
    ctx.set_arithmetic(ctx.ARITH_CPU_LANES if arith == "lanes" else ctx.ARITH_FAST)
    layer = make_layer(ctx, lw, shape.topk, 85)
    zeros = np.zeros_like(x)
    y, *_ = run_gpu(ctx, layer, x, zeros)
    for i in [0, 7, 20, 84]:
        yi, *_ = run_gpu(ctx, layer, x[i:i + 1], zeros[i:i + 1])
        assert np.array_equal(yi[0], y[i])
    y9, *_ = run_gpu(ctx, layer, x[:9], zeros[:9])
    assert np.array_equal(y9, y[:9])
    layer.free()


@pytest.mark.parametrize("arith", ARITH)
def test_routing_skew_with_bias_and_many_tokens_per_expert(oracle, ctx, arith):
    """A Zipf(1.2) router bias: a few experts take most tokens, so their groups
    span several 8-token register tiles, and t > 256 takes the multi-CTA dispatch."""
    shape = MoeShape("skew-small", 256, 64, 8, 64, fmt="q8")
    lw = layer_weights(oracle, shape, 5)
    bias = synth.zipf_router_bias(5, 64)
    for t in [1, 16, 256, 700]:
        x = workloads.hidden_states(shape, t, seed=5)
        y = check_block(oracle, ctx, shape, lw, x, bias=bias, arith=arith)
        assert y.shape == x.shape
    ref = oracle_moe(oracle, lw, workloads.hidden_states(shape, 700, seed=5), 8, bias)
    assert ref.counts.max() > 20 * max(1, ref.counts[ref.counts > 0].min())


@pytest.mark.parametrize("arith", ARITH)
def test_granite_3b_shape_and_skew_shape(oracle, ctx, arith):
    """hidden 1536 / 40 experts (4-bit) and hidden 2048 / 64 experts / intermediate 1024 (8-bit)."""
    for shape, t in [(MoeShape("3b", 1536, 40, 8, 512, fmt="q4"), 12), (MoeShape("skew", 2048, 64, 8, 1024, fmt="q8"), 16)]:
        lw = layer_weights(oracle, shape, 1)
        x = workloads.hidden_states(shape, t, seed=1)
        check_block(oracle, ctx, shape, lw, x, arith=arith)


def test_host_entry_point_and_graph_replay_equal_the_device_path(oracle, ctx):
    shape = MoeShape("e2e", 512, 16, 4, 128, fmt="q8")
    ctx.set_arithmetic(ctx.ARITH_FAST)
    lw = layer_weights(oracle, shape, 2)
    x = workloads.hidden_states(shape, 33, seed=2)
    y0 = workloads.hidden_states(shape, 33, seed=9)
    layer = make_layer(ctx, lw, shape.topk, 64)
    y_dev, *_ = run_gpu(ctx, layer, x, y0)
    y_host = y0.copy()
    layer.forward_host(x, y_host)
    assert np.array_equal(y_host, y_dev)
    # Captured once, replayed twice: y accumulates the same projection each time.
    xd, yd = ctx.to_device(x), ctx.to_device(y0)
    before = ctx.launch_count()
    ctx.capture_begin()
    layer.forward(xd, yd)
    g = ctx.capture_end()
    assert ctx.launch_count() == before
    g.launch()
    ctx.sync()
    assert np.array_equal(yd.get(), y_dev)
    assert ctx.launch_count() > before
    g.launch()
    ctx.sync()
    ref = oracle_moe(oracle, lw, x, shape.topk)
    assert np.allclose(yd.get(), y0 + ref.proj + ref.proj, atol=4e-3)
    g.free()
    layer.free()


@pytest.mark.parametrize("t", [5, 300])
def test_block_with_fused_norm_equals_norm_then_forward(oracle, ctx, t):
    """tc_moe_block (RMSNorm fused into the router kernel; for t <= 256 the
    dispatch too) gives exactly what tc_rmsnorm followed by tc_moe_forward gives,
    which is the oracle's rmsnorm -> moe -> residual add."""
    shape = MoeShape("blk", 512, 16, 4, 128, fmt="q8")
    ctx.set_arithmetic(ctx.ARITH_FAST)
    lw = layer_weights(oracle, shape, 2)
    y0 = workloads.hidden_states(shape, t, seed=4)
    w = (1.0 + synth.normal(4, 2, 512, scale=0.1)).astype(np.float32)
    layer = make_layer(ctx, lw, shape.topk, t)
    wd = ctx.to_device(w)
    ya, xb = ctx.to_device(y0), ctx.empty(y0.shape)
    ctx.rmsnorm(ya, wd, 1e-6, xb)
    layer.forward(xb, ya)
    yb = ctx.to_device(y0)
    layer.block(wd, 1e-6, yb)
    ctx.sync()
    assert np.array_equal(ya.get(), yb.get())
    with oracle.fast_arithmetic_model():
        ref = oracle_moe(oracle, lw, oracle.rmsnorm_rows(y0, w, 1e-6), shape.topk)
    got, want = yb.get(), y0 + ref.proj
    assert np.abs(got - want).max() <= OUT_ABS
    assert np.mean(np.all(got == want, axis=1)) > 0.5
    layer.free()


def test_bad_arguments_are_refused(ctx):
    from tachyon_b200 import cuda

    shape = MoeShape("bad", 64, 4, 2, 32)
    lw = workloads.layer_weights(shape, seed=0)
    with pytest.raises(cuda.TachyonCudaError):  # more experts per token than experts
        cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, 5, 8)
    with pytest.raises(cuda.TachyonCudaError):  # down has the wrong row count
        cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.gate_up, 2, 8)
    with pytest.raises(cuda.TachyonCudaError):  # a bf16 expert matrix
        bf = weights.Matrix.from_f32(np.zeros(4 * 64 * 64, np.float32), 4 * 64, 64, "bf16")
        cuda.MoeLayer(ctx, lw.router, bf, lw.down, 2, 8)
    layer = cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, 2, 8)
    x = ctx.to_device(np.zeros((9, 64), np.float32))
    with pytest.raises(cuda.TachyonCudaError):  # more tokens than the layer was sized for
        layer.forward(x, x)
    with pytest.raises(cuda.TachyonCudaError):  # empty batch (src/model.rs:565)
        layer.forward(x, x, t=0)
    layer.free()


def test_launch_overlap_does_not_change_results(oracle, ctx):
    """Programmatic dependent launch only moves work earlier in time."""
    shape = MoeShape("1b-small", 512, 16, 4, 128, fmt="q8")
    lw = layer_weights(oracle, shape, 2)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    outs = []
    for on in [True, False, True]:
        ctx.set_launch_overlap(on)
        for t in [3, 64]:  # sparse walk, dense walk with weight prefetch before the dependency wait
            x = workloads.hidden_states(shape, t, seed=4)
            layer = make_layer(ctx, lw, shape.topk, t)
            yd = ctx.to_device(x.copy())
            ones = ctx.to_device(np.ones(shape.hidden, np.float32))
            for _ in range(3):  # back-to-back blocks: each kernel starts under the previous one's tail
                layer.block(ones, 1e-6, yd)
            ctx.sync()
            outs.append(yd.get())
            for d in (yd, ones):
                d.free()
            layer.free()
    ctx.set_launch_overlap(True)
    assert np.array_equal(outs[0], outs[2]) and np.array_equal(outs[0], outs[4])
    assert np.array_equal(outs[1], outs[3]) and np.array_equal(outs[1], outs[5])
    assert np.all(np.isfinite(outs[1]))


@pytest.mark.parametrize("fmt", ["q8", "q4"])
def test_layer_without_the_uploaded_expert_matrices(oracle, ctx, fmt):
    """The layer computes from its re-tiled copies: once detached, the matrices as uploaded
    can be freed, every default-arithmetic path still gives the same bits, and the
    CPU-lane mode (the one reader of the uploaded copies) is refused."""
    from tachyon_b200 import cuda

    shape = MoeShape("detach", 512, 16, 4, 128, fmt=fmt)
    lw = layer_weights(oracle, shape, 6)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    layer = make_layer(ctx, lw, shape.topk, 600)
    sizes = [5, 40, 600]  # one kernel, one kernel through the window, tensor-core kernels
    xs = [workloads.hidden_states(shape, t, seed=50 + t) for t in sizes]

    def run():
        outs = []
        for x in xs:
            xd, yd = ctx.to_device(x), ctx.to_device(np.zeros_like(x))
            layer.forward(xd, yd)
            ctx.sync()
            outs.append(yd.get())
            xd.free()
            yd.free()
        return outs

    before = run()
    layer.detach_experts()
    assert layer.gate_up.handle is None and layer.down.handle is None
    scratch = ctx.to_device(np.full(1 << 22, 7, np.uint8))  # something else may now live where they were
    after = run()
    for a, b in zip(before, after):
        assert np.array_equal(a, b)
    ctx.set_arithmetic(ctx.ARITH_CPU_LANES)
    xd, yd = ctx.to_device(xs[0]), ctx.to_device(np.zeros_like(xs[0]))
    with pytest.raises(cuda.TachyonCudaError, match="detached"):
        layer.forward(xd, yd)
    ctx.set_arithmetic(ctx.ARITH_FAST)
    for d in (xd, yd, scratch):
        d.free()
    layer.free()
