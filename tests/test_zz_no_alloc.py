"""The dispatch entry point that allocates nothing (`tc_dispatch_static`).

Some callers of this library cannot allocate device memory once they are
running: a backend that gave the whole device to KV-cache blocks at start-up
has nothing left to ask for, and a scheduler loop cannot afford the
device-wide stall of cudaMalloc/cudaFree. For them the dispatch keeps its one
piece of scratch in an array built into the library. This test calls that entry
point through the C ABI, twice in a row (the array is shared and keeps the
previous call's contents), and checks every output against what the regular
forward path (workspace allocated at layer creation) produced for the same
routing. It lives in a file pytest collects last, and passes alone in a fresh
process as well as after the other tests.
"""
import numpy as np
import pytest

from tachyon_b200 import workloads
from tachyon_b200.workloads import MoeShape

pytestmark = pytest.mark.gpu


def test_static_dispatch_matches_the_forward_path_twice_in_a_row():
    from tachyon_b200 import build, cuda

    build.build()
    ctx = cuda.Context(0)
    shape = MoeShape("noalloc", 256, 24, 4, 64, fmt="q8")
    lw = workloads.layer_weights(shape, seed=11)
    cap = 16384  # the entry point's limit
    layer = cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.topk, cap)
    # Output buffers for the entry point: allocated here, by the caller, before any call.
    bufs = {name: ctx.empty(n, dt) for name, n, dt in [
        ("ids", cap * 4, np.uint32), ("counts", 24, np.uint32), ("offsets", 25, np.uint32),
        ("perm", cap * 4, np.uint32), ("pos", cap * 4, np.uint32), ("slot_token", cap * 4, np.uint32),
        ("active", 25, np.int32)]}
    # Calls in a row, each reusing the scratch the one before left dirty: above and below
    # one CTA's worth of tokens, and the largest batch the built-in array allows.
    for call, t in enumerate([700, 300, 100, cap]):
        x = workloads.hidden_states(shape, t, seed=20 + call)
        xd, yd = ctx.to_device(x), ctx.to_device(np.zeros_like(x))
        layer.forward(xd, yd)  # the regular path: scratch from the workspace
        ctx.sync()
        ids, _, counts, _ = layer.last_routing(t)
        offsets, perm = layer.last_dispatch(t)
        ctx.upload(bufs["ids"].ptr, ids.ravel())
        ctx.dispatch_static(bufs["ids"], t, shape.experts, shape.topk, bufs["counts"], bufs["offsets"],
                            bufs["perm"], bufs["pos"], bufs["slot_token"], bufs["active"])
        ctx.sync()
        n = t * shape.topk
        assert np.array_equal(bufs["counts"].get(), counts)
        assert np.array_equal(bufs["offsets"].get(), offsets)
        got_perm = bufs["perm"].get()[:n]
        assert np.array_equal(got_perm, perm)
        assert np.array_equal(bufs["slot_token"].get()[:n], perm // shape.topk)
        pos = bufs["pos"].get()[:n]
        assert np.array_equal(got_perm[pos], np.arange(n, dtype=np.uint32))
        active = bufs["active"].get()
        assert active[shape.experts] == np.count_nonzero(counts)
        assert np.array_equal(active[:active[shape.experts]], np.nonzero(counts)[0])
        xd.free()
        yd.free()
    # Sizes beyond the built-in array are refused with a message, not attempted.
    with pytest.raises(cuda.TachyonCudaError, match="16384"):
        ctx.dispatch_static(bufs["ids"], 16385, shape.experts, shape.topk, bufs["counts"], bufs["offsets"],
                            bufs["perm"], bufs["pos"], bufs["slot_token"], bufs["active"])
    with pytest.raises(cuda.TachyonCudaError):
        ctx.dispatch_static(bufs["ids"], 10, 257, shape.topk, bufs["counts"], bufs["offsets"],
                            bufs["perm"], bufs["pos"], bufs["slot_token"], bufs["active"])
    # An expert id the caller got wrong (out of range, or one expert twice for a token) is
    # checked before it is used as an index: the slot is left out, tc_sync reports it,
    # and the next call is clean.
    t = 300
    x = workloads.hidden_states(shape, t, seed=31)
    xd, yd = ctx.to_device(x), ctx.to_device(np.zeros_like(x))
    layer.forward(xd, yd)
    ctx.sync()
    ids, _, counts, _ = layer.last_routing(t)
    offsets, perm = layer.last_dispatch(t)
    bad = ids.copy()
    bad[7, 2] = shape.experts + 5       # out of range
    bad[9, 3] = bad[9, 0]               # the same expert twice
    ctx.upload(bufs["ids"].ptr, bad.ravel())
    ctx.dispatch_static(bufs["ids"], t, shape.experts, shape.topk, bufs["counts"], bufs["offsets"],
                        bufs["perm"], bufs["pos"], bufs["slot_token"], bufs["active"])
    with pytest.raises(cuda.TachyonCudaError, match="status 3"):
        ctx.sync()
    want_counts = counts.copy()
    want_counts[ids[7, 2]] -= 1
    want_counts[ids[9, 3]] -= 1
    assert np.array_equal(bufs["counts"].get(), want_counts)
    ctx.upload(bufs["ids"].ptr, ids.ravel())
    ctx.dispatch_static(bufs["ids"], t, shape.experts, shape.topk, bufs["counts"], bufs["offsets"],
                        bufs["perm"], bufs["pos"], bufs["slot_token"], bufs["active"])
    ctx.sync()
    assert np.array_equal(bufs["counts"].get(), counts)
    assert np.array_equal(bufs["perm"].get()[:t * shape.topk], perm)
    layer.free()
    ctx.close()
