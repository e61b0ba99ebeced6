"""The graph-per-bucket step on a fake context: bucket choice, padding, capture once per bucket."""
import numpy as np
import pytest

from tachyon_b200.buckets import GraphBuckets


class FakeArray:
    def __init__(self, mem, ptr, shape):
        self.mem, self.ptr, self.shape = mem, ptr, shape

    def free(self):
        pass


class FakeGraph:
    def __init__(self, ops):
        self.ops, self.launched, self.freed = ops, 0, False

    def launch(self):
        self.launched += 1
        for op in self.ops:
            op()

    def free(self):
        self.freed = True


class FakeContext:
    """Device memory is one byte array; work enqueued while capturing is recorded, not run."""

    def __init__(self):
        self.mem = np.zeros(1 << 20, np.uint8)
        self.top = 256
        self.capturing = None
        self.captures = 0

    def empty(self, shape, dtype=np.float32):
        n = int(np.prod(shape)) * np.dtype(dtype).itemsize
        a = FakeArray(self.mem, self.top, tuple(shape))
        self.top += (n + 255) // 256 * 256
        return a

    def _do(self, op):
        if self.capturing is not None:
            self.capturing.append(op)
        else:
            op()

    def copy_bytes(self, dst, src, n):
        self._do(lambda: self.mem.__setitem__(slice(dst, dst + n), self.mem[src:src + n].copy()))

    def memset(self, dst, value, n):
        assert self.capturing is None
        self.mem[dst:dst + n] = value

    def upload(self, dst, host):
        assert self.capturing is None
        b = np.ascontiguousarray(host).view(np.uint8).ravel()
        self.mem[dst:dst + b.size] = b

    def download(self, host, src):
        host.view(np.uint8).ravel()[:] = self.mem[src:src + host.nbytes]

    def sync(self):
        pass

    def capture_begin(self):
        self.capturing = []

    def capture_end(self):
        ops, self.capturing = self.capturing, None
        self.captures += 1
        return FakeGraph(ops)

    def rows(self, arr, t, hidden):
        return self.mem[arr.ptr:arr.ptr + t * hidden * 4].view(np.float32).reshape(t, hidden)


class FakeLayer:
    """y[:t] += 1 + row index: shows which rows a block saw and how many times it ran."""

    def __init__(self, ctx, hidden, max_tokens):
        self.ctx, self.hidden, self.max_tokens, self.calls = ctx, hidden, max_tokens, []

    def block(self, w, eps, y, t):
        self.calls.append(t)

        def op():
            self.ctx.rows(y, t, self.hidden)[:] += 1.0 + np.arange(t, dtype=np.float32)[:, None]

        self.ctx._do(op)


def make(buckets=(1, 2, 4, 8, 16), max_tokens=16, layers=2, hidden=8):
    ctx = FakeContext()
    ls = [FakeLayer(ctx, hidden, max_tokens) for _ in range(layers)]
    return ctx, ls, GraphBuckets(ctx, ls, [None] * layers, 1e-6, hidden, buckets)


def test_bucket_choice():
    _, _, gb = make()
    assert [gb.bucket_for(t) for t in (1, 2, 3, 4, 5, 8, 9, 16)] == [1, 2, 4, 4, 8, 8, 16, 16]
    with pytest.raises(ValueError):
        gb.bucket_for(17)
    with pytest.raises(ValueError):
        gb.bucket_for(0)


def test_buckets_above_the_layers_limit_are_dropped():
    _, _, gb = make(buckets=(1, 8, 64, 128), max_tokens=32)
    assert gb.buckets == (1, 8)
    with pytest.raises(ValueError):
        make(buckets=(64,), max_tokens=32)


def test_step_pads_with_zeros_and_returns_the_real_rows():
    ctx, layers, gb = make()
    x = np.arange(3 * 8, dtype=np.float32).reshape(3, 8)
    y = gb.step(x)
    assert np.array_equal(y, x + 2 * (1.0 + np.arange(3, dtype=np.float32)[:, None]))  # two layers
    assert np.array_equal(ctx.rows(gb.x_in, 4, 8)[3], np.zeros(8, np.float32))         # the pad row went in as zeros
    # A smaller step into the same bucket must not see the previous step's rows.
    y1 = gb.step(x[:1] + 100)
    assert y1.shape == (1, 8) and np.array_equal(y1, x[:1] + 100 + 2.0)


def test_one_capture_per_bucket_and_replays_after_that():
    ctx, layers, gb = make()
    x = np.ones((5, 8), np.float32)
    for _ in range(3):
        gb.step(x)       # bucket 8
    gb.step(x[:2])       # bucket 2
    gb.step(x[:7])       # bucket 8 again
    assert ctx.captures == 2 and sorted(gb.graphs) == [2, 8]
    assert gb.launches[8] == 4 and gb.launches[2] == 1
    # Each bucket: one eager pass and one captured pass per layer, whatever the number of steps.
    assert layers[0].calls.count(8) == 2 and layers[0].calls.count(2) == 2
    graphs = list(gb.graphs.values())
    gb.free()
    assert all(g.freed for g in graphs)
