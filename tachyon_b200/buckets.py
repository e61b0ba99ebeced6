"""A CUDA graph per batch-size bucket for the MoE blocks of a model.

Tachyon's scheduler runs one ``Backend::forward`` per step on however many
sequences are decoding (``src/scheduler.rs:625-630``); the batch size changes
from step to step. A captured graph is tied to its batch size, so a backend
that wants one launch per step keeps a graph for each of a few bucket sizes
and pads a step up to the next bucket. The pad rows are zeros: a token's
result does not depend on the other rows of its batch (every kernel here keeps
one arithmetic chain per output, whatever the batch), so the real rows come
out with the same bits as an eager call on exactly those rows, and the pad
rows' results are never read.

Graphs are captured on first use of a bucket. Every layer must exist before
the first capture (creating a layer may grow the context's scratch, which
invalidates earlier graphs).
"""
from __future__ import annotations

import numpy as np

DEFAULT_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128)


class GraphBuckets:
    """``step(x)``: x[t, hidden] += the MoE blocks of every layer, t padded to a bucket.

    ``layers`` are ``MoeLayer``-like objects with ``block(norm_weight, eps, y, t)`` and
    ``max_tokens``; ``norm_weights`` their RMSNorm weights on the device. ``ctx`` needs
    ``empty``, ``upload``, ``download``, ``memset``, ``copy_bytes``, ``capture_begin``,
    ``capture_end`` and ``sync`` (``tachyon_b200.cuda.Context`` has them).
    """

    def __init__(self, ctx, layers, norm_weights, eps: float, hidden: int, buckets=DEFAULT_BUCKETS):
        if len(layers) != len(norm_weights) or not layers:
            raise ValueError("one norm weight per layer, at least one layer")
        limit = min(layer.max_tokens for layer in layers)
        self.buckets = tuple(sorted({int(b) for b in buckets if 1 <= int(b) <= limit}))
        if not self.buckets:
            raise ValueError(f"no bucket fits layers created for {limit} tokens")
        self.ctx, self.layers, self.norm_weights = ctx, list(layers), list(norm_weights)
        self.eps, self.hidden = float(eps), int(hidden)
        rows = self.buckets[-1]
        self.x_in = ctx.empty((rows, hidden), np.float32)  # the step's rows, then zeros up to the bucket
        self.x = ctx.empty((rows, hidden), np.float32)     # the residual stream the graph works on
        self.graphs = {}
        self.launches = {b: 0 for b in self.buckets}

    def bucket_for(self, t: int) -> int:
        """The smallest bucket that holds t rows."""
        if t < 1:
            raise ValueError("empty batch")
        for b in self.buckets:
            if b >= t:
                return b
        raise ValueError(f"{t} rows, the largest bucket is {self.buckets[-1]}")

    def _enqueue(self, b: int):
        self.ctx.copy_bytes(self.x.ptr, self.x_in.ptr, b * self.hidden * 4)
        for layer, w in zip(self.layers, self.norm_weights):
            layer.block(w, self.eps, self.x, t=b)  # x += moe(rmsnorm(x)): src/model.rs:662-681

    def graph(self, b: int):
        """The bucket's graph, captured on first use (after one eager pass of the same work)."""
        g = self.graphs.get(b)
        if g is None:
            self._enqueue(b)
            self.ctx.sync()
            self.ctx.capture_begin()
            self._enqueue(b)
            g = self.graphs[b] = self.ctx.capture_end()
        return g

    def step(self, x_host: np.ndarray) -> np.ndarray:
        x_host = np.ascontiguousarray(x_host, np.float32)
        t = x_host.shape[0]
        if x_host.ndim != 2 or x_host.shape[1] != self.hidden:
            raise ValueError(f"expected [t, {self.hidden}] rows")
        b = self.bucket_for(t)
        g = self.graph(b)
        row = self.hidden * 4
        self.ctx.upload(self.x_in.ptr, x_host)
        if b > t:
            self.ctx.memset(self.x_in.ptr + t * row, 0, (b - t) * row)
        g.launch()
        self.ctx.sync()
        self.launches[b] += 1
        out = np.empty((t, self.hidden), np.float32)
        self.ctx.download(out, self.x.ptr)
        return out

    def free(self):
        for g in self.graphs.values():
            g.free()
        self.graphs.clear()
        for d in (self.x_in, self.x):
            d.free()
