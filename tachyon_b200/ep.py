"""Expert parallelism: host-side sharding rules and the per-rank layer.

Experts are split into contiguous ranges, the remainder going to the low ranks;
tokens are split the same way. The same rules run inside the library
(``tc_ep_expert_range``); they are restated here so that weights can be cut per
rank on the host and so that the exchange plan can be tested on CPU.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .cuda import Context, DeviceMatrix, MoeLayer, TachyonCudaError
from .weights import KIND_Q4, KIND_Q8, Matrix, q4_words


def shard_range(total: int, rank: int, size: int) -> tuple[int, int]:
    """(first, count) of rank's contiguous share of ``total`` items."""
    base, rem = divmod(total, size)
    return rank * base + min(rank, rem), base + (1 if rank < rem else 0)


def matrix_rows(m: Matrix, row0: int, rows: int) -> Matrix:
    """Rows [row0, row0+rows) of a quantized matrix, in the same storage format."""
    if m.kind == KIND_Q8:
        nb = m.cols // 32
        return Matrix(KIND_Q8, rows, m.cols, m.scales[row0 * nb:(row0 + rows) * nb].copy(),
                      m.data[row0 * m.cols:(row0 + rows) * m.cols].copy())
    if m.kind == KIND_Q4:
        w = q4_words(m.cols)
        return Matrix(KIND_Q4, rows, m.cols, m.scales[row0 * w:(row0 + rows) * w].copy(),
                      m.data[row0 * m.cols // 2:(row0 + rows) * m.cols // 2].copy())
    return Matrix(m.kind, rows, m.cols, None, m.data[row0 * m.cols:(row0 + rows) * m.cols].copy())


def local_experts(gate_up: Matrix, down: Matrix, experts: int, rank: int, size: int):
    """This rank's rows of the stacked expert matrices (src/model.rs:35-40)."""
    first, count = shard_range(experts, rank, size)
    gu_rows, dn_rows = gate_up.rows // experts, down.rows // experts
    return (matrix_rows(gate_up, first * gu_rows, count * gu_rows),
            matrix_rows(down, first * dn_rows, count * dn_rows))


def exchange_plan(hist_all: np.ndarray, rank: int):
    """From every rank's histogram over all experts [size, experts]: how many
    slots this rank sends to and receives from each rank (the all-to-all-v's
    split sizes), as the library computes them on the host."""
    size, experts = hist_all.shape
    send = np.zeros(size, np.int64)
    recv = np.zeros(size, np.int64)
    my_first, my_count = shard_range(experts, rank, size)
    for r in range(size):
        first, count = shard_range(experts, r, size)
        send[r] = hist_all[rank, first:first + count].sum()
        recv[r] = hist_all[r, my_first:my_first + my_count].sum()
    return send, recv


def unique_id(ctx: Context) -> bytes:
    buf = C.create_string_buffer(128)
    if ctx.lib.tc_ep_unique_id(buf) != 0:
        raise TachyonCudaError("tc_ep_unique_id failed (is NCCL available?)")
    return buf.raw


def init(ctx: Context, uid: bytes, rank: int, size: int, uniform_batch: bool = False):
    """Collective. uniform_batch=True promises that every rank calls each block with the
    same number of tokens: decode-size blocks then use the fixed-size exchange (an
    all-gather and a reduce-scatter, no host read, capturable in a CUDA graph)."""
    ctx._check(ctx.lib.tc_ep_init(ctx.handle, uid, rank, size), "tc_ep_init")
    ctx.ep_rank, ctx.ep_size = rank, size
    if uniform_batch:
        ctx._check(ctx.lib.tc_ep_set_uniform_batch(ctx.handle, 1), "tc_ep_set_uniform_batch")


def enable_peer_exchange(ctx: Context, hidden: int, experts_per_token: int, max_tokens: int):
    """Collective, before the layers are created: blocks of up to max_tokens tokens per
    rank exchange rows and expert outputs by NVLink stores into mapped peer windows
    (no NCCL call inside a block). Implies uniform batches."""
    ctx._check(ctx.lib.tc_ep_enable_peer_exchange(ctx.handle, hidden, experts_per_token, max_tokens),
               "tc_ep_enable_peer_exchange")


def barrier(ctx: Context):
    ctx._check(ctx.lib.tc_ep_barrier(ctx.handle), "tc_ep_barrier")


class EpMoeLayer(MoeLayer):
    """One MoE block with this rank's experts; forward()/block() exchange rows over NCCL."""

    def __init__(self, ctx: Context, router: Matrix, gate_up_local: Matrix, down_local: Matrix, experts: int,
                 experts_per_token: int, max_tokens: int):
        self.ctx = ctx
        self.hidden, self.experts = router.cols, experts
        self.inter, self.topk = down_local.cols, experts_per_token
        self.max_tokens = max_tokens
        self.router = DeviceMatrix(ctx, router)
        self.gate_up = DeviceMatrix(ctx, gate_up_local)
        self.down = DeviceMatrix(ctx, down_local)
        self.weight_bytes = self.router.nbytes + self.gate_up.nbytes + self.down.nbytes
        self.handle = ctx.lib.tc_moe_ep_layer_create(
            ctx.handle, self.hidden, experts, self.topk, self.inter, self.router.handle, self.gate_up.handle,
            self.down.handle, max_tokens)
        if not self.handle:
            raise TachyonCudaError(f"tc_moe_ep_layer_create: {ctx.last_error()}")
