"""Expert parallelism on real GPUs (needs at least two): every rank's shard of
the expert-parallel block must equal, bit for bit, the same tokens through the
single-GPU block on its own device."""
import os
import sys
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _device_count():
    import ctypes

    try:
        rt = ctypes.CDLL("libcudart.so.12")
    except OSError:
        try:
            import torch

            return torch.cuda.device_count()
        except Exception:
            return 0
    n = ctypes.c_int(0)
    return n.value if rt.cudaGetDeviceCount(ctypes.byref(n)) == 0 else 0


def _rank_main(rank, size, tmp, fmt, tokens, mode="alltoallv"):
    uniform = mode != "alltoallv"
    sys.path.insert(0, ROOT)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from tachyon_b200 import cuda, ep, workloads

    ctx = cuda.Context(rank)
    uid_path = os.path.join(tmp, "uid")
    if rank == 0:
        uid = ep.unique_id(ctx)
        with open(uid_path + ".tmp", "wb") as f:
            f.write(uid)
        os.rename(uid_path + ".tmp", uid_path)
    else:
        for _ in range(600):
            if os.path.exists(uid_path):
                break
            time.sleep(0.05)
        uid = open(uid_path, "rb").read()
    ep.init(ctx, uid, rank, size, uniform_batch=uniform)
    shape = workloads.MoeShape("ep", 512, 10, 4, 128, fmt=fmt)
    if mode == "peer":
        ep.enable_peer_exchange(ctx, shape.hidden, shape.topk, tokens // size)
    lw = workloads.layer_weights(shape, seed=6)
    full = cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.topk, tokens)
    gu, dn = ep.local_experts(lw.gate_up, lw.down, shape.experts, rank, size)
    t0, tn = ep.shard_range(tokens, rank, size)
    layer = ep.EpMoeLayer(ctx, lw.router, gu, dn, shape.experts, shape.topk, max(tn, 1))
    ones = ctx.to_device(np.ones(shape.hidden, np.float32))
    ep.barrier(ctx)  # ranks reach their first block together (the peer exchange's waits are bounded)

    def single_gpu(x_all, y0_all):
        xd, yd = ctx.to_device(x_all), ctx.to_device(y0_all)
        full.forward(xd, yd)
        ctx.sync()
        return yd.get()

    # Different inputs on every call: a consumer that read its buffers before the other
    # ranks' stores had arrived would find the previous call's rows, ids and outputs,
    # and those no longer give this call's answer.
    for it in range(3):
        x_all = workloads.hidden_states(shape, tokens, seed=70 + it)
        y0_all = workloads.hidden_states(shape, tokens, seed=80 + it)
        want = single_gpu(x_all, y0_all)
        xs, ys = ctx.to_device(x_all[t0:t0 + tn]), ctx.to_device(y0_all[t0:t0 + tn])
        layer.forward(xs, ys)
        ctx.sync()
        got = ys.get()
        assert np.array_equal(got, want[t0:t0 + tn]), (rank, it, np.abs(got - want[t0:t0 + tn]).max())
    # Three blocks in a row on the residual stream, each feeding the next, with no host
    # synchronisation between them: y += moe(rmsnorm(y)) three times.
    y0_all = workloads.hidden_states(shape, tokens, seed=90)
    yd = ctx.to_device(y0_all)
    for _ in range(3):
        full.block(ones, 1e-6, yd)
    ctx.sync()
    want = yd.get()
    ys = ctx.to_device(y0_all[t0:t0 + tn])
    for _ in range(3):
        layer.block(ones, 1e-6, ys)
    ctx.sync()
    assert np.array_equal(ys.get(), want[t0:t0 + tn]), (rank, "chained blocks")
    if uniform:
        # The fixed-size exchange reads nothing on the host: the block replays from a CUDA
        # graph, again with new inputs (and the previous replay's outputs) every time.
        xs, ys = ctx.to_device(x_all[t0:t0 + tn]), ctx.to_device(y0_all[t0:t0 + tn])
        ctx.capture_begin()
        layer.forward(xs, ys)
        graph = ctx.capture_end()
        for it in range(3):
            x_all = workloads.hidden_states(shape, tokens, seed=100 + it)
            y0_all = workloads.hidden_states(shape, tokens, seed=110 + it)
            want = single_gpu(x_all, y0_all)
            ctx.upload(xs.ptr, x_all[t0:t0 + tn])
            ctx.upload(ys.ptr, y0_all[t0:t0 + tn])
            graph.launch()
            ctx.sync()
            assert np.array_equal(ys.get(), want[t0:t0 + tn]), (rank, "graph replay", it)
        graph.free()
    layer.free()
    full.free()
    ctx.close()


def _wait_runs_out_main(rank, size, tmp):
    """One rank, peer-memory exchange, and a block whose rows are stored but never
    announced: the dispatch kernel's wait for the flag must run out (a short limit set
    by the test), the kernel must return, tc_sync must report it, and the next block
    must be right again. Nothing faults and nothing hangs: the flag simply stays unset."""
    sys.path.insert(0, ROOT)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    from tachyon_b200 import cuda, ep, workloads

    ctx = cuda.Context(rank)
    ep.init(ctx, ep.unique_id(ctx), 0, 1, uniform_batch=True)
    shape = workloads.MoeShape("ep", 512, 10, 4, 128, fmt="q8")
    tokens = 24
    ep.enable_peer_exchange(ctx, shape.hidden, shape.topk, tokens)
    lw = workloads.layer_weights(shape, seed=6)
    full = cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.topk, tokens)
    layer = ep.EpMoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.experts, shape.topk, tokens)
    x = workloads.hidden_states(shape, tokens, seed=1)
    y0 = workloads.hidden_states(shape, tokens, seed=2)
    xd, yd = ctx.to_device(x), ctx.to_device(y0)
    full.forward(xd, yd)
    ctx.sync()
    want = yd.get()
    ctx._check(ctx.lib.tc_ep_set_wait_limit(ctx.handle, 2000), "tc_ep_set_wait_limit")  # a few milliseconds
    ctx._check(ctx.lib.tc_ep_test_mute_signals(ctx.handle, 1), "tc_ep_test_mute_signals")
    ys = ctx.to_device(y0)
    t_begin = time.time()
    layer.forward(xd, ys)
    with pytest.raises(cuda.TachyonCudaError, match="status 2"):
        ctx.sync()
    assert time.time() - t_begin < 5.0
    ctx.sync()  # the status was cleared by the report: the context is usable
    ctx.upload(ys.ptr, y0)
    layer.forward(xd, ys)
    ctx.sync()
    assert np.array_equal(ys.get(), want)
    layer.free()
    full.free()
    ctx.close()


def test_a_wait_for_a_rank_that_never_signals_runs_out_and_the_context_recovers(tmp_path):
    if _device_count() < 1:
        pytest.skip("needs a GPU")
    import torch.multiprocessing as mp

    from tachyon_b200 import build

    build.build()
    mp.start_processes(_wait_runs_out_main, args=(1, str(tmp_path)), nprocs=1, join=True, start_method="spawn")


@pytest.mark.parametrize("fmt,tokens", [("q8", 64), ("q4", 37), ("q8", 600)])
def test_expert_parallel_block_equals_single_gpu(tmp_path, fmt, tokens):
    n = _device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    from tachyon_b200 import build

    build.build()
    size = 4 if n >= 4 else 2
    mp.start_processes(_rank_main, args=(size, str(tmp_path), fmt, tokens), nprocs=size, join=True,
                       start_method="spawn")


@pytest.mark.parametrize("fmt,tokens", [("q8", 64), ("q4", 36), ("q8", 1024)])
def test_fixed_size_exchange_equals_single_gpu_and_replays_from_a_graph(tmp_path, fmt, tokens):
    """Every rank brings tokens / size tokens: all-gather, dispatch over all of them,
    local experts, reduce-scatter; also captured and replayed."""
    n = _device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    from tachyon_b200 import build

    build.build()
    size = 4 if n >= 4 else 2
    mp.start_processes(_rank_main, args=(size, str(tmp_path), fmt, tokens, "fixed"), nprocs=size, join=True,
                       start_method="spawn")


@pytest.mark.parametrize("fmt,tokens", [("q8", 64), ("q4", 36), ("q8", 1024), ("q8", 16), ("q4", 128)])
def test_peer_memory_exchange_equals_single_gpu_and_replays_from_a_graph(tmp_path, fmt, tokens):
    """Rows and expert outputs stored straight into the other ranks' windows over NVLink,
    announced with flags; no collective call inside the block."""
    n = _device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    import torch.multiprocessing as mp

    from tachyon_b200 import build

    build.build()
    size = 4 if n >= 4 else 2
    mp.start_processes(_rank_main, args=(size, str(tmp_path), fmt, tokens, "peer"), nprocs=size, join=True,
                       start_method="spawn")


@pytest.mark.parametrize("mode", ["alltoallv", "fixed", "peer"])
@pytest.mark.parametrize("fmt,tokens", [("q8", 40), ("q4", 37), ("q8", 300), ("q8", 24), ("q4", 32)])
def test_one_rank_runs_every_exchange(tmp_path, fmt, tokens, mode):
    """A communicator of one rank on one GPU: the same kernels and buffers as with
    several ranks (the window is the rank's own), so the three exchanges are covered
    where only one GPU is present."""
    if _device_count() < 1:
        pytest.skip("needs a GPU")
    import torch.multiprocessing as mp

    from tachyon_b200 import build

    build.build()
    mp.start_processes(_rank_main, args=(1, str(tmp_path), fmt, tokens, mode), nprocs=1, join=True,
                       start_method="spawn")
