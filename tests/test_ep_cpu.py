"""Expert parallelism on CPU: two gloo ranks run the sharding rules and the
exchange plan of `tachyon_b200.ep` around the oracle's expert arithmetic and
must reproduce the single-process block exactly."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_ranges_cover_everything_remainder_to_low_ranks():
    from tachyon_b200 import ep

    for total, size in [(40, 2), (40, 4), (40, 8), (32, 8), (5, 3), (3, 4)]:
        parts = [ep.shard_range(total, r, size) for r in range(size)]
        assert parts[0][0] == 0 and sum(c for _, c in parts) == total
        for (f0, c0), (f1, c1) in zip(parts, parts[1:]):
            assert f1 == f0 + c0 and c0 >= c1 and c0 - c1 <= 1
    assert [ep.shard_range(40, r, 8)[1] for r in range(8)] == [5] * 8
    assert [ep.shard_range(5, r, 3)[1] for r in range(3)] == [2, 2, 1]


def test_local_expert_rows_are_the_stacked_matrix_rows(oracle):
    from tachyon_b200 import ep, workloads

    shape = workloads.MoeShape("t", 64, 5, 2, 32, fmt="q8")
    for fmt in ["q8", "q4"]:
        lw = workloads.layer_weights(shape, seed=1, fmt=fmt)
        gu, dn = ep.local_experts(lw.gate_up, lw.down, 5, 1, 3)  # rank 1 of 3 owns experts 2,3
        x = workloads.hidden_states(shape, 3, seed=2)
        full = oracle.OracleMatrix(lw.gate_up.kind, lw.gate_up.rows, 64, lw.gate_up.scales, lw.gate_up.data)
        part = oracle.OracleMatrix(gu.kind, gu.rows, 64, gu.scales, gu.data)
        assert gu.rows == 2 * 64 and dn.rows == 2 * 64
        assert np.array_equal(full.matmul_rows(x, row0=2 * 64, rows=2 * 64), part.matmul_rows(x))


def _rank_main(rank, size, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch
    import torch.distributed as dist

    from oracle import binding as oracle
    from tachyon_b200 import ep, workloads

    dist.init_process_group("gloo", rank=rank, world_size=size)
    shape = workloads.MoeShape("ep", 128, 6, 2, 64, fmt="q8")
    lw = workloads.layer_weights(shape, seed=3)
    tokens = 10
    x_all = workloads.hidden_states(shape, tokens, seed=4)
    t0, tn = ep.shard_range(tokens, rank, size)
    x = x_all[t0:t0 + tn]
    om = lambda m: oracle.OracleMatrix(m.kind, m.rows, m.cols, m.scales, m.data)
    E, k, H = shape.experts, shape.topk, shape.hidden
    # 1. local routing over all experts (router replicated)
    logits = om(lw.router).matmul_rows(x)
    picks = [oracle.route(logits[i], k) for i in range(tn)]
    ids = np.array([p[0] for p in picks]).reshape(tn, k)
    gates = np.array([p[1] for p in picks], np.float32).reshape(tn, k)
    order = np.argsort(ids.ravel(), kind="stable")  # slots sorted by global expert, token order kept
    hist = np.bincount(ids.ravel(), minlength=E).astype(np.int64)
    hist_all = [torch.zeros(E, dtype=torch.int64) for _ in range(size)]
    dist.all_gather(hist_all, torch.from_numpy(hist))
    hist_all = torch.stack(hist_all).numpy()
    send, recv = ep.exchange_plan(hist_all, rank)
    assert send.sum() == tn * k
    # 2. dispatch all-to-all-v of the slots' rows (and their expert ids, for the CPU model)
    rows = torch.from_numpy(np.ascontiguousarray(x[order // k]))
    eids = torch.from_numpy(ids.ravel()[order].astype(np.int64))
    got_rows = torch.empty(int(recv.sum()), H)
    got_eids = torch.empty(int(recv.sum()), dtype=torch.int64)
    dist.all_to_all_single(got_rows, rows, recv.tolist(), send.tolist())
    dist.all_to_all_single(got_eids, eids, recv.tolist(), send.tolist())
    # 3. this rank's experts over what it received
    first, count = ep.shard_range(E, rank, size)
    gu_l, dn_l = ep.local_experts(lw.gate_up, lw.down, E, rank, size)
    gu_o, dn_o = om(gu_l), om(dn_l)
    outs = np.zeros((int(recv.sum()), H), np.float32)
    gr = got_rows.numpy()
    for e in range(first, first + count):
        sel = np.nonzero(got_eids.numpy() == e)[0]
        if sel.size == 0:
            continue
        el = e - first
        gate_up = gu_o.matmul_rows(gr[sel], row0=el * 2 * shape.inter, rows=2 * shape.inter)
        hid = np.stack([oracle.silu_mul(r[:shape.inter], r[shape.inter:]) for r in gate_up])
        outs[sel] = dn_o.matmul_rows(hid, row0=el * H, rows=H)
    # 4. combine all-to-all-v back, then the reference's ascending-expert weighted sum
    back = torch.empty(tn * k, H)
    dist.all_to_all_single(back, torch.from_numpy(outs), send.tolist(), recv.tolist())
    back = back.numpy()
    pos = np.empty(tn * k, np.int64)
    pos[order] = np.arange(tn * k)
    proj = np.zeros((tn, H), np.float32)
    for i in range(tn):
        for j in np.argsort(ids[i]):
            proj[i] += np.float32(gates[i, j]) * back[pos[i * k + j]]
    np.save(os.path.join(out_dir, f"proj{rank}.npy"), proj)
    dist.barrier()
    dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_single_process_block(oracle, tmp_path):
    import torch.multiprocessing as mp

    from tachyon_b200 import ep, workloads

    port = 29500 + os.getpid() % 2000
    mp.start_processes(_rank_main, args=(2, port, str(tmp_path)), nprocs=2, join=True, start_method="spawn")
    shape = workloads.MoeShape("ep", 128, 6, 2, 64, fmt="q8")
    lw = workloads.layer_weights(shape, seed=3)
    x_all = workloads.hidden_states(shape, 10, seed=4)
    om = lambda m: oracle.OracleMatrix(m.kind, m.rows, m.cols, m.scales, m.data)
    ref = oracle.moe(om(lw.router), om(lw.gate_up), om(lw.down), x_all, shape.topk).proj
    got = np.concatenate([np.load(tmp_path / f"proj{r}.npy") for r in range(2)])
    assert np.array_equal(got, ref)
