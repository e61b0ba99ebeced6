#!/usr/bin/env python
"""Granite-MoE tokens/s on B200, next to the CPU path timed on the host.

A step is one pass of the hot path over one decode batch: every MoE block of
the Granite 1b-a400m shape (24 layers: RMSNorm -> router/top-8 -> dispatch ->
expert SwiGLU over int8 weights -> combine -> residual) for `--batch` tokens.
Attention, embeddings and the output head are not part of this path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

Prints one JSON line (rank 0). `value` is whole-job tokens/s with inputs
resident in HBM (CUDA-graph replay, CUDA events); `e2e` is the same metric
through host buffers (pinned host -> device copy of the step's hidden states,
the stack, device -> host read of the result) inside the timed region.
`--impl reference` times the CPU path (the oracle's restatement of Tachyon's
AVX2 code: no Rust toolchain exists here to build the original) on the host
cores, same config and metric.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from tachyon_b200 import synth, workloads  # noqa: E402

METRIC = "granite_moe_decode_tokens_per_s"

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the gate_up expert kernel,
# from the ncu capture summarised in profiles/expert_fast_kernel_granite1b_q8_batch32.md
# (read 35,761,408 B, written 0 B: the 0.5 MB of output stays in L2). Keyed by workload; other
# workloads have no capture and report null.
NCU_DRAM_BYTES_PER_LAUNCH = {("granite-1b-a400m", "q8", 32): 35761408}
UNIT = "tokens/s"
CLOCK_WINDOW_STEPS = 300  # untimed steps after the timed ones, for the clock sampler
EPS = 1e-6


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--batch", type=int, default=32, help="decode tokens per step per GPU")
    ap.add_argument("--layers", type=int, default=workloads.GRANITE_1B.layers)
    ap.add_argument("--model", default="1b-a400m", choices=["1b-a400m", "3b-a800m-q8"],
                    help="expert shape: the headline granite-1b-a400m, or the 3b-a800m shape with int8 weights")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--ep-exchange", default="peer", choices=["peer", "fixed", "alltoallv"],
                    help="N > 1: NVLink stores into mapped peer windows with flag waits (no NCCL call in a block), "
                         "all-gather + reduce-scatter of fixed size (both from a CUDA graph), or the "
                         "variable-size all-to-all enqueued directly")
    ap.add_argument("--four-kernels", action="store_true",
                    help="decode-size blocks as four kernels (router, gate_up, down, combine) instead of one")
    ap.add_argument("--no-overlap", action="store_true",
                    help="plain stream order between the kernels of a block (no programmatic dependent launch)")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.rows, self.proc = device, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.device}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": float(np.median(sm)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons),
                "samples": len(sm)}


def build_weights(shape, layers, seed, threads):
    t0 = time.time()
    out = [workloads.layer_weights(shape, seed=seed, layer=l, threads=threads) for l in range(layers)]
    return out, time.time() - t0


def cpu_stack_step(oracle, mats, x0, topk, threads):
    """One pass of the CPU path over the stack: xb = rmsnorm(x); x += moe(xb)."""
    x = x0.copy()
    ones = np.ones(x.shape[1], np.float32)
    for router, gate_up, down in mats:
        xb = oracle.rmsnorm_rows(x, ones, EPS)
        x += oracle.moe(router, gate_up, down, xb, topk, threads=threads).proj
    return x


def run_cpu(args, shape, weights_host, x0, steps, warmup, budget_s=25.0):
    from oracle import binding as oracle

    oracle.build()
    threads = oracle.default_threads()
    mats = [tuple(oracle.OracleMatrix(m.kind, m.rows, m.cols, m.scales, m.data)
                  for m in (lw.router, lw.gate_up, lw.down)) for lw in weights_host]
    for _ in range(warmup):
        cpu_stack_step(oracle, mats, x0, shape.topk, threads)
    times = []
    t_begin = time.time()
    for _ in range(steps):
        t0 = time.perf_counter()
        cpu_stack_step(oracle, mats, x0, shape.topk, threads)
        times.append(time.perf_counter() - t0)
        if time.time() - t_begin > budget_s:
            break
    mean = float(np.mean(times))
    return {"tokens_per_s": x0.shape[0] / mean, "ms_per_step": mean * 1e3, "steps": len(times),
            "threads": threads, "best_ms": float(np.min(times)) * 1e3}


def config_dict(args, shape, world):
    return {
        "workload": f"{shape.name} MoE stack, decode: {args.layers} layers x (RMSNorm + MoE block: "
                    f"router top-{shape.topk} of {shape.experts}, SwiGLU experts inter {shape.inter}, "
                    f"int8 weights), hidden {shape.hidden}, batch {args.batch} tokens/step/GPU",
        "batch_per_gpu": args.batch,
        "global_batch": args.batch * world,
        "layers": args.layers,
        "weights": "q8 (int8 + f16 scale per 32), router bf16",
        "parallelism": "1 GPU" if world == 1 else
                       f"ep{world}: experts sharded over {world} GPUs (contiguous ranges), tokens data-parallel, "
                       + ("rows and expert outputs stored into mapped peer windows over NVLink with flag waits "
                          "(no NCCL call inside a block), one CUDA graph per step" if args.ep_exchange == "peer"
                          else "NCCL all-gather of the 8-bit rows and reduce-scatter of the expert outputs per block, "
                          "one CUDA graph per step" if args.ep_exchange == "fixed"
                          else "NCCL all-to-all-v dispatch and combine per block"),
        "l2": "each step streams every layer's expert weights (1.28 GB at 24 layers), more than the 126 MB L2",
    }


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    shape = workloads.GRANITE_1B if args.model == "1b-a400m" else workloads.GRANITE_3B_Q8
    host_threads = max(1, (os.cpu_count() or 8) // max(1, world) - 1)

    if args.impl == "reference":
        if rank != 0:
            return
        weights_host, _ = build_weights(shape, args.layers, args.seed, max(1, (os.cpu_count() or 8) - 2))
        x0 = workloads.hidden_states(shape, args.batch, seed=args.seed)
        r = run_cpu(args, shape, weights_host, x0, args.steps, args.warmup, budget_s=150.0)
        line = {
            "impl": "reference", "metric": METRIC, "value": r["tokens_per_s"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": r["steps"], "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "int8 x int8 -> i32, f32 scales", "data": "synthetic",
            "config": config_dict(args, shape, 1),
            "cpu_baseline": {"value": r["tokens_per_s"], "unit": UNIT, "cores": r["threads"], "kind": "port",
                             "sample": f"{r['steps']} full steps of the same {args.layers}-layer stack at batch "
                                       f"{args.batch}; C++ restatement of Tachyon's AVX2 path, not the Rust binary"},
            "e2e": {"value": r["tokens_per_s"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        }
        print(json.dumps(line))
        return

    from tachyon_b200 import build as cuda_build
    from tachyon_b200 import cuda

    if rank == 0:
        cuda_build.build()
    dist = None
    if world > 1:
        import torch.distributed as dist  # plumbing only: barrier and max over ranks

        dist.init_process_group("gloo")
        dist.barrier()
    ctx = cuda.Context(local_rank)
    if args.no_overlap:
        ctx.set_launch_overlap(False)
    if args.four_kernels:
        ctx.set_decode_block(False)

    if world == 1:
        weights_host, gen_s = build_weights(shape, args.layers, args.seed, host_threads)
        layers = [cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.topk, args.batch) for lw in weights_host]
    else:
        from tachyon_b200 import ep

        box = [ep.unique_id(ctx) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ep.init(ctx, box[0], rank, world, uniform_batch=args.ep_exchange != "alltoallv")
        if args.ep_exchange == "peer":
            ep.enable_peer_exchange(ctx, shape.hidden, shape.topk, args.batch)
        first, count = ep.shard_range(shape.experts, rank, world)
        t0 = time.time()
        layers = []
        for l in range(args.layers):
            lw = workloads.layer_weights_local(shape, first, count, seed=args.seed, layer=l, threads=host_threads)
            layers.append(ep.EpMoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.experts, shape.topk, args.batch))
        gen_s = time.time() - t0
        weights_host = None
    ones = ctx.to_device(np.ones(shape.hidden, np.float32))
    x_host = ctx.pinned((args.batch, shape.hidden))
    x_host[:] = workloads.hidden_states(shape, args.batch, seed=args.seed + rank)
    y_host = ctx.pinned((args.batch, shape.hidden))
    x_in = ctx.to_device(x_host)
    x = ctx.empty((args.batch, shape.hidden))

    def enqueue_stack():
        ctx.copy(x, x_in)
        for layer in layers:
            layer.block(ones, EPS, x)  # x += moe(rmsnorm(x)): src/model.rs:662-681

    if dist:
        dist.barrier()  # ranks enter their first block together: the peer exchange's waits are bounded
    # ---- eager pass with per-kernel events: which kernel dominates, and its bandwidth
    enqueue_stack()
    ctx.sync()
    distinct, prof = [], {}
    if world == 1:
        ctx.profile_enable(True)
        for s in range(3):
            ctx.copy(x, x_in)
            for layer in layers:
                layer.block(ones, EPS, x)
                if s == 0:
                    _, _, counts, _ = layer.last_routing(args.batch)
                    distinct.append(int(np.count_nonzero(counts)))
        prof = ctx.profile_read()
        ctx.profile_enable(False)

    # ---- the timed stack, device-resident inputs: one CUDA graph per step. (The variable-size
    # expert-parallel exchange reads its sizes on the host, so that one is enqueued directly.)
    class Eager:
        def launch(self):
            enqueue_stack()

    if world == 1 or args.ep_exchange != "alltoallv":
        ctx.capture_begin()
        enqueue_stack()
        graph = ctx.capture_end()
    else:
        graph = Eager()
    for _ in range(max(args.warmup, 3)):
        graph.launch()
    ctx.sync()
    if dist:
        dist.barrier()
    launches0 = ctx.launch_count()
    with ClockSampler(local_rank) as clocks:
        ctx.timer_start()
        for _ in range(args.steps):
            graph.launch()
        ms = ctx.timer_stop_ms()
        launches = ctx.launch_count() - launches0
        # The timed region lasts tens of milliseconds and nvidia-smi samples every 100 ms: keep the
        # same load running (untimed; the same count on every rank) until a few samples are in.
        for _ in range(CLOCK_WINDOW_STEPS if args.batch * args.layers <= 256 * 24 else 20):
            graph.launch()
        ctx.sync()
    ctx.sync()
    if dist:
        import torch

        tmax = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        ms = float(tmax.item())
        dist.barrier()
    ms_per_step = ms / args.steps
    value = args.batch * world / (ms_per_step * 1e-3)

    # ---- end to end through host buffers
    for _ in range(2):
        ctx.upload(x_in.ptr, x_host)
        graph.launch()
        ctx.download(y_host, x.ptr)
    if dist:
        dist.barrier()
    ctx.timer_start()
    for _ in range(args.steps):
        ctx.upload(x_in.ptr, x_host)
        graph.launch()
        ctx.download(y_host, x.ptr)
    e2e_ms = ctx.timer_stop_ms()
    if dist:
        import torch

        tmax = torch.tensor([e2e_ms], dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        e2e_ms = float(tmax.item())
    e2e_value = args.batch * world / (e2e_ms / args.steps * 1e-3)
    assert np.all(np.isfinite(y_host))

    if rank != 0:
        return
    if world > 1:
        peak, peak_kind = measured_peaks()
        # Bytes every rank's HBM must deliver per step: its share of the selected experts' weights
        # (all experts are hit at these batch sizes), routers, activations.
        step_bytes = args.layers * workloads.decode_algorithmic_bytes(shape, args.batch * world, shape.experts)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> i32, f32 scales", "data": "synthetic",
            "config": config_dict(args, shape, world),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(x_host.nbytes),
                    "d2h_bytes_per_step": int(y_host.nbytes), "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": int(launches),
            "clocks": clocks.summary(),
            "roofline": {"bound": "hbm", "kernel": "whole step, all ranks", "achieved": step_bytes / (ms_per_step * 1e-3) / 1e9,
                         "peak": peak * world, "unit": "GB/s", "frac": step_bytes / (ms_per_step * 1e-3) / 1e9 / (peak * world),
                         "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs x {world} GPUs)", "traffic": None},
            "setup_s": {"weights_host": gen_s},
        }
        print(json.dumps(line))
        return

    # ---- roofline of the dominant kernel (gate_up expert products)
    peak, peak_kind = measured_peaks()
    eb_gu = 2 * shape.inter * shape.hidden * 34 // 32            # one expert's gate_up rows as stored
    eb_dn = shape.hidden * shape.inter * 34 // 32
    nbp = -(-(shape.hidden // 32) // 8) * 8
    mean_u = float(np.mean(distinct))
    gu_bytes = (mean_u * eb_gu + args.batch * (shape.hidden + 4 * nbp)
                + args.batch * shape.topk * shape.inter * 4)
    stage_ms = {k: v[0] / max(1, v[1]) for k, v in prof.items() if v[1]}
    if "decode_block" in stage_ms:
        one_kernel_block = True
        gu_bytes = float(np.mean([workloads.decode_algorithmic_bytes(shape, args.batch, u) for u in distinct]))
        stage_ms["gate_up"] = stage_ms["decode_block"]
        stage_ms["down"] = stage_ms["decode_block"]
    gu_ms = stage_ms["gate_up"]
    achieved = gu_bytes / (gu_ms * 1e-3) / 1e9
    total_prof = sum(v[0] for v in prof.values())
    roofline = {
        "bound": "hbm", "kernel": "expert_kernel<q8, gate_up>", "achieved": achieved, "peak": peak,
        "unit": "GB/s", "frac": achieved / peak, "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)",
        "frac_of_8TBs_nominal": achieved / 8000.0,
        "algorithmic_bytes_per_launch": gu_bytes, "avg_launch_us": gu_ms * 1e3,
        "distinct_experts_per_layer": mean_u,
        "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((shape.name, shape.fmt, args.batch)),
        "kernel_share_of_step": {k: v[0] / total_prof for k, v in prof.items() if v[1]},
        "down_kernel": {"achieved": (mean_u * eb_dn + args.batch * shape.topk * (shape.inter + 4 * 8)
                                     + args.batch * shape.topk * shape.hidden * 4) / (stage_ms["down"] * 1e-3) / 1e9,
                        "avg_launch_us": stage_ms["down"] * 1e3},
        "whole_step": {"algorithmic_bytes": sum(workloads.decode_algorithmic_bytes(shape, args.batch, u) for u in distinct),
                       "achieved": sum(workloads.decode_algorithmic_bytes(shape, args.batch, u) for u in distinct)
                                   / (ms_per_step * 1e-3) / 1e9},
    }
    roofline["whole_step"]["frac"] = roofline["whole_step"]["achieved"] / peak

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int8 -> i32, f32 scales", "data": "synthetic",
        "config": config_dict(args, shape, world),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(x_host.nbytes),
                "d2h_bytes_per_step": int(y_host.nbytes), "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
        "roofline": roofline,
        "setup_s": {"weights_host": gen_s},
    }
    if world == 1 and not args.no_cpu_baseline:
        r = run_cpu(args, shape, weights_host, np.array(x_host), steps=30, warmup=1, budget_s=20.0)
        line["cpu_baseline"] = {
            "value": r["tokens_per_s"], "unit": UNIT, "cores": r["threads"], "kind": "port",
            "sample": f"{r['steps']} full steps of the same {args.layers}-layer stack at batch {args.batch} "
                      f"(mean {r['ms_per_step']:.1f} ms/step); C++ restatement of Tachyon's AVX2 path",
        }
    print(json.dumps(line))


if __name__ == "__main__":
    main()
