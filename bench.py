#!/usr/bin/env python
"""Granite-MoE tokens/s on B200, next to the CPU path timed on the host.

A step is one pass of the hot path over one decode batch: every MoE block of
the Granite 1b-a400m shape (24 layers: RMSNorm -> router/top-8 -> expert SwiGLU
over int8 weights -> combine -> residual) for `--batch` tokens. Attention,
embeddings and the output head are not part of this path.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--impl reference]

Prints one JSON line (rank 0). `value` is whole-job tokens/s with inputs
resident in HBM (CUDA-graph replay, CUDA events around exactly K steps, median
of `--repeats` such regions); `e2e` is the same metric through host buffers
(pinned host -> device copy of the step's hidden states, the stack, device ->
host read of the result) inside the timed region. Further keys of the same
line cover the rest of the metric: `int8_peak` (the measured dense int8
tensor-core rate), `prefill` (one block at 4096 tokens on the tcgen05 kernels,
as a fraction of that rate), `decode_sweep` (other batch sizes), `skew` (the
routing-skew shape); with N > 1 GPUs `ep_parity` (the expert-parallel block
against one GPU, bit for bit) and `config4` (prefill-size expert-parallel
blocks of the 3b-a800m shape).

`--impl reference` times the CPU path (the oracle's restatement of Tachyon's
AVX2 code: no Rust toolchain exists here to build the original) on the host
cores, same config and metric.
"""
from __future__ import annotations

import argparse
import datetime
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
UNIT = "tokens/s"
EPS = 1e-6
DTYPE = "int8 x int8 -> i32, f32 scales"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=250, help="steps per timed region")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=5, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--batch", type=int, default=32, help="decode tokens per step per GPU")
    ap.add_argument("--layers", type=int, default=workloads.GRANITE_1B.layers)
    ap.add_argument("--model", default="1b-a400m", choices=["1b-a400m", "3b-a800m-q8"],
                    help="expert shape: the headline granite-1b-a400m, or the 3b-a800m shape with int8 weights")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--headline-only", action="store_true",
                    help="skip the int8 peak, prefill, batch-size, skew and config-4 sections")
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
            d = json.load(f)
        return float(d["hbm_gbs"]), float(d.get("bf16_tflops", 1590.0)), "measured"
    return 6650.0, 1590.0, "fallback"


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


# ---------------------------------------------------------------- the CPU arm

def cpu_stack_step(oracle, mats, x0, topk, threads):
    """One pass of the CPU path over the stack: xb = rmsnorm(x); x += moe(xb)."""
    x = x0.copy()
    ones = np.ones(x.shape[1], np.float32)
    for router, gate_up, down in mats:
        xb = oracle.rmsnorm_rows(x, ones, EPS)
        x += oracle.moe(router, gate_up, down, xb, topk, threads=threads).proj
    return x


def run_cpu(shape, weights_host, x0, steps, warmup, budget_s=25.0):
    """Warm-up pass, then the best of the timed steps (the protocol of the reference's
    bench-batch, src/main.rs:1135-1151), within a time budget."""
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
    best, mean = float(np.min(times)), float(np.mean(times))
    return {"tokens_per_s": x0.shape[0] / best, "ms_per_step": best * 1e3, "steps": len(times),
            "threads": threads, "mean_ms": mean * 1e3}


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


def reference_arm(args, shape, world):
    """The CPU path on the host cores, on the same global batch as the GPU arm at this N."""
    threads = max(1, (os.cpu_count() or 8) - 2)
    weights_host, _ = build_weights(shape, args.layers, args.seed, threads)
    tokens = args.batch * world
    x0 = np.concatenate([workloads.hidden_states(shape, args.batch, seed=args.seed + r) for r in range(world)])
    warm = max(1, min(args.warmup, 5))
    r = run_cpu(shape, weights_host, x0, min(args.steps, 200), warm, budget_s=120.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": r["tokens_per_s"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": r["steps"], "warmup": warm, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": DTYPE, "data": "synthetic",
        "config": config_dict(args, shape, world),
        "cpu_baseline": {"value": r["tokens_per_s"], "unit": UNIT, "cores": r["threads"], "kind": "port",
                         "sample": f"best of {r['steps']} full steps of the same {args.layers}-layer stack at "
                                   f"{tokens} tokens per step (mean {r['mean_ms']:.1f} ms); C++ restatement of "
                                   f"Tachyon's AVX2 path, not the Rust binary"},
        "e2e": {"value": r["tokens_per_s"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def emit(line):
    sys.stdout.write(json.dumps(line) + "\n")
    sys.stdout.flush()


# ---------------------------------------------------------------- timing helpers

def timed_regions(ctx, launch, steps, repeats, barrier=None):
    """`repeats` regions of exactly `steps` calls of launch(), each between CUDA events on the
    context's stream with a synchronize on both sides. Returns milliseconds per region."""
    out = []
    for _ in range(repeats):
        ctx.sync()
        if barrier:
            barrier()
        ctx.timer_start()
        for _ in range(steps):
            launch()
        out.append(ctx.timer_stop_ms())
    return out


def steps_for(ms_per_step, target_ms, lo=3, hi=2000):
    return int(min(hi, max(lo, round(target_ms / max(ms_per_step, 1e-3)))))


class Stack:
    """The MoE blocks of a model on one context, with a residual stream of `batch` tokens."""

    def __init__(self, ctx, shape, layers, batch, seed=0):
        self.ctx, self.shape, self.layers, self.batch = ctx, shape, layers, batch
        self.ones = ctx.to_device(np.ones(shape.hidden, np.float32))
        self.x_host = ctx.pinned((batch, shape.hidden))
        self.x_host[:] = workloads.hidden_states(shape, batch, seed=seed)
        self.y_host = ctx.pinned((batch, shape.hidden))
        self.x_in = ctx.to_device(self.x_host)
        self.x = ctx.empty((batch, shape.hidden))

    def enqueue(self):
        self.ctx.copy(self.x, self.x_in)
        for layer in self.layers:
            layer.block(self.ones, EPS, self.x, t=self.batch)  # x += moe(rmsnorm(x)): src/model.rs:662-681

    def capture(self):
        self.enqueue()
        self.ctx.sync()
        self.ctx.capture_begin()
        self.enqueue()
        return self.ctx.capture_end()

    def routing_spread(self):
        """Distinct experts picked per layer (what the algorithmic bytes depend on)."""
        distinct = []
        self.ctx.copy(self.x, self.x_in)
        for layer in self.layers:
            layer.block(self.ones, EPS, self.x, t=self.batch)
            _, _, counts, _ = layer.last_routing(self.batch)
            distinct.append(int(np.count_nonzero(counts)))
        return distinct

    def free(self):
        for d in (self.ones, self.x_in, self.x):
            d.free()


def decode_point(ctx, shape, layers, batch, target_ms, repeats, peak):
    """ms per step and whole-step HBM fraction of the stack at one batch size."""
    st = Stack(ctx, shape, layers, batch)
    distinct = st.routing_spread()
    graph = st.capture()
    for _ in range(5):
        graph.launch()
    ctx.sync()
    probe = timed_regions(ctx, graph.launch, 10, 1)[0] / 10
    k = steps_for(probe, target_ms)
    ms = float(np.median(timed_regions(ctx, graph.launch, k, repeats))) / k
    nbytes = sum(workloads.decode_algorithmic_bytes(shape, batch, u) for u in distinct)
    graph.free()
    st.free()
    return {"batch": batch, "ms_per_step": ms, "tokens_per_s": batch / (ms * 1e-3), "steps_per_region": k,
            "distinct_experts_per_layer": float(np.mean(distinct)), "algorithmic_bytes_per_step": nbytes,
            "whole_step_gbs": nbytes / (ms * 1e-3) / 1e9, "whole_step_frac": nbytes / (ms * 1e-3) / 1e9 / peak}


def block_point(ctx, cuda, shape, lw, tokens, bias, int8_pops, target_ms, repeats):
    """One MoE block at `tokens` tokens (prefill-size: the tcgen05 kernels when the batch averages
    32 tokens per expert): time per block, per-kernel shares, and the expert kernels' rate."""
    layer = cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.topk, tokens)
    if bias is not None:
        layer.set_router_bias(bias)
    x = ctx.to_device(workloads.hidden_states(shape, tokens, seed=1))
    y = ctx.to_device(np.zeros((tokens, shape.hidden), np.float32))
    layer.forward(x, y)
    ctx.sync()
    _, _, counts, _ = layer.last_routing(tokens)
    ctx.capture_begin()
    layer.forward(x, y)
    graph = ctx.capture_end()
    for _ in range(3):
        graph.launch()
    ctx.sync()
    probe = timed_regions(ctx, graph.launch, 5, 1)[0] / 5
    k = steps_for(probe, target_ms, lo=5)
    ms = float(np.median(timed_regions(ctx, graph.launch, k, repeats))) / k
    # Per-kernel times from CUDA events around each launch (eager, so launches do not overlap).
    ctx.profile_enable(True)
    for _ in range(5):
        layer.forward(x, y)
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    stage_us = {name: v[0] / 5 * 1e3 for name, v in prof.items() if v[1]}
    total = sum(stage_us.values())
    ops = 2.0 * tokens * shape.topk * 3 * shape.inter * shape.hidden  # int8 multiply-adds x 2
    expert_us = stage_us.get("gate_up", 0.0) + stage_us.get("down", 0.0)
    out = {"tokens": tokens, "ms_per_block": ms, "tokens_per_s": tokens / (ms * 1e-3), "steps_per_region": k,
           "tokens_per_expert_max": int(counts.max()), "tokens_per_expert_min_nonzero": int(counts[counts > 0].min()),
           "kernel_us_eager": stage_us, "kernel_share": {n: v / total for n, v in stage_us.items()},
           "int8_ops_per_block": ops}
    if expert_us > 0:
        out["expert_kernels_pops"] = ops / (expert_us * 1e-6) / 1e15
        out["whole_block_pops"] = ops / (ms * 1e-3) / 1e15
        if int8_pops:
            out["expert_kernels_frac_of_int8_peak"] = out["expert_kernels_pops"] / int8_pops
            out["whole_block_frac_of_int8_peak"] = out["whole_block_pops"] / int8_pops
    graph.free()
    for d in (x, y):
        d.free()
    layer.free()
    return out


def q4_layer(shape, seed, threads):
    """One layer's weights through the numpy mirror of the 4-bit quantizer, row ranges on a thread pool."""
    from concurrent.futures import ThreadPoolExecutor

    from tachyon_b200.q4 import quantize_q4_matrix
    from tachyon_b200.weights import KIND_Q4, Matrix, q4_words

    h, e, i = shape.hidden, shape.experts, shape.inter

    def quant(stream, rows, cols):
        words = q4_words(cols)
        scales = np.empty(rows * words, np.uint32)
        qs = np.empty(rows * cols // 2, np.uint8)
        step = max(256, -(-rows // (4 * threads)))

        def part(r0):
            r1 = min(rows, r0 + step)
            data = synth.normal(seed, stream, (r1 - r0) * cols, 0, scale=0.02, start=r0 * cols)
            s, q = quantize_q4_matrix(data, r1 - r0, cols)
            scales[r0 * words:r1 * words] = s
            qs[r0 * cols // 2:r1 * cols // 2] = q

        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(part, range(0, rows, step)))
        return Matrix(KIND_Q4, rows, cols, scales, qs)

    router = workloads._normal_matrix(seed, synth.STREAM_ROUTER, 0, e, h, "bf16")
    return workloads.LayerWeights(router, quant(synth.STREAM_GATE_UP, e * 2 * i, h), quant(synth.STREAM_DOWN, e * h, i))


# ---------------------------------------------------------------- the GPU arm

def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    shape = workloads.GRANITE_1B if args.model == "1b-a400m" else workloads.GRANITE_3B_Q8
    host_threads = max(1, (os.cpu_count() or 8) // max(1, world) - 1)

    if args.impl == "reference":
        if rank == 0:
            reference_arm(args, shape, world)
        return

    from tachyon_b200 import build as cuda_build
    from tachyon_b200 import cuda

    if rank == 0:
        cuda_build.build()
    dist = None
    if world > 1:
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # (its banner would land on stdout beside the JSON line)
        import torch.distributed as dist  # plumbing only: barrier and max over ranks

        dist.init_process_group("gloo", timeout=datetime.timedelta(minutes=5))
        dist.barrier()
    ctx = cuda.Context(local_rank)
    if args.no_overlap:
        ctx.set_launch_overlap(False)
    if args.four_kernels:
        ctx.set_decode_block(False)
    peak_hbm, peak_bf16, peak_kind = measured_peaks()
    sweep_batches = [1, 8, 64, 128] if world == 1 and not args.headline_only else []
    max_batch = max([args.batch] + sweep_batches)

    if world == 1:
        weights_host, gen_s = build_weights(shape, args.layers, args.seed, host_threads)
        layers = [cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.topk, max_batch) for lw in weights_host]
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

    def barrier():
        if dist:
            dist.barrier()

    def max_over_ranks(v):
        if not dist:
            return v
        import torch

        tmax = torch.tensor([v], dtype=torch.float64)
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        return float(tmax.item())

    stack = Stack(ctx, shape, layers, args.batch, seed=args.seed + rank)
    barrier()  # ranks enter their first block together: the peer exchange's waits are bounded
    stack.enqueue()
    ctx.sync()
    distinct = stack.routing_spread() if world == 1 else []

    # ---- the timed stack, device-resident inputs: one CUDA graph per step. (The variable-size
    # expert-parallel exchange reads its sizes on the host, so that one is enqueued directly.)
    class Eager:
        def launch(self):
            stack.enqueue()

        def free(self):
            pass

    graph = stack.capture() if (world == 1 or args.ep_exchange != "alltoallv") else Eager()
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        graph.launch()
    ctx.sync()
    barrier()
    launches0 = ctx.launch_count()
    with ClockSampler(local_rank) as clocks:
        regions = timed_regions(ctx, graph.launch, args.steps, args.repeats, barrier=barrier)
        launches = (ctx.launch_count() - launches0) // args.repeats
        # nvidia-smi samples every 100 ms: keep the same load running a little longer if the
        # regions were short (untimed; the same count on every rank).
        extra = steps_for(float(np.median(regions)) / args.steps, 600.0) if sum(regions) < 600.0 else 0
        extra = int(max_over_ranks(float(extra)))
        for _ in range(extra):
            graph.launch()
        ctx.sync()
    regions = [max_over_ranks(r) for r in regions]
    ms_per_step = float(np.median(regions)) / args.steps
    value = args.batch * world / (ms_per_step * 1e-3)

    # ---- end to end through host buffers
    def e2e_step():
        ctx.upload(stack.x_in.ptr, stack.x_host)
        graph.launch()
        ctx.download(stack.y_host, stack.x.ptr)

    for _ in range(3):
        e2e_step()
    barrier()
    e2e_steps = min(args.steps, 200)
    e2e_regions = [max_over_ranks(r) for r in timed_regions(ctx, e2e_step, e2e_steps, max(3, args.repeats // 2 + 1),
                                                             barrier=barrier)]
    e2e_ms = float(np.median(e2e_regions)) / e2e_steps
    e2e_value = args.batch * world / (e2e_ms * 1e-3)
    assert np.all(np.isfinite(stack.y_host))
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": int(stack.x_host.nbytes),
           "d2h_bytes_per_step": int(stack.y_host.nbytes), "ms_per_step": e2e_ms, "steps_per_region": e2e_steps}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic", "config": config_dict(args, shape, world), "e2e": e2e,
        "gpu_launches": int(launches), "repeats": args.repeats, "region_ms": regions,
        "setup_s": {"weights_host": gen_s},
    }

    if world > 1:
        line.update(multi_gpu_sections(args, ctx, cuda, dist, shape, layers, stack, rank, world, host_threads,
                                       peak_hbm, peak_kind, ms_per_step))
        if rank == 0:
            line["clocks"] = clocks.summary()
            emit(line)
        dist.barrier()
        return

    # ---- roofline of the dominant kernel. At decode sizes the whole block is one kernel
    # (moe_decode_kernel), so the step is `layers` launches of it plus one small copy: its average
    # launch duration is the timed region divided by the launches in it. Per-launch CUDA events
    # (eager, no overlap between launches) and the kernel's own phase stamps go beside it.
    ctx.profile_enable(True)
    for _ in range(3):
        stack.enqueue()
    prof = ctx.profile_read()
    ctx.profile_enable(False)
    stage_us = {k: v[0] / max(1, v[1]) * 1e3 for k, v in prof.items() if v[1]}
    total_prof = sum(v[0] for v in prof.values())
    step_bytes = [workloads.decode_algorithmic_bytes(shape, args.batch, u) for u in distinct]
    mean_u = float(np.mean(distinct))
    one_kernel = "decode_block" in stage_us
    if one_kernel:
        bytes_per_launch = float(np.mean(step_bytes))
        launch_us = ms_per_step * 1e3 / args.layers
        kernel = f"moe_decode_kernel<{shape.fmt}> (router + gate_up + down + combine of one block)"
        ctx.profile_phases(True)
        g2 = stack.capture()
        for _ in range(3):
            g2.launch()
        phases = ctx.read_phases()
        ctx.profile_phases(False)
        g2.free()
    else:
        eb_gu = 2 * shape.inter * shape.hidden * 34 // 32  # one expert's gate_up rows as stored
        nbp = -(-(shape.hidden // 32) // 8) * 8
        bytes_per_launch = (mean_u * eb_gu + args.batch * (shape.hidden + 4 * nbp)
                            + args.batch * shape.topk * shape.inter * 4)
        launch_us = stage_us["gate_up"]
        kernel = f"expert_fast_kernel<{shape.fmt}, gate_up>"
        phases = None
    achieved = bytes_per_launch / (launch_us * 1e-6) / 1e9
    whole = sum(step_bytes) / (ms_per_step * 1e-3) / 1e9
    line["roofline"] = {
        "bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peak_hbm, "unit": "GB/s",
        "frac": achieved / peak_hbm, "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)",
        "frac_of_8TBs_nominal": achieved / 8000.0, "algorithmic_bytes_per_launch": bytes_per_launch,
        "avg_launch_us": launch_us, "avg_launch_source": "timed region / launches in it" if one_kernel
        else "CUDA events around each eager launch",
        "eager_event_us": stage_us, "distinct_experts_per_layer": mean_u, "traffic": None,
        "kernel_share_of_step": {k: v[0] / total_prof for k, v in prof.items() if v[1]},
        "phase_us_cta0": phases,
        "whole_step": {"algorithmic_bytes": sum(step_bytes), "achieved": whole, "frac": whole / peak_hbm},
    }
    line["clocks"] = clocks.summary()
    graph.free()

    if not args.headline_only:
        # (Each section on its own: whatever goes wrong in one must not cost the line its headline.)
        t0 = time.time()
        peak = {"pops": None}

        def section(name, fn):
            try:
                line[name] = fn()
            except Exception as e:  # noqa: BLE001
                line[name] = {"error": f"{type(e).__name__}: {e}"}

        def int8_peak():
            peak.update(ctx.int8_peak(50.0))
            peak["vs_2x_measured_bf16"] = peak["pops"] / (2.0 * peak_bf16 / 1e3)
            return dict(peak)

        def prefill():
            # One block at 4096 tokens (4 sequences x 1024): the 1b shape in int8, the 3b shape in 4 bits.
            pre = {"1b-a400m-q8": block_point(ctx, cuda, shape, weights_host[0], 4096, None, peak["pops"], 60.0, 3)}
            s3 = workloads.GRANITE_3B
            pre["3b-a800m-q4"] = block_point(ctx, cuda, s3, q4_layer(s3, args.seed, host_threads), 4096, None,
                                             peak["pops"], 60.0, 3)
            return pre

        def skew():
            # The routing-skew shape: hidden 2048, 64 experts, intermediate 1024, Zipf(1.2) router bias.
            sk = workloads.SKEW
            lw = workloads.layer_weights(sk, seed=args.seed, threads=host_threads)
            bias = synth.zipf_router_bias(args.seed, sk.experts)
            return {"shape": "hidden 2048, 64 experts, top-8, intermediate 1024, int8, Zipf(1.2) router bias",
                    "points": [block_point(ctx, cuda, sk, lw, t, bias, peak["pops"], 40.0, 3) for t in (256, 4096)]}

        section("int8_peak", int8_peak)
        section("decode_sweep", lambda: [decode_point(ctx, shape, layers, b, 100.0, 3, peak_hbm) for b in sweep_batches])
        section("prefill", prefill)
        section("skew", skew)
        line["setup_s"]["sections"] = time.time() - t0

    if not args.no_cpu_baseline:
        r = run_cpu(shape, weights_host, np.array(stack.x_host), steps=30, warmup=1, budget_s=20.0)
        line["cpu_baseline"] = {
            "value": r["tokens_per_s"], "unit": UNIT, "cores": r["threads"], "kind": "port",
            "sample": f"best of {r['steps']} full steps of the same {args.layers}-layer stack at batch {args.batch} "
                      f"(best {r['ms_per_step']:.1f} ms, mean {r['mean_ms']:.1f} ms per step); C++ restatement of "
                      f"Tachyon's AVX2 path",
        }
    emit(line)


def multi_gpu_sections(args, ctx, cuda, dist, shape, layers, stack, rank, world, host_threads, peak_hbm, peak_kind,
                       ms_per_step):
    """Whole-job roofline, the expert-parallel block against one GPU, and prefill-size blocks."""
    import torch

    from tachyon_b200 import ep

    out = {}
    step_bytes = args.layers * workloads.decode_algorithmic_bytes(shape, args.batch * world, shape.experts)
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    out["roofline"] = {"bound": "hbm", "kernel": "whole step, all ranks", "achieved": achieved,
                       "peak": peak_hbm * world, "unit": "GB/s", "frac": achieved / (peak_hbm * world),
                       "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs x {world} GPUs)", "traffic": None}

    # ---- correctness where the driver can see it: layer 0 through the expert-parallel block on
    # every rank's own tokens, against the same tokens through a single-GPU layer on rank 0.
    x_local = np.array(stack.x_host)
    y0_local = workloads.hidden_states(shape, args.batch, seed=1000 + rank)
    xd, yd = ctx.to_device(x_local), ctx.to_device(y0_local)
    dist.barrier()
    layers[0].forward(xd, yd)
    ctx.sync()
    got = torch.from_numpy(yd.get())
    gathered = [torch.empty_like(got) for _ in range(world)]
    dist.all_gather(gathered, got)
    if rank == 0:
        lw = workloads.layer_weights(shape, seed=args.seed, layer=0, threads=host_threads)
        full = cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, shape.topk, args.batch * world)
        x_all = np.concatenate([workloads.hidden_states(shape, args.batch, seed=args.seed + r) for r in range(world)])
        y_all = np.concatenate([workloads.hidden_states(shape, args.batch, seed=1000 + r) for r in range(world)])
        xa, ya = ctx.to_device(x_all), ctx.to_device(y_all)
        full.forward(xa, ya)
        ctx.sync()
        want = ya.get()
        have = np.concatenate([g.numpy() for g in gathered])
        out["ep_parity"] = "bit-equal" if np.array_equal(have, want) else \
            {"max_abs": float(np.abs(have - want).max())}
        for d in (xa, ya):
            d.free()
        full.free()
    for d in (xd, yd):
        d.free()
    dist.barrier()

    # ---- where a block's time goes on rank 0 (wall-clock stamps of CTA 0 inside the one-kernel block)
    try:
        ctx.profile_phases(True)
        g2 = stack.capture()
        dist.barrier()
        for _ in range(3):
            g2.launch()
        out["phase_us_cta0"] = ctx.read_phases()
        dist.barrier()
        ctx.profile_phases(False)
        g2.free()
    except Exception as e:  # (a path without phase stamps: the four-kernel exchanges)
        out["phase_us_cta0"] = str(e)
    dist.barrier()

    if args.headline_only:
        return out
    # (Measured last and on its own: whatever goes wrong in it must not cost the line its headline.)
    try:
        out["config4"] = config4_section(args, ctx, cuda, dist, ep, torch, rank, world, host_threads)
    except Exception as e:  # noqa: BLE001
        out["config4"] = {"error": f"{type(e).__name__}: {e}"}
    return out


def config4_section(args, ctx, cuda, dist, ep, torch, rank, world, host_threads):
    """Prefill-size expert-parallel blocks (the 3b-a800m shape in int8, 8192 tokens per step over all ranks)."""
    # ---- prefill-size expert-parallel blocks: the 3b-a800m shape with int8 weights, 8192 tokens per
    # step over all ranks, 2 layers. Twice: rows and expert outputs stored into the other ranks'
    # windows over NVLink by the kernels that produce them (a second context whose windows are sized
    # for these blocks), and the variable-size all-to-all over NCCL.
    s4 = workloads.GRANITE_3B_Q8
    tokens = 8192 // world
    first, count = ep.shard_range(s4.experts, rank, world)
    lws4 = [workloads.layer_weights_local(s4, first, count, seed=args.seed, layer=l, threads=host_threads)
            for l in range(2)]
    k = 10

    def time_config4(c):
        l4 = [ep.EpMoeLayer(c, lw.router, lw.gate_up, lw.down, s4.experts, s4.topk, tokens) for lw in lws4]
        st4 = Stack(c, s4, l4, tokens, seed=args.seed + rank)
        dist.barrier()
        for _ in range(3):
            st4.enqueue()
        c.sync()
        regs = []
        for r in timed_regions(c, st4.enqueue, k, 3, barrier=dist.barrier):
            tmax = torch.tensor([r], dtype=torch.float64)
            dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
            regs.append(float(tmax.item()))
        st4.free()
        for layer in l4:
            layer.free()
        dist.barrier()
        return float(np.median(regs)) / k

    def fresh_context(peer):
        c = cuda.Context(ctx.device)
        box = [ep.unique_id(c) if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ep.init(c, box[0], rank, world, uniform_batch=peer)
        if peer:
            ep.enable_peer_exchange(c, s4.hidden, s4.topk, tokens)
        return c

    c_nccl = fresh_context(False)
    ms4_nccl = time_config4(c_nccl)
    c_nccl.close()
    c_peer = fresh_context(True)
    ms4 = time_config4(c_peer)
    c_peer.close()
    c4 = {"workload": "granite-3b-a800m shape, int8 weights, 40 experts sharded, 8192 tokens per step over all ranks, "
                      "2 MoE blocks; rows and expert outputs stored into the other ranks' windows over NVLink "
                      "(tcgen05 expert kernels on the local experts)",
          "tokens_per_rank": tokens, "ms_per_step": ms4, "ms_per_block": ms4 / 2,
          "tokens_per_s": 8192 / (ms4 * 1e-3), "steps_per_region": k,
          "nccl_all_to_all_v": {"ms_per_step": ms4_nccl, "tokens_per_s": 8192 / (ms4_nccl * 1e-3)}}
    if rank == 0:
        # The same two blocks on one GPU, for the ratio.
        lws = [workloads.layer_weights(s4, seed=args.seed, layer=l, threads=host_threads) for l in range(2)]
        full = [cuda.MoeLayer(ctx, lw.router, lw.gate_up, lw.down, s4.topk, 8192) for lw in lws]
        st1 = Stack(ctx, s4, full, 8192, seed=args.seed)
        for _ in range(3):
            st1.enqueue()
        ctx.sync()
        ms1 = float(np.median(timed_regions(ctx, st1.enqueue, k, 3))) / k
        c4["one_gpu_ms_per_step"] = ms1
        c4["speedup_vs_one_gpu"] = ms1 / ms4
        st1.free()
        for layer in full:
            layer.free()
    dist.barrier()
    return c4


if __name__ == "__main__":
    main()
