#!/usr/bin/env python
"""Benchmark of the AWQ W4A16 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload ("step"): one pass over the four AWQ linears of a Qwen2.5-72B decoder layer
(qkv 8192x10240, o_proj 8192x8192, gate_up 8192x59136, down 29568x8192; group 128) for a decode
batch of M = 16 tokens -- 438.8 MB of int4 weights per step, more than the 126 MB L2, so every
step streams its weights from HBM.  Inputs are seeded synthetic tensors with the value
distributions of the benchmark configuration (nibbles uniform 0..15, scales uniform
[0.002, 0.02], activations N(0,1)).

metric  awq_w4a16_gemm_hbm_TBps = int4 weight bytes streamed per second, whole job.
value   device-resident: the step is captured once in a CUDA graph and replayed; timed with
        CUDA events on the launching stream between barriers, max over ranks.
e2e     the same step through the layer API (AWQLinearMethod.apply) with the activations in
        pinned host memory: host->device copy, four kernels, device->host copy of the outputs,
        every step; weights stay resident in HBM as they do while serving.  Four steps are in
        flight on four streams (copies of one step overlap kernels of another).
N > 1   replicas (the TP=1 scaling mode of the harness): every rank runs the same step on its
        own GPU, value is the sum; reported as weak scaling.  The tensor-parallel variant
        (column/row shards + NCCL all-reduce of the row-parallel outputs) is timed as well and
        reported under "tp".
--impl reference   the reference arithmetic (dequantise-then-matmul in fp32, PyTorch on the
        host cores) on the same metric; each step is a bounded sample (the o_proj shape).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "server-benchmark_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

METRIC = "awq_w4a16_gemm_hbm_TBps"
UNIT = "TB/s"
M_TOKENS = 16
GROUP = 128
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the M = 16 kernel, as a ratio to the
# launch's algorithmic bytes, from an ncu capture of a smaller case (K = 8192, N = 29568: 130.2 MB
# of traffic for 126.6 MB); the traffic of the full-size launches is scaled by their bytes
NCU_TRAFFIC_RATIO = 1.028
E2E_DEPTH = 4  # steps in flight in the end-to-end leg (2: 0.255, 3: 0.206, 4: 0.201, 6: 0.198 ms per step)


def shapes():
    from awq_b200 import synth
    return list(synth.QWEN25_72B_SHAPES.items())


def weight_bytes_per_step() -> int:
    return sum(k * n // 2 for _, (k, n) in shapes())


def all_bytes_per_step(m: int) -> int:
    tot = 0
    for _, (k, n) in shapes():
        tot += k * n // 2 + (k // GROUP) * n * 2 + (k // GROUP) * (n // 8) * 4 + m * k * 2 + m * n * 2
    return tot


def measured_tensor_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["bf16_tflops"]), "measured (burst)"
    except Exception:
        return 1590.0, "fallback"


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons through nvidia-smi while the timed region runs
    (read-only queries)."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                pass

    def summary(self, t0: float, t1: float):
        rows = [s for t, s in self.samples if t0 <= t <= t1 + 0.06] or [s for _, s in self.samples]
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            f = [x.strip() for x in r.split(",")]
            try:
                mhz.append(float(f[0]))
                mx = max(mx, float(f[1]))
            except Exception:
                continue
            for name, val in zip(names, f[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        med = mhz[len(mhz) // 2] if mhz else None
        return {"sm_mhz": med, "sm_max_mhz": mx or None, "reasons": sorted(reasons),
                "samples": len(mhz)}


# ------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle's dequantise-then-matmul on the host cores
# ------------------------------------------------------------------------------------------


def cpu_reference_sample(reps: int):
    """Times the fp32 dequantise-then-matmul of the o_proj shape (K = N = 8192, M = 16) on the
    host.  Returns (seconds per call (best), cores, description)."""
    import torch
    from awq_b200 import synth
    from oracle import awq_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    k, n = 8192, 8192
    qw, s, qz = synth.awq_linear_tensors(k, n, GROUP, seed=0)
    x = synth.activations(M_TOKENS, k, seed=0)
    O.awq_gemm_fp32_torch(x, qw, s, qz, GROUP)  # warm-up
    times = []
    for _ in range(reps):
        t = time.perf_counter()
        O.awq_gemm_fp32_torch(x, qw, s, qz, GROUP)
        times.append(time.perf_counter() - t)
    return min(times), sum(times) / len(times), cores, \
        f"o_proj K=8192 N=8192 M={M_TOKENS} group 128, torch fp32 dequantise+matmul, {reps} calls"


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    reps = max(1, min(args.steps, 20))
    for _ in range(min(args.warmup, 2)):
        pass
    best, mean, cores, sample = cpu_reference_sample(reps)
    wbytes = 8192 * 8192 // 2
    val = wbytes / mean / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": reps, "warmup": 1, "ms_per_step": mean * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "awq_w4a16_linear_M16_qwen2.5-72b_layer (sampled: o_proj shape)",
                   "group_size": GROUP, "tokens": M_TOKENS},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# CUDA arm
# ------------------------------------------------------------------------------------------


def run_cuda(args):
    import torch
    import torch.distributed as dist

    import build as awq_build
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if rank == 0:
        awq_build.build()
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist.barrier()
    if rank != 0:
        awq_build.build()
    import awq_b200
    from awq_b200 import synth, tp

    dev = torch.device("cuda", local)
    m = M_TOKENS
    method = awq_b200.AWQLinearMethod(awq_b200.AWQConfig(group_size=GROUP))
    layers, xs = [], []
    for i, (name, (k, n)) in enumerate(shapes()):
        layer = awq_b200.AWQLinear()
        method.create_weights(layer, k, [n], k, n, torch.float16, device=dev)
        qw, s, qz = synth.awq_linear_tensors(k, n, GROUP, seed=i)
        layer.qweight.data.copy_(qw)
        layer.scales.data.copy_(s)
        layer.qzeros.data.copy_(qz)
        method.process_weights_after_loading(layer)
        layers.append(layer)
        xs.append(synth.activations(m, k, seed=i))
    x_dev = [x.to(dev) for x in xs]
    x_pin = [x.pin_memory() for x in xs]
    y_pin = [torch.empty((m, n), dtype=torch.float16).pin_memory() for _, (k, n) in shapes()]

    def step_device():
        for layer, x in zip(layers, x_dev):
            awq_b200.awq_gemm(x, layer.qweight, layer.scales, layer.qzeros, 8)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        step_device()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step_device()
        for _ in range(max(args.warmup, 3)):
            graph.replay()
        barrier()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
            time.sleep(0.12)
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        barrier()
        t_wall0 = time.time()
        e0.record(stream)
        for _ in range(args.steps):
            graph.replay()
        e1.record(stream)
        barrier()
        t_wall1 = time.time()
        ms = e0.elapsed_time(e1)

        # ---- e2e through the layer API with host buffers ----
        # E2E_DEPTH steps are in flight, each on its own stream with its own pinned result
        # buffers (a serving loop with that many requests in flight): the copies of one step
        # overlap the kernels of another.  Every step still copies its inputs from pinned host
        # memory and its four outputs back, and the host waits for a step's outputs before
        # the buffers are used again.
        side = [torch.cuda.Stream(device=dev) for _ in range(E2E_DEPTH)]
        y_pins = [y_pin] + [[torch.empty_like(y).pin_memory() for y in y_pin]
                            for _ in range(E2E_DEPTH - 1)]
        landed = [None] * E2E_DEPTH

        def step_e2e(i):
            j = i % E2E_DEPTH
            if landed[j] is not None:
                landed[j].synchronize()  # outputs of the step that last used these buffers
            with torch.cuda.stream(side[j]):
                # inputs up, the four linears back to back (consecutive kernels of the library
                # overlap their start-up with the end of the one before), outputs down
                xds = [xp.to(dev, non_blocking=True) for xp in x_pin]
                ys = [method.apply(layer, xd) for layer, xd in zip(layers, xds)]
                for yp, y in zip(y_pins[j], ys):
                    yp.copy_(y, non_blocking=True)
                landed[j] = torch.cuda.Event()
                landed[j].record(side[j])

        def drain():
            for j in range(E2E_DEPTH):
                if landed[j] is not None:
                    landed[j].synchronize()
                stream.wait_stream(side[j])

        e2e_steps = max(1, min(args.steps, 300))
        for i in range(3 * E2E_DEPTH):
            step_e2e(i)
        drain()
        barrier()
        f0 = torch.cuda.Event(enable_timing=True)
        f1 = torch.cuda.Event(enable_timing=True)
        f0.record(stream)
        for j in range(E2E_DEPTH):
            side[j].wait_stream(stream)
        for i in range(e2e_steps):
            step_e2e(i)
        drain()
        f1.record(stream)
        barrier()
        ms_e2e = f0.elapsed_time(f1)
        if rank == 0:
            sampler.stop()

        # ---- benchmark configurations 2 and 3 (1 GPU only): shape sweep and MoE layer ----
        sweep = moe = None
        if world == 1 and not args.no_sweep:
            del graph
            sweep = run_sweep(dev, stream)
            moe = run_moe(dev, stream)

        # ---- tensor-parallel variant (N > 1): column/row shards + all-reduce ----
        tp_result = None
        if world > 1:
            tp_result = run_tp(args, world, rank, dev, stream, barrier)

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    if rank == 0:
        wbytes = weight_bytes_per_step()
        sec = ms * 1e-3 / args.steps
        value = world * wbytes / sec / 1e12
        sec_e2e = ms_e2e * 1e-3 / e2e_steps
        peak, peak_kind = measured_peak()
        achieved = wbytes / sec / 1e9  # GB/s of int4 weight bytes, one GPU
        achieved_all = all_bytes_per_step(m) / sec / 1e9
        launches_per_step = len(layers)
        cpu_best, cpu_mean, cores, sample = (None, None, None, None)
        cpu = None
        if world == 1:
            cpu_best, cpu_mean, cores, sample = cpu_reference_sample(3)
            cpu = {"value": (8192 * 8192 // 2) / cpu_best / 1e12, "unit": UNIT, "cores": cores,
                   "kind": "port", "sample": sample}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": "awq_w4a16_linear_M16_qwen2.5-72b_layer (qkv,o_proj,gate_up,down)",
                       "group_size": GROUP, "tokens": m, "parallelism": f"replicas x{world}",
                       "l2": "inputs larger than L2 (438.8 MB of weights per step)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "kernel": "gemm_ts_kernel (4 launches per step: qkv, o_proj, gate_up, "
                                   "down); achieved = weight bytes of the step / step time",
                         "achieved_all_bytes": achieved_all,
                         "traffic": NCU_TRAFFIC_RATIO * all_bytes_per_step(m) / launches_per_step},
            "cpu_baseline": cpu,
            "e2e": {"value": world * wbytes / sec_e2e / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": sum(m * k * 2 for _, (k, n) in shapes()),
                    "d2h_bytes_per_step": sum(m * n * 2 for _, (k, n) in shapes()),
                    "steps": e2e_steps, "ms_per_step": sec_e2e * 1e3, "steps_in_flight": E2E_DEPTH},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": sampler.summary(t_wall0, t_wall1),
        }
        if tp_result is not None:
            line["tp"] = tp_result
        if sweep is not None:
            tpeak = measured_tensor_peak()
            big = max((r for r in sweep if r["M"] >= 1024), key=lambda r: r["TFLOPs"])
            line["roofline_tensor"] = {"bound": "tensor", "achieved": big["TFLOPs"],
                                       "peak": tpeak[0], "unit": "TFLOP/s",
                                       "frac": big["TFLOPs"] / tpeak[0], "peak_kind": f"of {tpeak[1]}",
                                       "kernel": "gemm_tc_kernel<256,2>",
                                       "point": {"shape": big["shape"], "M": big["M"]}}
            line["sweep"] = sweep
            line["moe"] = moe
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def graph_time(fns, stream, reps=3):
    """Seconds per call of the callables in `fns` (each enqueues one op): captured once in a CUDA
    graph, replayed `reps` times, CUDA events on `stream`."""
    import torch
    with torch.cuda.stream(stream):
        for f in fns:
            f()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for f in fns:
                f()
        g.replay()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            g.replay()
        e1.record(stream)
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / (reps * len(fns))


def run_sweep(dev, stream):
    """Benchmark configuration 2: the four 72B layer shapes x M in {1 .. 4096}, 1 GPU.  Weights are
    rotated over enough copies that every launch reads more than the L2 holds."""
    import torch
    import awq_b200
    from awq_b200 import synth
    out = []
    for name, (k, n) in shapes():
        wbytes = k * n // 2
        copies = max(1, -(-200_000_000 // wbytes))
        base = [a.to(dev) for a in synth.awq_linear_tensors(k, n, GROUP, seed=1)]
        sets = [base] + [[a.clone() for a in base] for _ in range(copies - 1)]
        decode = [awq_b200.awq_repack(q[0]) for q in sets]
        for m in synth.SWEEP_M:
            x = synth.activations(m, k).to(dev)
            fns = [(lambda q=q: awq_b200.awq_gemm(x, q[0], q[1], q[2], 8)) for q in sets]
            t = graph_time(fns, stream, reps=3 if m >= 1024 else 10)
            row = {"shape": name, "K": k, "N": n, "M": m, "us": round(t * 1e6, 2),
                   "weight_GBps": round(wbytes / t / 1e9, 1),
                   "TFLOPs": round(2.0 * m * k * n / t / 1e12, 2)}
            if m <= 8:
                # the same layer with the optional decode-layout copy of qweight (made once, at
                # load time: AWQConfig(repack_decode=True)); "us" above is the checkpoint layout
                fns = [(lambda q=q, r=r: awq_b200.awq_gemm(x, r, q[1], q[2], 8,
                                                          kernel=awq_b200.KERNEL_STREAM_RP))
                       for q, r in zip(sets, decode)]
                tr = graph_time(fns, stream, reps=10)
                row["us_decode_layout"] = round(tr * 1e6, 2)
                row["weight_GBps_decode_layout"] = round(wbytes / tr / 1e9, 1)
            out.append(row)
        del sets, base, decode
    return out


def run_moe(dev, stream):
    """Benchmark configuration 3: Qwen3-30B-A3B fused-MoE layer (router -> permutation -> expert GEMMs ->
    sum), T in {1 .. 4096}, 1 GPU."""
    import torch
    import awq_b200
    from awq_b200 import synth
    cfg = synth.QWEN3_MOE
    e, h, i, k = cfg["experts"], cfg["hidden"], cfg["intermediate"], cfg["topk"]
    w1, w2 = synth.moe_layer_tensors(e, h, i, GROUP)
    w1 = tuple(a.to(dev) for a in w1)
    w2 = tuple(a.to(dev) for a in w2)
    d1, d2 = awq_b200.awq_repack(w1[0]), awq_b200.awq_repack(w2[0])
    from awq_b200 import _lib
    block_of = lambda t: _lib.load().awq_b200_moe_block_size(t, k, e, h, i, GROUP)  # noqa: E731
    out = []
    for t in synth.MOE_TOKENS:
        x = synth.activations(t, h).to(dev)
        logits = synth.gating_logits(t, e).to(dev)
        _, ids, _ = awq_b200.fused_topk(x, logits, k, True)
        hit = int(torch.unique(ids).numel())
        sec = graph_time([lambda: awq_b200.fused_moe(x, w1, w2, logits, k, True)], stream,
                         reps=5 if t >= 1024 else 20)
        byts = hit * (2359296 + 73728 + 18432) + t * h * 2 * 2
        row = {"T": t, "experts_hit": hit, "us": round(sec * 1e6, 1),
               "GBps": round(byts / sec / 1e9, 1),
               "TFLOPs": round(t * 75497472 / sec / 1e12, 2)}
        if block_of(t) in (8, 16):
            # the same layer with the optional decode-layout copies of the expert weights
            def layer():
                w, ids2, _ = awq_b200.fused_topk(x, logits, k, True)
                return awq_b200.fused_experts(x, w1, w2, w, ids2, w1_decode=d1, w2_decode=d2)
            sd = graph_time([layer], stream, reps=20)
            row["us_decode_layout"] = round(sd * 1e6, 1)
        out.append(row)
    return out


def run_tp(args, world, rank, dev, stream, barrier):
    """The same layer sharded over `world` GPUs: qkv/gate_up column-parallel, o_proj/down
    row-parallel with the fp16 [M, 8192] partial outputs all-reduced over NVLink (NCCL).  The
    down projection's K (231 groups) is padded to a multiple of the TP degree."""
    import torch
    import torch.distributed as dist
    from awq_b200 import synth, tp

    m = M_TOKENS
    shards, xs = [], []
    for i, (name, (k, n)) in enumerate(shapes()):
        qw, s, qz = synth.awq_linear_tensors(k, n, GROUP, seed=i)
        if name in ("qkv", "gate_up"):
            sh = tp.shard_columns(qw, s, qz, rank, world)
            x = synth.activations(m, k, seed=i)
            shards.append(("col", tuple(a.to(dev) for a in sh)))
        else:
            qw, s, qz = tp.pad_k_for_tp(qw, s, qz, world)
            sh = tp.shard_rows(qw, s, qz, rank, world)
            x = tp.shard_input(tp.pad_x_for_tp(synth.activations(m, k, seed=i), qw.shape[0]),
                               rank, world)
            shards.append(("row", tuple(a.to(dev) for a in sh)))
        xs.append(x.to(dev))

    def step():
        for (kind, sh), x in zip(shards, xs):
            if kind == "col":
                tp.column_parallel_forward(x, sh)
            else:
                tp.row_parallel_forward(x, sh)

    steps = max(1, min(args.steps, 500))
    for _ in range(5):
        step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    sec = float(t[0]) * 1e-3 / steps
    return {"parallelism": f"tp{world}", "scaling": "strong", "ms_per_step": sec * 1e3,
            "value": weight_bytes_per_step() / sec / 1e12, "unit": UNIT, "steps": steps,
            "collective": "nccl all_reduce fp16 [16, 8192] after o_proj and down"}


def run_case(args):
    """`--case kernel:M:K:N` launches one AWQ linear of that shape `--steps` times after
    `--warmup` launches and prints its CUDA-event time: the small, bounded command the ncu
    captures under profiles/ are taken with.  kernel: auto | stream | stream_exact | stream_rp
    (decode-layout copy of qweight) | tcgen05 | ts | wt | generic | dequantize | moe:T (Qwen3-30B-A3B layer with T tokens; K and N ignored)."""
    import torch

    import build as awq_build
    awq_build.build()
    import awq_b200
    from awq_b200 import synth

    f = args.case.split(":")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    if f[0] == "moe":
        t = int(f[1])
        cfg = synth.QWEN3_MOE
        w1, w2 = synth.moe_layer_tensors(cfg["experts"], cfg["hidden"], cfg["intermediate"])
        w1 = tuple(a.to(dev) for a in w1)
        w2 = tuple(a.to(dev) for a in w2)
        x = synth.activations(t, cfg["hidden"]).to(dev)
        logits = synth.gating_logits(t, cfg["experts"]).to(dev)
        fn = lambda: awq_b200.fused_moe(x, w1, w2, logits, cfg["topk"], True)  # noqa: E731
        work = f"moe T={t}"
    else:
        m, k, n = int(f[1]), int(f[2]), int(f[3])
        qw, s, qz = [a.to(dev) for a in synth.awq_linear_tensors(k, n, GROUP, seed=0)]
        x = synth.activations(m, k).to(dev)
        if f[0] == "dequantize":
            fn = lambda: awq_b200.awq_dequantize(qw, s, qz, 0, 0, 0)  # noqa: E731
        else:
            kern = {"auto": awq_b200.KERNEL_AUTO, "stream": awq_b200.KERNEL_STREAM,
                    "stream_exact": awq_b200.KERNEL_STREAM_EXACT,
                    "tcgen05": awq_b200.KERNEL_TCGEN05, "ts": awq_b200.KERNEL_TS, "wt": awq_b200.KERNEL_WT,
                    "stream_rp": awq_b200.KERNEL_STREAM_RP,
                    "generic": awq_b200.KERNEL_GENERIC}[f[0]]
            if f[0] == "stream_rp":
                qw = awq_b200.awq_repack(qw)
            fn = lambda: awq_b200.awq_gemm(x, qw, s, qz, 8, kernel=kern)  # noqa: E731
        work = f"{f[0]} M={m} K={k} N={n}"
    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    print(json.dumps({"case": work, "launches": args.steps,
                      "us_per_call": e0.elapsed_time(e1) * 1e3 / max(args.steps, 1)}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default=None, help="kernel:M:K:N -- run one small case (for ncu)")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--no-sweep", action="store_true",
                    help="skip the shape sweep and the MoE layer (extra keys of the 1-GPU line)")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
