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
value   device-resident: the step (AWQLinearMethod.apply of the four layers) is captured once in
        a CUDA graph and replayed; exactly --steps replays are timed with CUDA events on the
        launching stream between barriers, max over ranks.  The measurement is repeated until
        it has covered about 0.6 s, so that the nvidia-smi sampler (50 ms period) sees the
        clocks under load many times; the median repeat is reported, min and max beside it.
e2e     the same step through the layer API with the activations in pinned host memory:
        host->device copies, the kernels, device->host copies of the four outputs, every step;
        weights stay resident in HBM as they do while serving.  Each in-flight step (copies
        included) is one CUDA graph on its own stream; four are in flight, and the figure for
        one step at a time (what a single decoding sequence sees) is reported beside it.
layers  the layers are loaded with AWQConfig(decode_kmajor=True): gate_up keeps a K-major copy
        of its weights and runs the kernel that widens nibbles with tcgen05.cp (2 launches:
        activation digits + GEMM); qkv, o_proj and down run the registers->TMEM kernel.
bars    every row of the shape sweep and of the MoE table also times the installed vLLM's own
        kernels on the same GPU with the same protocol (awq_b200/vllm_ref.py): awq_gemm,
        awq_dequantize + matmul, awq_marlin_repack + marlin_gemm, fused_marlin_moe.
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
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the two M = 16 kernels, as a ratio to
# the launch's algorithmic bytes, from ncu captures of smaller cases (gemm_ts: K = 8192, N = 29568,
# 130.2 MB of traffic for 126.6 MB; gemm_q8: K = 8192, N = 36864, 164.0 MB for 158.6 MB); the
# traffic of the full-size launches is scaled by their bytes
NCU_TRAFFIC_RATIO = {"gemm_ts": 1.028, "gemm_q8": 1.034}
E2E_DEPTH = 4          # steps in flight in the end-to-end leg
TIMED_SECONDS = 0.6    # what the repeated device-resident measurement covers at least
ROTATE_BYTES = 400_000_000  # weight sets rotated per shape: at least this much and at least two


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


def cpu_model() -> str:
    try:
        for line in open("/proc/cpuinfo"):
            if line.lower().startswith("model name"):
                return line.split(":", 1)[1].strip()
    except Exception:
        pass
    return "unknown"


def cpu_reference_sample(reps: int, warmup: int = 3):
    """Times the fp32 dequantise-then-matmul of the o_proj shape (K = N = 8192, M = 16) on the
    host, and the matmul alone on the already dequantised matrix.  Returns a dict with the best
    and the mean of `reps` calls (after `warmup` untimed ones) for both."""
    import torch
    from awq_b200 import synth
    from oracle import awq_oracle as O

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    k, n = 8192, 8192
    qw, s, qz = synth.awq_linear_tensors(k, n, GROUP, seed=0)
    x = synth.activations(M_TOKENS, k, seed=0)
    for _ in range(max(1, warmup)):
        O.awq_gemm_fp32_torch(x, qw, s, qz, GROUP)
    times = []
    for _ in range(reps):
        t = time.perf_counter()
        O.awq_gemm_fp32_torch(x, qw, s, qz, GROUP)
        times.append(time.perf_counter() - t)
    w = torch.from_numpy(O.dequantize_fp32(qw.numpy(), s.numpy(), qz.numpy(), GROUP))
    xf = x.float()
    xf @ w
    mm = []
    for _ in range(max(reps, 3)):
        t = time.perf_counter()
        xf @ w
        mm.append(time.perf_counter() - t)
    return {"best": min(times), "mean": sum(times) / len(times), "cores": cores,
            "matmul_only_best": min(mm), "cpu_model": cpu_model(),
            "sample": f"o_proj K=8192 N=8192 M={M_TOKENS} group 128, torch fp32 "
                      f"dequantise+matmul on {cores} threads, best and mean of {reps} calls "
                      f"after {max(1, warmup)} warm-up calls"}


def cpu_baseline_block(c):
    wbytes = 8192 * 8192 // 2
    return {"value": wbytes / c["best"] / 1e12, "unit": UNIT, "cores": c["cores"], "kind": "port",
            "sample": c["sample"], "value_mean": wbytes / c["mean"] / 1e12,
            "ms_best": c["best"] * 1e3, "ms_mean": c["mean"] * 1e3,
            "matmul_only_ms_best": c["matmul_only_best"] * 1e3, "cpu_model": c["cpu_model"]}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    reps = max(3, min(args.steps, 20))
    warm = max(3, min(args.warmup, 5))      # a step is about 0.1 s of host time
    c = cpu_reference_sample(reps, warm)
    block = cpu_baseline_block(c)
    val = block["value"]
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": reps, "warmup": warm, "ms_per_step": c["best"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "awq_w4a16_linear_M16_qwen2.5-72b_layer (sampled: o_proj shape)",
                   "group_size": GROUP, "tokens": M_TOKENS},
        "cpu_baseline": block,
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ------------------------------------------------------------------------------------------
# CUDA arm
# ------------------------------------------------------------------------------------------


def bind_to_gpu_numa_node(device_index: int) -> dict:
    """Run this process on the CPUs of the NUMA node its GPU hangs off, so that the pinned host
    buffers allocated afterwards (first touch) and the copy submissions are local to the GPU's
    PCIe root.  Reads sysfs only; returns what it did for the JSON line."""
    import torch
    try:
        bus = torch.cuda.get_device_properties(device_index).pci_bus_id
        dom = torch.cuda.get_device_properties(device_index).pci_domain_id
        dev = torch.cuda.get_device_properties(device_index).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        with open(path) as f:
            node = int(f.read().strip())
        if node < 0:
            return {"numa_node": node, "bound": False}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return {"numa_node": node, "bound": False}
        os.sched_setaffinity(0, allowed)
        return {"numa_node": node, "bound": True, "cpus": len(allowed)}
    except Exception as e:   # sysfs not readable in this container: leave the affinity alone
        return {"bound": False, "note": f"{type(e).__name__}"}


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
    numa = bind_to_gpu_numa_node(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist.barrier()
    if rank != 0:
        awq_build.build()
    import awq_b200
    from awq_b200 import synth, _lib

    dev = torch.device("cuda", local)
    m = M_TOKENS
    method = awq_b200.AWQLinearMethod(awq_b200.AWQConfig(group_size=GROUP, decode_kmajor=True))
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
    kernels = ["gemm_q8_kernel (+ q8_prep_kernel)" if getattr(l, "qweight_kmajor", None) is not None
               else "gemm_ts_kernel" for l in layers]
    launches_per_step = sum(2 if "q8" in kname else 1 for kname in kernels)

    def step_device():
        return [method.apply(layer, x) for layer, x in zip(layers, x_dev)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def device_status():
        import ctypes
        v = ctypes.c_int(-1)
        _lib.load().awq_b200_device_status_clear(ctypes.byref(v))
        return v.value

    stream = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(stream):
        step_device()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step_device()
        warm = max(args.warmup, 3)
        w0 = torch.cuda.Event(enable_timing=True)
        w1 = torch.cuda.Event(enable_timing=True)
        w0.record(stream)
        for _ in range(warm):
            graph.replay()
        w1.record(stream)
        barrier()
        est = max(w0.elapsed_time(w1) * 1e-3 / warm, 1e-6)     # seconds per step, for sizing
        repeats = int(min(200, max(5, -(-TIMED_SECONDS // (est * args.steps)))))
        if world > 1:
            t = torch.tensor([repeats], device=dev, dtype=torch.int64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            repeats = int(t[0])
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
            time.sleep(0.12)
        barrier()
        t_wall0 = time.time()
        rep_ms = []
        for _ in range(repeats):
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record(stream)
            for _ in range(args.steps):          # exactly --steps steps between the events
                graph.replay()
            e1.record(stream)
            barrier()
            rep_ms.append(e0.elapsed_time(e1))
        t_wall1 = time.time()
        if world > 1:                              # every repeat: max over ranks
            t = torch.tensor(rep_ms, device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            rep_ms = t.tolist()
        rep_sorted = sorted(rep_ms)
        ms = rep_sorted[len(rep_sorted) // 2]
        status_after_timed = device_status()

        # ---- e2e through the layer API with host buffers ----
        # One CUDA graph per in-flight step, on its own stream with its own pinned buffers:
        # the four host->device copies, the four layers back to back, the four device->host
        # copies.  The host waits for a slot's outputs before it launches the slot again.
        def make_slot():
            st = torch.cuda.Stream(device=dev)
            xd = [torch.empty_like(x, device=dev) for x in xs]
            yp = [torch.empty((m, n), dtype=torch.float16).pin_memory() for _, (k, n) in shapes()]

            def body():
                for d, h in zip(xd, x_pin):
                    d.copy_(h, non_blocking=True)
                ys = [method.apply(layer, d) for layer, d in zip(layers, xd)]
                for h, y in zip(yp, ys):
                    h.copy_(y, non_blocking=True)

            with torch.cuda.stream(st):
                body()
                st.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    body()
            return {"stream": st, "graph": g, "y": yp, "done": None}

        def run_e2e(depth, steps):
            slots = [make_slot() for _ in range(depth)]

            def launch(i):
                sl = slots[i % depth]
                if sl["done"] is not None:
                    sl["done"].synchronize()      # the host has the outputs of the slot's last step
                with torch.cuda.stream(sl["stream"]):
                    sl["graph"].replay()
                    sl["done"] = torch.cuda.Event()
                    sl["done"].record(sl["stream"])

            def drain():
                for sl in slots:
                    if sl["done"] is not None:
                        sl["done"].synchronize()
                    stream.wait_stream(sl["stream"])

            for i in range(3 * depth):
                launch(i)
            drain()
            barrier()
            f0 = torch.cuda.Event(enable_timing=True)
            f1 = torch.cuda.Event(enable_timing=True)
            f0.record(stream)
            for sl in slots:
                sl["stream"].wait_stream(stream)
            for i in range(steps):
                launch(i)
            drain()
            f1.record(stream)
            barrier()
            out = f0.elapsed_time(f1)
            ref = [y.clone() for y in slots[0]["y"]]
            del slots
            return out, ref

        e2e_steps = max(20, min(args.steps * repeats, 2000))
        ms_e2e, y_host = run_e2e(E2E_DEPTH, e2e_steps)
        ms_e2e_serial, _ = run_e2e(1, max(20, e2e_steps // 4))
        if rank == 0:
            sampler.stop()
        # the outputs that came back to the host are the ones the device-resident step produces
        y_dev = step_device()
        torch.cuda.synchronize()
        e2e_matches = all(torch.equal(a, b.cpu()) for a, b in zip(y_host, y_dev))

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
        t = torch.tensor([ms_e2e, ms_e2e_serial], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e, ms_e2e_serial = float(t[0]), float(t[1])

    if rank == 0:
        wbytes = weight_bytes_per_step()
        sec = ms * 1e-3 / args.steps
        value = world * wbytes / sec / 1e12
        sec_e2e = ms_e2e * 1e-3 / e2e_steps
        sec_e2e_serial = ms_e2e_serial * 1e-3 / max(20, e2e_steps // 4)
        peak, peak_kind = measured_peak()
        achieved = wbytes / sec / 1e9  # GB/s of int4 weight bytes, one GPU
        achieved_all = all_bytes_per_step(m) / sec / 1e9
        cpu = cpu_baseline_block(cpu_reference_sample(3)) if world == 1 else None
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "repeats": repeats,
            "ms_per_step_min": rep_sorted[0] / args.steps, "ms_per_step_max": rep_sorted[-1] / args.steps,
            "config": {"workload": "awq_w4a16_linear_M16_qwen2.5-72b_layer (qkv,o_proj,gate_up,down)",
                       "group_size": GROUP, "tokens": m, "parallelism": f"replicas x{world}",
                       "l2": "inputs larger than L2 (438.8 MB of weights per step)",
                       "load_time_copies": "gate_up: K-major copy (AWQConfig(decode_kmajor=True))"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                         "kernel": "one step = " + ", ".join(
                             f"{name}: {kn}" for (name, _), kn in zip(shapes(), kernels)) +
                                   "; achieved = int4 weight bytes of the step / step time",
                         "achieved_all_bytes": achieved_all,
                         "traffic": sum(
                             NCU_TRAFFIC_RATIO["gemm_q8" if "q8" in kn else "gemm_ts"] *
                             (k * n // 2 + (k // GROUP) * n * 2 + (k // GROUP) * (n // 8) * 4 +
                              m * k * 2 + m * n * 2)
                             for (_, (k, n)), kn in zip(shapes(), kernels)),
                         "traffic_basis": "per step (sum of the step's launches); achieved is per "
                                          "step as well"},
            "cpu_baseline": cpu,
            "e2e": {"value": world * wbytes / sec_e2e / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": sum(m * k * 2 for _, (k, n) in shapes()),
                    "d2h_bytes_per_step": sum(m * n * 2 for _, (k, n) in shapes()),
                    "steps": e2e_steps, "ms_per_step": sec_e2e * 1e3, "steps_in_flight": E2E_DEPTH,
                    "one_step_at_a_time_ms": sec_e2e_serial * 1e3,
                    "one_step_at_a_time_value": world * wbytes / sec_e2e_serial / 1e12,
                    "outputs_equal_device_resident": bool(e2e_matches),
                    "host_binding": numa,
                    "pcie_GBps_per_gpu": (sum(m * k * 2 for _, (k, n) in shapes()) +
                                          sum(m * n * 2 for _, (k, n) in shapes())) / sec_e2e / 1e9},
            "gpu_launches": launches_per_step * args.steps,
            "device_status": status_after_timed,
            "clocks": sampler.summary(t_wall0, t_wall1),
        }
        if tp_result is not None:
            line["tp"] = tp_result
        if sweep is not None:
            tpeak = measured_tensor_peak()
            big = max((r for r in sweep if r.get("M", 0) >= 1024), key=lambda r: r["TFLOPs"])
            line["roofline_tensor"] = {"bound": "tensor", "achieved": big["TFLOPs"],
                                       "peak": tpeak[0], "unit": "TFLOP/s",
                                       "frac": big["TFLOPs"] / tpeak[0], "peak_kind": f"of {tpeak[1]}",
                                       "kernel": "gemm_tc_kernel<256,2>",
                                       "point": {"shape": big["shape"], "M": big["M"]}}
            line["sweep"] = sweep
            line["moe"] = moe
        line["serving"] = recorded_serving()
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


def _vllm_ref():
    """awq_b200.vllm_ref if the installed vLLM's compiled ops load, else None."""
    try:
        from awq_b200 import vllm_ref
        return vllm_ref if vllm_ref.available() else None
    except Exception:
        return None


def run_sweep(dev, stream):
    """Benchmark configuration 2: the four 72B layer shapes x M in {1 .. 4096}, 1 GPU.  Weights are
    rotated over at least two copies and at least ROTATE_BYTES (more than three times the L2),
    so every launch streams from HBM.  Every row also times vLLM's kernels for the same work
    with the same protocol."""
    import torch
    import awq_b200
    from awq_b200 import synth
    V = _vllm_ref()
    out = []
    for name, (k, n) in shapes():
        wbytes = k * n // 2
        copies = max(2, -(-ROTATE_BYTES // wbytes))
        base = [a.to(dev) for a in synth.awq_linear_tensors(k, n, GROUP, seed=1)]
        sets = [base] + [[a.clone() for a in base] for _ in range(copies - 1)]
        decode = [awq_b200.awq_repack(q[0]) for q in sets]
        kmajor = [awq_b200.awq_repack_kmajor(q[0]) for q in sets]
        marlin = [V.marlin_prepare(*q) for q in sets] if V is not None else None
        for m in synth.SWEEP_M:
            x = synth.activations(m, k).to(dev)
            reps = 3 if m >= 1024 else 10
            fns = [(lambda q=q: awq_b200.awq_gemm(x, q[0], q[1], q[2], 8)) for q in sets]
            t = graph_time(fns, stream, reps=reps)
            row = {"shape": name, "K": k, "N": n, "M": m, "weight_sets": copies,
                   "us": round(t * 1e6, 2), "weight_GBps": round(wbytes / t / 1e9, 1),
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
            if m <= 16:
                # ... and with the K-major copy (AWQConfig(decode_kmajor=True)): nibbles widened
                # by tcgen05.cp, int8 MMAs
                fns = [(lambda q=q, r=r: awq_b200.awq_gemm(x, r, q[1], q[2], 8,
                                                          kernel=awq_b200.KERNEL_Q8))
                       for q, r in zip(sets, kmajor)]
                tq = graph_time(fns, stream, reps=10)
                row["us_kmajor"] = round(tq * 1e6, 2)
                row["weight_GBps_kmajor"] = round(wbytes / tq / 1e9, 1)
            best = min(v for kk, v in row.items() if kk.startswith("us"))
            if V is None:
                row["vllm"] = "compiled ops of the installed vLLM did not load"
            else:
                try:
                    if m < 256:   # the route AWQLinearMethod.apply takes below 256 tokens
                        tv = graph_time([(lambda q=q: V.awq_gemm(x, q[0], q[1], q[2]))
                                         for q in sets], stream, reps=max(2, reps // 2))
                        row["vllm_awq_us"] = round(tv * 1e6, 2)
                    else:         # ... and from 256 tokens on: dequantize + matmul
                        tv = graph_time([(lambda q=q: V.awq_dequant_matmul(x, q[0], q[1], q[2]))
                                         for q in sets], stream, reps=2)
                        row["vllm_dequant_matmul_us"] = round(tv * 1e6, 2)
                    tm = graph_time([(lambda mq=mq: V.marlin_gemm(x, mq)) for mq in marlin],
                                    stream, reps=max(2, reps // 2))
                    row["vllm_marlin_us"] = round(tm * 1e6, 2)
                    row["speedup_vs_vllm_marlin"] = round(row["vllm_marlin_us"] / best, 2)
                except Exception as e:   # a vLLM op that refuses a shape is a missing column
                    row["vllm"] = f"{type(e).__name__}: {str(e)[:120]}"
            out.append(row)
        if name == "gate_up":
            # awq_dequantize (the materialising op of the >= 256-token route), 2.5 B per weight
            td = graph_time([(lambda q=q: awq_b200.awq_dequantize(q[0], q[1], q[2], 0, 0, 0))
                             for q in sets], stream, reps=3)
            out.append({"shape": name, "K": k, "N": n, "op": "awq_dequantize",
                        "us": round(td * 1e6, 1), "GBps": round(2.5 * k * n / td / 1e9, 1)})
        del sets, base, decode, kmajor, marlin
        torch.cuda.empty_cache()
    return out


def run_moe(dev, stream):
    """Benchmark configuration 3: Qwen3-30B-A3B fused-MoE layer (router -> permutation -> expert GEMMs ->
    sum), T in {1 .. 4096}, 1 GPU; vLLM's router + fused_marlin_moe beside it."""
    import torch
    import awq_b200
    from awq_b200 import synth
    V = _vllm_ref()
    cfg = synth.QWEN3_MOE
    e, h, i, k = cfg["experts"], cfg["hidden"], cfg["intermediate"], cfg["topk"]
    # two copies of the layer (302 MB of int4 each) alternate: more than the L2 holds
    layers = []
    for seed in (0, 1):
        w1, w2 = synth.moe_layer_tensors(e, h, i, GROUP, seed=seed)
        w1 = tuple(a.to(dev) for a in w1)
        w2 = tuple(a.to(dev) for a in w2)
        layers.append((w1, w2, awq_b200.awq_repack(w1[0]), awq_b200.awq_repack(w2[0]),
                       V.marlin_moe_prepare(w1, w2) if V is not None else None))
    from awq_b200 import _lib
    block_of = lambda t: _lib.load().awq_b200_moe_block_size(t, k, e, h, i, GROUP)  # noqa: E731
    awq_b200.reserve_workspace(awq_b200.moe_workspace_bytes(max(synth.MOE_TOKENS), k, e, h, i), dev)
    out = []
    from awq_b200 import ops as awq_ops
    # the benchmark's token counts, plus the few-token decode points where the direct mode (no
    # permutation kernel, slot sum inside the down GEMM) competes with the permuted chain
    for t in sorted(set(synth.MOE_TOKENS) | {2, 4, 8}):
        x = synth.activations(t, h).to(dev)
        logits = synth.gating_logits(t, e).to(dev)
        _, ids, _ = awq_b200.fused_topk(x, logits, k, True)
        hit = int(torch.unique(ids).numel())
        reps = 5 if t >= 1024 else 20
        with torch.cuda.stream(stream):
            awq_b200.reserve_workspace(awq_b200.moe_workspace_bytes(max(synth.MOE_TOKENS), k, e, h, i), dev)
        sec = graph_time([(lambda L=L: awq_b200.fused_moe(x, L[0], L[1], logits, k, True))
                          for L in layers], stream, reps=reps)
        byts = hit * (2359296 + 73728 + 18432) + t * h * 2 * 2
        row = {"T": t, "experts_hit": hit, "us": round(sec * 1e6, 1),
               "GBps": round(byts / sec / 1e9, 1),
               "TFLOPs": round(t * 75497472 / sec / 1e12, 2)}
        if t * k <= 64:
            # both chains at the few-token points: pairs at or below the limit go direct
            keep = awq_ops.MOE_DIRECT_MAX_PAIRS
            for name, limit in (("us_direct", 64), ("us_permuted", 0)):
                awq_ops.MOE_DIRECT_MAX_PAIRS = limit
                sm = graph_time([(lambda L=L: awq_b200.fused_moe(x, L[0], L[1], logits, k, True))
                                 for L in layers], stream, reps=reps)
                row[name] = round(sm * 1e6, 1)
            awq_ops.MOE_DIRECT_MAX_PAIRS = keep
            row["direct_by_default"] = t * k <= keep
        if block_of(t) in (8, 16):
            # the same layer with the optional decode-layout copies of the expert weights
            def layer(L):
                w, ids2, _ = awq_b200.fused_topk(x, logits, k, True)
                return awq_b200.fused_experts(x, L[0], L[1], w, ids2, w1_decode=L[2], w2_decode=L[3])
            sd = graph_time([(lambda L=L: layer(L)) for L in layers], stream, reps=reps)
            row["us_decode_layout"] = round(sd * 1e6, 1)
        if V is None:
            row["vllm"] = "compiled ops of the installed vLLM did not load"
        else:
            try:
                def theirs(L):
                    w, ids2 = V.topk_softmax(logits, k, True)
                    return V.marlin_moe(x, L[4], w, ids2)
                sv = graph_time([(lambda L=L: theirs(L)) for L in layers], stream,
                                reps=max(2, reps // 2))
                row["vllm_marlin_moe_us"] = round(sv * 1e6, 1)
                best = min(v for kk, v in row.items() if kk.startswith("us"))
                row["speedup_vs_vllm_marlin_moe"] = round(row["vllm_marlin_moe_us"] / best, 2)
            except Exception as ex:
                row["vllm"] = f"{type(ex).__name__}: {str(ex)[:120]}"
        out.append(row)
    return out


def _device_status() -> int:
    import ctypes
    from awq_b200 import _lib
    v = ctypes.c_int(-1)
    _lib.load().awq_b200_device_status_clear(ctypes.byref(v))
    return v.value


def run_tp(args, world, rank, dev, stream, barrier):
    """The same layer sharded over `world` GPUs: qkv/gate_up column-parallel, o_proj/down
    row-parallel with the fp16 [M, 8192] partial outputs all-reduced over NVLink (NCCL).  The
    down projection's K (231 groups) is padded to a multiple of the TP degree.  Before timing,
    the row-parallel results are compared with the unsharded layer computed on this GPU; the
    step is timed both as eager launches and captured in a CUDA graph (NCCL included)."""
    import torch
    import torch.distributed as dist
    import awq_b200
    from awq_b200 import synth, tp

    m = M_TOKENS
    shards, xs, full = [], [], []
    for i, (name, (k, n)) in enumerate(shapes()):
        qw, s, qz = synth.awq_linear_tensors(k, n, GROUP, seed=i)
        x_full = synth.activations(m, k, seed=i)
        if name in ("qkv", "gate_up"):
            sh = tp.shard_columns(qw, s, qz, rank, world)
            x = x_full
            shards.append(("col", tuple(a.to(dev) for a in sh)))
            full.append(None)
        else:
            full.append((x_full.to(dev), qw.to(dev), s.to(dev), qz.to(dev)))
            qw, s, qz = tp.pad_k_for_tp(qw, s, qz, world)
            sh = tp.shard_rows(qw, s, qz, rank, world)
            x = tp.shard_input(tp.pad_x_for_tp(x_full, qw.shape[0]), rank, world)
            shards.append(("row", tuple(a.to(dev) for a in sh)))
        xs.append(x.to(dev))

    def step():
        outs = []
        for (kind, sh), x in zip(shards, xs):
            outs.append(tp.column_parallel_forward(x, sh) if kind == "col"
                        else tp.row_parallel_forward(x, sh))
        return outs

    # the same step with the one-shot peer-memory all-reduce fed directly by the GEMM epilogue
    comm, comm_note = None, None
    try:
        comm = tp.PeerAllReduce(m * 8192 * 2)
    except Exception as e:
        comm_note = f"{type(e).__name__}: {str(e)[:160]}"

    def step_peer():
        outs, call = [], 0
        for (kind, sh), x in zip(shards, xs):
            if kind == "col":
                outs.append(tp.column_parallel_forward(x, sh))
            else:
                outs.append(tp.row_parallel_forward(x, sh, comm=comm, slot=tp.slot_for_call(call)))
                call += 1
        return outs

    # ---- parity: the all-reduced row-parallel outputs against the unsharded product ----
    outs = step()
    torch.cuda.synchronize()
    worst = 0.0
    for o, f in zip(outs, full):
        if f is None:
            continue
        ref = awq_b200.awq_gemm(f[0], f[1], f[2], f[3], 8).float()
        err = float((o.float() - ref).abs().max() / ref.abs().max())
        worst = max(worst, err)
    worst_peer = 0.0
    if comm is not None:
        outs_peer = step_peer()
        torch.cuda.synchronize()
        for o, f in zip(outs_peer, full):
            if f is None:
                continue
            ref = awq_b200.awq_gemm(f[0], f[1], f[2], f[3], 8).float()
            worst_peer = max(worst_peer, float((o.float() - ref).abs().max() / ref.abs().max()))
    t = torch.tensor([worst, worst_peer], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    parity, parity_peer = float(t[0]), float(t[1])
    del full

    def timed(fn, steps):
        for _ in range(5):
            fn()
        barrier()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            fn()
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]) * 1e-3 / steps

    steps = max(1, min(args.steps, 500))
    sec_eager = timed(step, steps)
    sec_graph = None
    try:
        step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            step()
        sec_graph = timed(g.replay, steps)
    except Exception as e:  # NCCL capture not possible in this configuration
        graph_note = f"{type(e).__name__}: {str(e)[:100]}"
    # without the collectives: what the exchange step costs
    def step_no_ar():
        for (kind, sh), x in zip(shards, xs):
            tp.column_parallel_forward(x, sh)
    sec_no_ar = None
    try:
        step_no_ar()
        torch.cuda.synchronize()
        g2 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g2, stream=stream):
            step_no_ar()
        sec_no_ar = timed(g2.replay, steps)
    except Exception:
        pass
    sec_peer = sec_peer_eager = None
    if comm is not None:
        sec_peer_eager = timed(step_peer, steps)
        g3 = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g3, stream=stream):
            step_peer()
        sec_peer = timed(g3.replay, steps)
        step_peer()                    # the replays left the call numbering consistent
        torch.cuda.synchronize()
    # the exchange alone (no GEMM in front of it): 20 calls per replayed graph, fp16 [M, 8192]
    alone = None
    if comm is not None:
        try:
            calls = 20
            xa = torch.randn(m, 8192, device=dev).half()

            def peer_alone():
                for i in range(calls):
                    comm.reduce(i & 1, m, 8192)

            def nccl_alone():
                for i in range(calls):
                    dist.all_reduce(xa)

            alone = {}
            for name, body in (("peer_us", peer_alone), ("nccl_us", nccl_alone)):
                body()
                torch.cuda.synchronize()
                ga = torch.cuda.CUDAGraph()
                with torch.cuda.graph(ga, stream=stream):
                    body()
                alone[name] = round(timed(ga.replay, max(10, steps // 10)) / calls * 1e6, 2)
                del ga
        except Exception as e:
            alone = {"note": f"{type(e).__name__}: {str(e)[:100]}"}
    sec = min(x for x in (sec_graph, sec_eager, sec_peer) if x is not None)
    res = {"parallelism": f"tp{world}", "scaling": "strong", "ms_per_step": sec * 1e3,
           "ms_per_step_graph_peer_all_reduce": None if sec_peer is None else sec_peer * 1e3,
           "ms_per_step_eager_peer_all_reduce":
               None if sec_peer_eager is None else sec_peer_eager * 1e3,
           "parity_rel_err_peer_all_reduce": parity_peer if comm is not None else None,
           "peer_all_reduce": "one-shot kernel over peer-mapped regions, GEMM writes its partial "
                              "into the region (awq_b200_allreduce)" if comm is not None
                              else f"unavailable: {comm_note}",
           "exchange_alone": alone,
           "device_status": _device_status(),
           "ms_per_step_eager": sec_eager * 1e3,
           "ms_per_step_graph": None if sec_graph is None else sec_graph * 1e3,
           "ms_per_step_graph_without_all_reduce": None if sec_no_ar is None else sec_no_ar * 1e3,
           "value": weight_bytes_per_step() / sec / 1e12, "unit": UNIT, "steps": steps,
           "parity_rel_err": parity,
           "collective": "nccl all_reduce fp16 [16, 8192] after o_proj and down"}
    if sec_graph is None:
        res["graph_note"] = graph_note
    if comm is not None:
        del g3
        comm.close()
    return res


def recorded_serving():
    """The serving result files committed under profiles/serving (written by
    ``python -m awq_b200.serving.run`` in the reference's result layout), parsed with the
    reference report's labels.  They are recordings of earlier runs on B200 boxes of this pool,
    not measurements of this invocation: ``bench.py --serving`` measures live."""
    import glob
    import re
    from awq_b200.serving import client
    runs = []
    for path in sorted(glob.glob(os.path.join(ROOT, "profiles", "serving", "*_vllm_benchmark.txt"))):
        name = os.path.basename(path)
        mt = re.match(r"(b200_x_(\d+))_(.+?)(-stock-(fill|off))?-c(\d+)_vllm_benchmark\.txt", name)
        if not mt:
            continue
        with open(path) as f:
            parsed = client.parse_result_block(f.read())
        if parsed:
            runs.append({"file": "profiles/serving/" + name, "gpus": int(mt.group(2)),
                         "kernels": "stock vLLM (Marlin), same seeded weights" if mt.group(4)
                         else "this package (plug-in)" +
                         (", decode-layout copies of the weights" if "decode-copies" in name else ""),
                         "concurrency": int(mt.group(6)), **parsed})
    return {"source": "recorded result files (not measured by this invocation)",
            "workload": "Qwen3-30B-A3B architecture, random-init AWQ, 1000 in / 1000 out, "
                        "vllm bench serve on /v1/chat/completions, TP=1 replicas",
            "runs": runs}


def run_serving(args):
    """Live serving measurement on ``--gpus`` replicas (no torchrun: the servers own the GPUs)."""
    from awq_b200.serving import run as srun
    sargs = srun.parser().parse_args([
        "--instances", str(args.gpus), "--concurrency", args.serving_concurrency,
        "--num-prompts", args.serving_prompts, "--plugin", args.serving_plugin,
        "--results-dir", os.path.join(ROOT, "results"), "--force"])
    out = srun.run(sargs)
    best = max(out["runs"], key=lambda r: r.get("output_throughput", 0.0))
    print(json.dumps({"metric": "decode output tok/s per box", "value": best["output_throughput"],
                      "unit": "tok/s", "n_gpus": args.gpus, "higher_is_better": True,
                      "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
                      "config": {"workload": "qwen3-30b-a3b random-init AWQ, 1000 in / 1000 out, "
                                             f"concurrency {best['concurrency']}",
                                 "parallelism": f"replicas x{args.gpus}"},
                      "serving": out}))


def run_case(args):
    """`--case kernel:M:K:N` launches one AWQ linear of that shape `--steps` times after
    `--warmup` launches and prints its CUDA-event time: the small, bounded command the ncu
    captures under profiles/ are taken with.  kernel: auto | stream | stream_exact | stream_rp
    (decode-layout copy of qweight) | q8 (K-major copy) | tcgen05 | ts | wt | generic | dequantize | moe:T (Qwen3-30B-A3B layer with T tokens; K and N ignored)."""
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
                    "stream_rp": awq_b200.KERNEL_STREAM_RP, "q8": awq_b200.KERNEL_Q8,
                    "generic": awq_b200.KERNEL_GENERIC}[f[0]]
            if f[0] == "stream_rp":
                qw = awq_b200.awq_repack(qw)
            if f[0] == "q8":
                qw = awq_b200.awq_repack_kmajor(qw)
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
    ap.add_argument("--serving", action="store_true",
                    help="serve the random-init Qwen3-30B-A3B model on --gpus replicas and run the "
                         "OpenAI-endpoint client (minutes; run without torchrun)")
    ap.add_argument("--serving-concurrency", default="64,256")
    ap.add_argument("--serving-prompts", default="256,1024")
    ap.add_argument("--serving-plugin", default="on", choices=["on", "fill", "off"])
    args = ap.parse_args()
    if args.serving:
        run_serving(args)
    elif args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_cuda(args)


if __name__ == "__main__":
    main()
