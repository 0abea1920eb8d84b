#!/usr/bin/env python
"""Benchmark of the executor hot path: inferences/sec on the ResNet-style tower (f32, batch 256 per
GPU), one process per GPU, batch-sharded with no collective.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  A "step" is one pass of the planned step list over one batch.
  value      inferences/s with the inputs already resident in HBM (run_async only), timed with
             CUDA events on the executor's stream, L2 flushed between timed iterations
  e2e        the same metric through the public `evaluate` call with host buffers: pinned
             host -> device copy of the inputs, the steps, device -> host copy of the outputs
  roofline   the dominant kernel (trunk 3x3 convolution): algorithmic FLOP per launch / measured
             launch time, against the measured dense tensor peak
  cpu_baseline  the CPU oracle (numpy restatement of the reference's cpu_eval_graph) timed on this
             box's host cores on a bounded sample
`--impl reference` times that CPU oracle alone (the reference's own CPU implementation is Rust and
cannot be built in this image).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "inferences_per_sec"
UNIT = "inferences/s"
BATCH = 256
WORKLOAD = "resnet_tower_f32_b256 (21x8x8 planes, stem + 16 residual blocks @128ch, policy 73x8x8 softmax, value 3 softmax)"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            try:
                clocks.append(float(s[0]))
                max_clock = float(s[1])
            except ValueError:
                continue
            for name, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": max_clock,
                "reasons": sorted(reasons), "samples": len(clocks)}


def cpu_oracle_rate(sample_batch: int, repeats: int):
    """inferences/s of the CPU oracle on `sample_batch` boards of the same tower."""
    from kyanite_b200.configs import resnet_tower
    from oracle.cpu_eval import cpu_eval_graph, parse_graph
    graph, make_inputs = resnet_tower()
    parsed = parse_graph(graph.to_bytes())
    inputs = make_inputs(sample_batch, 1)
    cpu_eval_graph(parsed, sample_batch, inputs)   # warm the BLAS threads
    t0 = time.perf_counter()
    for _ in range(repeats):
        cpu_eval_graph(parsed, sample_batch, inputs)
    dt = time.perf_counter() - t0
    return sample_batch * repeats / dt, dt


def run_reference(args, rank, world):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    sample = BATCH
    rates = []
    for _ in range(args.warmup):
        cpu_oracle_rate(sample, 1)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        r, _ = cpu_oracle_rate(sample, 1)
        rates.append(r)
    dt = time.perf_counter() - t0
    value = statistics.mean(rates)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1000.0 * dt / max(1, args.steps), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch_per_step": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{sample} boards per step through the numpy oracle (im2col + BLAS sgemm on all cores)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--math", default="tf32", choices=["tf32", "f32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    from kyanite_b200.configs import resnet_tower, resnet_tower_flops
    from kyanite_b200.executor import MATH_F32, MATH_TF32, CudaExecutor

    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    graph, make_inputs = resnet_tower()
    math_mode = MATH_TF32 if args.math == "tf32" else MATH_F32
    ex = CudaExecutor(local_rank, graph, BATCH, math_mode=math_mode)
    inputs = make_inputs(BATCH, 1 + rank)
    for dst, src in zip(ex.host_inputs, inputs):
        dst[...] = src
    steps_per_run, launches_per_run = ex.step_count()

    stream = torch.cuda.ExternalStream(ex.stream(), device=torch.device("cuda", local_rank))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")   # 2x the 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- warm-up (also captures the CUDA graph)
    for _ in range(args.warmup):
        ex.evaluate_staged()
    ex.synchronize()

    sampler = ClockSampler(local_rank)
    launches = 0

    # ---- device-resident: K timed iterations of run_async, L2 flushed in between
    barrier()
    sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with torch.cuda.stream(stream):
        for i in range(args.steps):
            flush.zero_()
            starts[i].record(stream)
            ex.run_async()
            ends[i].record(stream)
            launches += launches_per_run
    barrier()
    dev_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))

    # ---- end to end through evaluate(): pinned H2D + steps + D2H, host buffers
    h2d = sum(a.nbytes for a in ex.host_inputs)
    d2h = sum(a.nbytes for a in ex.host_outputs)
    barrier()
    e2e_start = torch.cuda.Event(enable_timing=True)
    e2e_end = torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e2e_start.record(stream)
        for i in range(args.steps):
            ex.evaluate_staged()
            launches += launches_per_run
        e2e_end.record(stream)
    barrier()
    e2e_ms = e2e_start.elapsed_time(e2e_end)
    clocks = sampler.stop()

    # ---- dominant kernel: every trunk convolution step, each launched back to back between one pair
    # of CUDA events on the executor's stream (its operands, 8.4 MB activations and 0.6 MB filter, are
    # L2-resident there exactly as they are inside the step list)
    ex.set_profile(True)
    ex.run_async()
    trunk = []
    for line in ex.last_profile().splitlines():
        parts = line.split()
        if len(parts) > 6 and parts[1].startswith("Conv") and "c=128" in line and "k=128" in line and "rs=3x3" in line:
            trunk.append((int(parts[0]), float(parts[4]), parts[1]))
    ex.set_profile(False)
    conv_us = [(ex.time_step(idx, 20), flop, kind) for idx, flop, kind in trunk]

    t = torch.tensor([dev_ms, e2e_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = t.tolist()

    if rank == 0:
        peaks = load_peaks()
        total = BATCH * world * args.steps
        value = total / (dev_ms / 1000.0)
        e2e_value = total / (e2e_ms / 1000.0)
        tensor_peak = peaks["bf16_tflops"] / 2.0   # TF32 dense = half the bf16 rate
        roofline = None
        if conv_us:
            us = statistics.mean(u for u, _, _ in conv_us)
            flop = conv_us[0][1]
            achieved = flop / (us * 1e-6) / 1e12
            kind = conv_us[0][2]
            roofline = {"bound": "tensor", "kernel": "trunk conv3x3 128->128 (" + kind + ")", "achieved": achieved,
                        "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak, "traffic": None,
                        "peak_source": f"{peaks['source']} bf16 burst / 2 (tf32)", "us_per_launch": us}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32 operands, f32 storage and accumulate" if args.math == "tf32" else "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_per_gpu": BATCH, "parallelism": f"batch-sharded x{world}, no collective",
                       "l2": "flushed with a 256 MiB write between timed iterations",
                       "gflop_per_step": resnet_tower_flops(BATCH) / 1e9, "steps_per_run": steps_per_run},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": roofline,
        }
        if world == 1 and not args.no_cpu_baseline:
            rate, dt = cpu_oracle_rate(BATCH, 4)
            line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": f"4 x {BATCH} boards through the numpy oracle in {dt:.1f} s"}
        print(json.dumps(line), flush=True)

    ex.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
