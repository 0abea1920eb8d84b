#!/usr/bin/env python
"""Benchmark of the executor hot path: inferences/sec on the ResNet-style tower (f32, batch 256 per
GPU), one process per GPU, batch-sharded with no collective.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line (rank 0).  A "step" is one pass of the planned step list over one batch.
  value      inferences/s with the inputs already resident in HBM: two executors of the graph per GPU run
             alternate batches (run_async), a pool of input sets larger than L2 rotates through their input
             buffers; timed with CUDA events.  `config.one_executor_flushed` is the same with one executor,
             one step after the other and an L2 flush between timed iterations
  e2e        the same metric through the public `evaluate` halves with host buffers: pinned host -> device
             copy of the inputs, the steps, device -> host copy of the outputs, the next batch submitted
             before the current one is waited for; `e2e.one_executor_serial` is plain `evaluate` in series
  roofline   the dominant kernel (the convolution chain that runs the residual tower): algorithmic FLOP per launch / measured
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
# DRAM bytes (read + written) per launch of the trunk convolution at batch 256, from one ncu capture of
# this bench: 9.05 MB for conv+bias+relu and 17.44 MB with the residual operand (the output stays in L2,
# 0 bytes written back); the two alternate in the trunk, so the mean is quoted.
TRUNK_CONV_DRAM_BYTES = 13.24e6
# DRAM bytes per launch of the convolution chain (all 33 tower layers) at batch 256, from one ncu capture
# of this bench: 20.53 MB read (filters and input, once), 0 written back (the output stays in L2).
CHAIN_DRAM_BYTES = 20.54e6
WORKLOAD = "resnet_tower_f32_b256 (21x8x8 planes, stem + 16 residual blocks @128ch, policy 73x8x8 softmax, value 3 softmax)"


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML polled every 5 ms from
    a thread (read-only queries), or `nvidia-smi -lms` when NVML cannot be loaded.  Sampling starts before
    the warm-up; only samples that arrive between `mark_start()` and `stop()` are summarised."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, device_index: int, uuid: str = None):
        self.device_index = device_index
        self.uuid = uuid
        self.samples = []          # (arrival time, sm MHz, set of reasons)
        self.max_clock = None
        self.proc = None
        self.thread = None
        self.running = False
        self.t_start = None
        self.source = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            handle = (pynvml.nvmlDeviceGetHandleByUUID(self.uuid.encode()) if self.uuid
                      else pynvml.nvmlDeviceGetHandleByIndex(self.device_index))
            self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
            masks = {"hw_slowdown": pynvml.nvmlClocksThrottleReasonHwSlowdown,
                     "hw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonHwThermalSlowdown,
                     "sw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonSwThermalSlowdown,
                     "sw_power_cap": pynvml.nvmlClocksThrottleReasonSwPowerCap}
            self.running = True
            self.source = "nvml"

            def poll():
                while self.running:
                    try:
                        mhz = float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM))
                        bits = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                        self.samples.append((time.perf_counter(), mhz, {n for n, m in masks.items() if bits & m}))
                    except pynvml.NVMLError:
                        pass
                    time.sleep(0.005)

            self.thread = threading.Thread(target=poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.running = False
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20",
                 "-i", self.uuid or str(self.device_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.source = "nvidia-smi"
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                mhz = float(parts[0])
                self.max_clock = float(parts[1])
            except ValueError:
                continue
            reasons = {n for n, v in zip(self.NAMES, parts[2:6]) if v.lower().startswith("active")}
            self.samples.append((time.perf_counter(), mhz, reasons))

    def mark_start(self):
        self.t_start = time.perf_counter()

    def stop(self):
        t_end = time.perf_counter()
        if self.source is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source available"], "samples": 0}
        self.running = False
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        elif self.thread is not None:
            self.thread.join(timeout=1)
        t0 = self.t_start if self.t_start is not None else 0.0
        window = [s for s in list(self.samples) if t0 <= s[0] <= t_end]
        clocks = [s[1] for s in window]
        reasons = set().union(*[s[2] for s in window]) if window else set()
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": self.max_clock,
                "reasons": sorted(reasons), "samples": len(clocks), "source": self.source}


def oracle_runner(sample_batch: int):
    """Returns a function that pushes `sample_batch` boards of the same tower through the CPU oracle once."""
    from kyanite_b200.configs import resnet_tower
    from oracle.cpu_eval import cpu_eval_graph, parse_graph
    graph, make_inputs = resnet_tower()
    parsed = parse_graph(graph.to_bytes())
    inputs = make_inputs(sample_batch, 1)
    return lambda: cpu_eval_graph(parsed, sample_batch, inputs)


def cpu_oracle_rate(sample_batch: int, repeats: int):
    """inferences/s of the CPU oracle on `sample_batch` boards of the same tower."""
    run = oracle_runner(sample_batch)
    run()   # warm the BLAS threads
    t0 = time.perf_counter()
    for _ in range(repeats):
        run()
    dt = time.perf_counter() - t0
    return sample_batch * repeats / dt, dt


def run_reference(args, rank, world):
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    # bounded sample: boards per step chosen so that warm-up + steps take about 90 s on this host
    probe_rate, _ = cpu_oracle_rate(32, 1)
    budget_boards = probe_rate * 90.0
    sample = int(max(8, min(BATCH, budget_boards // max(1, args.steps + args.warmup))))
    sample -= sample % 8
    run = oracle_runner(sample)
    for _ in range(args.warmup):
        run()
    rates = []
    t0 = time.perf_counter()
    for _ in range(args.steps):
        t1 = time.perf_counter()
        run()
        rates.append(sample / (time.perf_counter() - t1))
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
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--math", default="tf32", choices=["tf32", "f32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-chain", action="store_true", help="one launch per convolution instead of the merged chain kernel (A/B)")
    ap.add_argument("--e2e-executors", type=int, default=2, help="executors per GPU in the end-to-end measurement")
    ap.add_argument("--e2e-dense", type=int, default=0, help="1: the end-to-end executors use KN_FLAG_DENSE_CONV_CHAIN")
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
    from kyanite_b200.executor import FLAG_DENSE_CONV_CHAIN, FLAG_NO_CONV_CHAIN, MATH_F32, MATH_TF32, CudaExecutor

    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    graph, make_inputs = resnet_tower()
    math_mode = MATH_TF32 if args.math == "tf32" else MATH_F32
    ex = CudaExecutor(local_rank, graph, BATCH, math_mode=math_mode, flags=FLAG_NO_CONV_CHAIN if args.no_chain else 0)
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

    sampler = ClockSampler(local_rank, "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid))
    sampler.start()

    # ---- warm-up (also captures the CUDA graph)
    for _ in range(args.warmup):
        ex.evaluate_staged()
    ex.synchronize()

    launches = 0

    # ---- device-resident: K timed iterations of run_async, L2 flushed in between
    barrier()
    sampler.mark_start()
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
    # (a) one executor, one call after the other: upload, steps and download of a batch in series
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
    serial_ms = e2e_start.elapsed_time(e2e_end)
    # (b) two executors of the same graph on this GPU, the way the reference's hosts keep a GPU busy (several
    # executor threads per device): the next batch is submitted before the current one is waited for, so its
    # upload and the previous download run on the copy engines while the GPU computes.  Every batch is
    # still uploaded from and downloaded to pinned host memory inside the timed region, and every result
    # is complete in host memory when its evaluate_staged_end returns.
    e2e_flags = FLAG_NO_CONV_CHAIN if args.no_chain else (FLAG_DENSE_CONV_CHAIN if args.e2e_dense else 0)
    pair = []
    for k in range(args.e2e_executors):
        e = CudaExecutor(local_rank, graph, BATCH, math_mode=math_mode, flags=e2e_flags)
        for dst, src in zip(e.host_inputs, make_inputs(BATCH, 1001 + 17 * k + rank)):
            dst[...] = src
        pair.append(e)
    streams = [torch.cuda.ExternalStream(e.stream(), device=torch.device("cuda", local_rank)) for e in pair]
    for e in pair:
        for _ in range(max(2, args.warmup)):
            e.evaluate_staged()
    barrier()
    e2e_start = torch.cuda.Event(enable_timing=True)
    e2e_end = torch.cuda.Event(enable_timing=True)
    n_ex = len(pair)
    e2e_launches = pair[0].step_count()[1]
    e2e_start.record(streams[0])
    for k in range(min(n_ex - 1, args.steps)):
        pair[k].evaluate_staged_begin()
    for i in range(args.steps):
        if i + n_ex - 1 < args.steps:
            pair[(i + n_ex - 1) % n_ex].evaluate_staged_begin()
        pair[i % n_ex].evaluate_staged_end()
        launches += e2e_launches
    e2e_end.record(streams[(args.steps - 1) % n_ex])
    barrier()
    e2e_ms = e2e_start.elapsed_time(e2e_end)

    # ---- device-resident throughput (`value`): the same executors, batches already in HBM.  No flush here:
    # a pool of input sets larger than the 126 MB L2 rotates through the executors' input buffers (one
    # device-to-device copy per step, inside the timed region), so no step finds its input in L2, while the
    # 20 MB of weights stay there as they do in steady-state serving.  With two executors alternating, CTAs of
    # the next batch fill the SMs the current one leaves idle (128 CTAs for 148 SMs).
    class _DevArray:
        def __init__(self, ptr, shape):
            self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (ptr, False), "version": 3}

    pool_sets = 128
    gen = torch.Generator(device="cuda")
    gen.manual_seed(1234 + rank)
    pools, dev_in = [], [[] for _ in pair]
    for idx, arr in enumerate(inputs):
        pool = (torch.rand((pool_sets,) + tuple(arr.shape), device="cuda", generator=gen) < 0.1).to(torch.float32)
        pools.append(pool)
        for k, e in enumerate(pair):
            ptr, _ = e.device_buffer(False, idx)
            dev_in[k].append(torch.as_tensor(_DevArray(ptr, arr.shape), device="cuda"))
    pool_bytes = sum(p.numel() * 4 for p in pools)
    barrier()
    pipe_start = torch.cuda.Event(enable_timing=True)
    pipe_ends = [torch.cuda.Event(enable_timing=True) for _ in pair]
    pipe_start.record(streams[0])
    for st in streams[1:]:
        st.wait_event(pipe_start)
    for i in range(args.steps):
        k = i % n_ex
        with torch.cuda.stream(streams[k]):
            for pool, dst in zip(pools, dev_in[k]):
                dst.copy_(pool[i % pool_sets], non_blocking=True)
        pair[k].run_async()
        launches += e2e_launches
    for ev, st in zip(pipe_ends, streams):
        ev.record(st)
    barrier()
    pipe_ms = max(pipe_start.elapsed_time(ev) for ev in pipe_ends)
    clocks = sampler.stop()
    for e in pair:
        e.close()

    # ---- dominant kernel: the contraction step with the most FLOP (the convolution chain that runs the
    # whole residual tower in one launch; with chains switched off, the trunk convolutions, which are
    # timed one by one and averaged).  Each is launched 20x back to back between one pair of CUDA events
    # on the executor's stream.
    ex.set_profile(True)
    ex.run_async()
    contractions = []
    for line in ex.last_profile().splitlines():
        parts = line.split()
        if len(parts) > 6 and parts[0].isdigit() and parts[1].split("/")[0] in ("Conv", "ConvChain", "Gemm"):
            contractions.append((int(parts[0]), float(parts[4]), parts[1], " ".join(parts[5:])))
    ex.set_profile(False)
    dominant = []
    if contractions:
        top = max(c[1] for c in contractions)
        dominant = [(ex.time_step(idx, 20), flop, kind, desc) for idx, flop, kind, desc in contractions if flop == top]

    t = torch.tensor([dev_ms, e2e_ms, serial_ms, pipe_ms], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, serial_ms, pipe_ms = t.tolist()

    if rank == 0:
        peaks = load_peaks()
        total = BATCH * world * args.steps
        value = total / (pipe_ms / 1000.0)
        e2e_value = total / (e2e_ms / 1000.0)
        tensor_peak = peaks["bf16_tflops"] / 2.0   # TF32 dense = half the bf16 rate
        roofline = None
        if dominant:
            us = statistics.mean(u for u, _, _, _ in dominant)
            flop, kind, desc = dominant[0][1], dominant[0][2], dominant[0][3]
            achieved = flop / (us * 1e-6) / 1e12
            chain = kind.startswith("ConvChain")
            roofline = {"bound": "tensor", "kernel": ("conv_chain_kernel: " if chain else "tc_conv_cl_kernel: ") + desc,
                        "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s", "frac": achieved / tensor_peak,
                        "traffic": CHAIN_DRAM_BYTES if chain else TRUNK_CONV_DRAM_BYTES,
                        "peak_source": f"{peaks['source']} bf16 burst / 2 (tf32)", "us_per_launch": us,
                        "gflop_per_launch": flop / 1e9, "launches_per_step": len(dominant)}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": pipe_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32 operands, f32 storage and accumulate" if args.math == "tf32" else "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_per_gpu": BATCH, "parallelism": f"batch-sharded x{world}, no collective",
                       "executors_per_gpu": args.e2e_executors,
                       "l2": f"no flush: {pool_sets} input sets ({pool_bytes / 1e6:.0f} MB, larger than the 126 MB L2) rotate "
                             "through the executors' input buffers, one device-to-device copy per step inside the timed "
                             "region; weights (20 MB) stay in L2",
                       "one_executor_flushed": {"value": total / (dev_ms / 1000.0), "ms_per_step": dev_ms / args.steps,
                                                "l2": "one executor, steps one after the other, 256 MiB L2 flush "
                                                      "between timed iterations"},
                       "gflop_per_step": resnet_tower_flops(BATCH) / 1e9, "steps_per_run": steps_per_run},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps,
                    "executors_per_gpu": args.e2e_executors, "dense_conv_chain": bool(args.e2e_dense),
                    "mode": "several executors per GPU, the next batches submitted before the current one is waited for "
                            "(kn_executor_evaluate_begin / _end); every batch is uploaded from and downloaded to "
                            "pinned host memory inside the timed region",
                    "one_executor_serial": {"value": total / (serial_ms / 1000.0), "ms_per_step": serial_ms / args.steps}},
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
