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
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p.get("bf16_tflops_sustained"),
                "source": "measured"}
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


def tower_parity(ex, make_inputs, math):
    """Max abs / rel difference between the executor and the CPU oracle on the bench workload itself (all 256
    boards of one batch), per output, with the tolerance the tests assert."""
    from kyanite_b200.configs import resnet_tower
    from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph
    graph, _ = resnet_tower()
    inputs = make_inputs(BATCH, 4242)
    got = [np.array(a) for a in ex.evaluate(inputs)]
    expected = cpu_eval_graph(graph.to_bytes(), BATCH, inputs)
    tol = 4e-3 if math == "tf32" else 1e-3
    out = {"config": "resnet_tower_f32_b256, all 256 boards of one batch against the CPU oracle",
           "rule": f"a value mismatches iff abs >= {tol} * max|expected| of its tensor AND rel >= {tol}", "tol": tol}
    names = ["policy", "value"]
    worst_abs = worst_rel = 0.0
    for name, e, g in zip(names, expected, got):
        max_abs, max_rel = assert_tensors_match([e], [g], tol, tol, abs_scaled=True)
        out[name] = {"max_abs": max_abs, "max_rel": max_rel, "scale": float(np.abs(e).max())}
        worst_abs, worst_rel = max(worst_abs, max_abs), max(worst_rel, max_rel)
    out["max_abs"], out["max_rel"] = worst_abs, worst_rel
    return out


def library_proxy(make_inputs, seconds=1.0):
    """The same tower through the vendor libraries, as information only: cuDNN's fused convolution + bias
    (+ residual) + ReLU in TF32, channels-last, the whole forward pass captured in a CUDA graph and replayed
    at batch 256.  That is what the reference's cudnnConvolutionBiasActivationForward
    (kn-cuda-sys/src/wrapper/operation.rs:219-239) and cublasSgemm calls would do on this GPU; torch stands
    in for the Rust bindings.  Random weights of the same shapes; inputs rotate through a pool larger
    than L2."""
    import torch
    import torch.nn.functional as F
    torch.backends.cudnn.allow_tf32 = True
    torch.backends.cuda.matmul.allow_tf32 = False     # the reference's cublasSgemm is exact f32
    dev = torch.device("cuda")
    gen = torch.Generator(device="cuda")
    gen.manual_seed(7)
    cl = torch.channels_last

    def w(co, ci, k):
        return (torch.randn((co, ci, k, k), device=dev, generator=gen) * (2.0 / (ci * k * k)) ** 0.5).contiguous(memory_format=cl)

    def b(c):
        return 0.1 * torch.randn((c,), device=dev, generator=gen)

    stem = (w(128, 21, 3), b(128))
    blocks = [((w(128, 128, 3), b(128)), (w(128, 128, 3) * (1 / 32 ** 0.5), b(128))) for _ in range(16)]
    pol, val = (w(73, 128, 1), b(73)), (w(32, 128, 1), b(32))
    w1, b1 = torch.randn((256, 2048), device=dev, generator=gen) * (2 / 2048) ** 0.5, b(256)
    w2, b2 = torch.randn((3, 256), device=dev, generator=gen) * (2 / 256) ** 0.5, b(3)
    fused = hasattr(torch, "cudnn_convolution_relu") and hasattr(torch, "cudnn_convolution_add_relu")

    def conv_relu(x, wb, pad):
        if fused:
            return torch.cudnn_convolution_relu(x, wb[0], wb[1], (1, 1), (pad, pad), (1, 1), 1)
        return F.relu(F.conv2d(x, wb[0], wb[1], padding=pad))

    def conv_add_relu(x, wb, z):
        if fused:
            return torch.cudnn_convolution_add_relu(x, wb[0], z, 1.0, wb[1], (1, 1), (1, 1), (1, 1), 1)
        return F.relu(F.conv2d(x, wb[0], wb[1], padding=1) + z)

    def trunk(x):
        cur = conv_relu(x, stem, 1)
        for c1, c2 in blocks:
            cur = conv_add_relu(conv_relu(cur, c1, 1), c2, cur)
        return cur

    def forward(x):
        cur = trunk(x)
        p = torch.softmax(F.conv2d(cur, pol[0], pol[1]).flatten(1), 1)
        v = F.conv2d(cur, val[0], val[1]).flatten(1)
        v = torch.softmax(F.linear(F.relu(F.linear(v, w1, b1)), w2, b2), 1)
        return p, v

    pool_sets = 128
    pool = (torch.rand((pool_sets, BATCH, 21, 8, 8), device=dev, generator=gen) < 0.1).float()
    x = pool[0].clone().contiguous(memory_format=cl)
    result = {"what": "torch " + torch.__version__ + ": cuDNN " + str(torch.backends.cudnn.version()) +
                      (" fused conv+bias(+residual)+relu" if fused else " conv2d + relu") +
                      ", TF32, channels-last, CUDA graph, batch 256, f32 linears"}
    side = torch.cuda.Stream()
    with torch.cuda.stream(side), torch.no_grad():
        for _ in range(3):
            forward(x)
        side.synchronize()
        g_full, g_trunk = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_full, stream=side):
            forward(x)
        with torch.cuda.graph(g_trunk, stream=side):
            trunk(x)
        for name, graph in (("whole_step", g_full), ("trunk_33_convs", g_trunk)):
            for i in range(5):
                x.copy_(pool[i % pool_sets])
                graph.replay()
            side.synchronize()
            t0 = time.perf_counter()
            n, ms_total = 0, 0.0
            while time.perf_counter() - t0 < seconds:
                a, c = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(side)
                for i in range(50):
                    x.copy_(pool[(n + i) % pool_sets])
                    graph.replay()
                c.record(side)
                c.synchronize()
                ms_total += a.elapsed_time(c)
                n += 50
            result[name] = {"ms_per_step": ms_total / n, "inferences_per_s": BATCH * n / (ms_total / 1000.0)}
    return result


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--math", default="tf32", choices=["tf32", "f32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-library-proxy", action="store_true")
    ap.add_argument("--no-chain", action="store_true", help="one launch per convolution instead of the merged chain kernel (A/B)")
    ap.add_argument("--e2e-executors", type=int, default=2, help="executors per GPU in the pipelined measurements")
    ap.add_argument("--no-bind", action="store_true", help="leave the process's CPU affinity alone (A/B)")
    ap.add_argument("--min-seconds", type=float, default=1.5,
                    help="each pipelined leg repeats its window of --steps steps until this much time is covered")
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
    from kyanite_b200.executor import FLAG_NO_CONV_CHAIN, MATH_F32, MATH_TF32, CudaExecutor
    from kyanite_b200.sharding import bind_process_near_gpu

    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    # one process per GPU: keep this rank's host buffers and the threads that fill them next to its GPU
    affinity = bind_process_near_gpu("GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid)) if not args.no_bind else \
        {"bound": False, "why": "--no-bind"}

    graph, make_inputs = resnet_tower()
    math_mode = MATH_TF32 if args.math == "tf32" else MATH_F32
    flags = FLAG_NO_CONV_CHAIN if args.no_chain else 0
    ex = CudaExecutor(local_rank, graph, BATCH, math_mode=math_mode, flags=flags)
    inputs = make_inputs(BATCH, 1 + rank)
    for dst, src in zip(ex.host_inputs, inputs):
        dst[...] = src
    steps_per_run, launches_per_run = ex.step_count()
    K = args.steps

    stream = torch.cuda.ExternalStream(ex.stream(), device=torch.device("cuda", local_rank))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")   # 2x the 126 MB L2

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def time_dominant():
        """[(us per launch, flop, kind, description)] of the contraction step(s) with the most FLOP: 20 launches back
        to back between one pair of CUDA events on the executor's stream."""
        nonlocal launches
        ex.set_profile(True)
        ex.run_async()
        launches += launches_per_run
        contractions = []
        for line in ex.last_profile().splitlines():
            parts = line.split()
            if len(parts) > 6 and parts[0].isdigit() and parts[1].split("/")[0] in ("Conv", "ConvChain", "Gemm"):
                contractions.append((int(parts[0]), float(parts[4]), parts[1], " ".join(parts[5:])))
        ex.set_profile(False)
        if not contractions:
            return []
        top = max(c[1] for c in contractions)
        launches += 21 * sum(1 for c in contractions if c[1] == top)
        return [(ex.time_step(idx, 20), flop, kind, desc) for idx, flop, kind, desc in contractions if flop == top]

    # clocks: one sampler (rank 0's GPU), every 50 ms, so that N ranks do not add N polling threads to the host
    sampler = None
    if rank == 0:
        sampler = ClockSampler(local_rank, "GPU-" + str(torch.cuda.get_device_properties(local_rank).uuid))
        sampler.start()

    # ---- warm-up (also captures the CUDA graph)
    for _ in range(args.warmup):
        ex.evaluate_staged()
    ex.synchronize()

    launches = args.warmup * launches_per_run
    # the dominant kernel before the GPU has been under load for seconds (burst clocks); timed again at the end
    dominant_before_load = time_dominant()

    # ---- one executor, one step after the other, L2 flushed before every timed step (`config.one_executor_flushed`)
    barrier()
    if sampler:
        sampler.mark_start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    with torch.cuda.stream(stream):
        for i in range(K):
            flush.zero_()
            starts[i].record(stream)
            ex.run_async()
            ends[i].record(stream)
            launches += launches_per_run
    barrier()
    dev_ms = sum(s.elapsed_time(e) for s, e in zip(starts, ends))

    # ---- `e2e.one_executor_serial`: plain evaluate() calls in series with caller-owned input arrays
    h2d = sum(a.nbytes for a in ex.host_inputs)
    d2h = sum(a.nbytes for a in ex.host_outputs)
    host_sets = 16            # caller-owned (pageable) input arrays the calls rotate through
    host_pool = [[np.ascontiguousarray(a) for a in make_inputs(BATCH, 5000 + 31 * j + rank)] for j in range(host_sets)]
    barrier()
    e2e_start = torch.cuda.Event(enable_timing=True)
    e2e_end = torch.cuda.Event(enable_timing=True)
    e2e_start.record(stream)
    for i in range(K):
        ex.evaluate_begin(host_pool[i % host_sets])
        ex.evaluate_end()
        launches += launches_per_run
    e2e_end.record(stream)
    barrier()
    serial_ms = e2e_start.elapsed_time(e2e_end)

    # ---- the pipelined legs: several executors of the same graph on this GPU, the way the reference's hosts keep
    # a GPU busy (several executor threads per device).  Each leg first fills the pipeline with untimed steps,
    # then times windows of K steps back to back WITHOUT draining in between (a CUDA event behind the last step
    # of every window, on the stream that step runs on), until --min-seconds are covered; the median window is
    # reported, with the spread.
    pair = []
    for k in range(args.e2e_executors):
        e = CudaExecutor(local_rank, graph, BATCH, math_mode=math_mode, flags=flags)
        for dst, src in zip(e.host_inputs, make_inputs(BATCH, 1001 + 17 * k + rank)):
            dst[...] = src
        pair.append(e)
    streams = [torch.cuda.ExternalStream(e.stream(), device=torch.device("cuda", local_rank)) for e in pair]
    n_ex = len(pair)
    for e in pair:
        for _ in range(max(2, args.warmup)):
            e.evaluate_staged()
            launches += launches_per_run

    def run_windows(submit, finish, est_ms_per_step):
        """`submit(i)` enqueues step i on executor i % n_ex, `finish(i)` waits for it (or None).  Returns the list
        of window durations in ms and the host time spent inside submit per step (us)."""
        nonlocal launches
        windows = max(3, int(np.ceil(args.min_seconds * 1000.0 / max(1e-3, est_ms_per_step * K))))
        total = windows * K
        lead = n_ex - 1 if finish else 0
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(windows + 1)]
        fill = 2 * n_ex + lead                      # untimed steps that fill the pipeline
        host_s = 0.0
        for i in range(fill):
            submit(i)
            if finish and i >= lead:
                finish(i - lead)
        marks[0].record(streams[(fill - 1) % n_ex])   # behind the newest submitted step
        for j in range(total):
            i = fill + j
            t0 = time.perf_counter()
            submit(i)
            host_s += time.perf_counter() - t0
            if (j + 1) % K == 0:
                marks[(j + 1) // K].record(streams[i % n_ex])
            if finish:
                finish(i - lead)
        if finish:
            for i in range(fill + total - lead, fill + total):
                finish(i)
        launches += (fill + total) * launches_per_run
        barrier()
        return [a.elapsed_time(b) for a, b in zip(marks[:-1], marks[1:])], 1e6 * host_s / total

    # (a) `e2e`: every batch copied from a caller-owned array to pinned staging, uploaded, computed and downloaded
    # inside the timed region; the next batch is submitted before the current one is waited for.
    barrier()
    e2e_windows, e2e_host_us = run_windows(lambda i: pair[i % n_ex].evaluate_begin(host_pool[i % host_sets]),
                                           lambda i: pair[i % n_ex].evaluate_end(), serial_ms / K / 1.5)

    # (b) the copy-only ceiling of (a): the same host -> pinned, pinned -> device and device -> pinned bytes per
    # step on the same streams, no kernels
    def copy_submit(i):
        e = pair[i % n_ex]
        e.synchronize()
        for dst, src in zip(e.host_inputs, host_pool[i % host_sets]):
            np.copyto(dst, src)
        e.upload_inputs()
        e.download_outputs()

    barrier()
    saved = launches
    copy_windows, _ = run_windows(copy_submit, None, statistics.median(e2e_windows) / K / 2)
    launches = saved                                  # no kernel launches in that leg

    # (c) `value`: batches already in HBM.  No flush here: a pool of input sets larger than the 126 MB L2
    # rotates through the executors' input buffers (one device-to-device copy per step, inside the timed
    # region), so no step finds its input in L2, while the 20 MB of weights stay there as they do in
    # steady-state serving.  With two executors alternating, CTAs of the next batch fill the SMs the current
    # one leaves idle (128 CTAs for 148 SMs).
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

    def value_submit(i):
        k = i % n_ex
        with torch.cuda.stream(streams[k]):
            for pool, dst in zip(pools, dev_in[k]):
                dst.copy_(pool[i % pool_sets], non_blocking=True)
        pair[k].run_async()

    barrier()
    pipe_windows, pipe_host_us = run_windows(value_submit, None, statistics.median(e2e_windows) / K)
    clocks = sampler.stop() if sampler else None
    for e in pair:
        e.close()

    # ---- dominant kernel: the contraction step with the most FLOP (the convolution chain that runs the
    # whole residual tower in one launch; with chains switched off, the trunk convolutions, which are
    # timed one by one and averaged).  Each is launched 20x back to back between one pair of CUDA events
    # on the executor's stream.
    dominant = time_dominant()

    pipe_ms, e2e_ms, copy_ms = (statistics.median(w) for w in (pipe_windows, e2e_windows, copy_windows))
    mine = torch.tensor([dev_ms, e2e_ms, serial_ms, pipe_ms, copy_ms, pipe_host_us, e2e_host_us], dtype=torch.float64,
                        device="cuda")
    if world > 1:
        gathered = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine)
        per_rank = torch.stack(gathered).cpu().numpy()
        affinities = [None] * world
        dist.all_gather_object(affinities, affinity)
    else:
        per_rank = mine.cpu().numpy()[None]
        affinities = [affinity]
    dev_ms, e2e_ms, serial_ms, pipe_ms, copy_ms = (float(per_rank[:, c].max()) for c in range(5))   # MAX over ranks

    if rank == 0:
        peaks = load_peaks()
        total = BATCH * world * K
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
                        "gflop_per_launch": flop / 1e9, "launches_per_step": len(dominant),
                        "when": "20 launches back to back after the timed legs, the GPU under its power cap for seconds; "
                                "`achieved` and `frac` are this figure against the BURST peak"}
            if peaks.get("bf16_tflops_sustained"):
                sustained = peaks["bf16_tflops_sustained"] / 2.0
                roofline["against_sustained_peak"] = {"peak": sustained, "frac": achieved / sustained}
            if dominant_before_load:
                us0 = statistics.mean(u for u, _, _, _ in dominant_before_load)
                roofline["before_load"] = {"us_per_launch": us0, "achieved": flop / (us0 * 1e-6) / 1e12,
                                           "frac": flop / (us0 * 1e-6) / 1e12 / tensor_peak,
                                           "what": "the same 20 launches right after warm-up, at burst clocks, against the burst peak"}

        def spread(windows):
            return {"windows": len(windows), "min_ms_per_step": min(windows) / K, "median_ms_per_step": statistics.median(windows) / K,
                    "max_ms_per_step": max(windows) / K}

        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": args.warmup,
            "ms_per_step": pipe_ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "tf32 operands, f32 storage and accumulate" if args.math == "tf32" else "f32",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "batch_per_gpu": BATCH, "parallelism": f"batch-sharded x{world}, no collective",
                       "cpu_affinity_per_rank": affinities,
                       "executors_per_gpu": args.e2e_executors,
                       "timing": f"steady state: the pipeline is filled with untimed steps, then windows of {K} steps are "
                                 "timed back to back with CUDA events (no drain in between) for at least "
                                 f"{args.min_seconds} s; value and e2e are the MEDIAN window, max over ranks; "
                                 "ms_per_step x steps = one window",
                       "value_windows_rank0": spread(pipe_windows), "host_enqueue_us_per_step": float(per_rank[:, 5].max()),
                       "per_rank_ms_per_step": [float(x) / K for x in per_rank[:, 3]],
                       "l2": f"no flush: {pool_sets} input sets ({pool_bytes / 1e6:.0f} MB, larger than the 126 MB L2) rotate "
                             "through the executors' input buffers, one device-to-device copy per step inside the timed "
                             "region; weights (20 MB) stay in L2",
                       "one_executor_flushed": {"value": total / (dev_ms / 1000.0), "ms_per_step": dev_ms / K,
                                                "l2": "one executor, steps one after the other, 256 MiB L2 flush "
                                                      "between timed iterations"},
                       "gflop_per_step": resnet_tower_flops(BATCH) / 1e9, "steps_per_run": steps_per_run},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / K, "executors_per_gpu": args.e2e_executors,
                    "windows_rank0": spread(e2e_windows), "host_enqueue_us_per_step": float(per_rank[:, 6].max()),
                    "per_rank_ms_per_step": [float(x) / K for x in per_rank[:, 1]],
                    "mode": "kn_executor_evaluate_begin(inputs) / _end on several executors per GPU, the next batch "
                            "submitted before the current one is waited for; inputs are caller-owned pageable arrays "
                            f"({host_sets} sets in rotation): the library copies them to pinned staging, uploads, runs "
                            "the steps and downloads every output to pinned host memory, all inside the timed region",
                    "copy_only": {"value": total / (copy_ms / 1000.0), "ms_per_step": copy_ms / K,
                                  "per_rank_ms_per_step": [float(x) / K for x in per_rank[:, 4]],
                                  "what": "the same host->pinned, pinned->device and device->pinned bytes per step on "
                                          "the same streams with no kernels: the ceiling the copies alone set at this "
                                          "number of GPUs"},
                    "one_executor_serial": {"value": total / (serial_ms / 1000.0), "ms_per_step": serial_ms / K}},
            "gpu_launches": launches,
            "clocks": clocks,
            "roofline": roofline,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["parity"] = tower_parity(ex, make_inputs, args.math)
            launches += launches_per_run
            line["gpu_launches"] = launches
            rate, dt = cpu_oracle_rate(BATCH, 4)
            line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": f"4 x {BATCH} boards through the numpy oracle in {dt:.1f} s"}
            try:
                from threadpoolctl import threadpool_limits
                with threadpool_limits(limits=1):
                    rate1, dt1 = cpu_oracle_rate(32, 1)
                line["cpu_baseline"]["one_thread"] = {"value": rate1, "cores": 1,
                                                      "sample": f"32 boards with the BLAS pool limited to one thread in {dt1:.1f} s "
                                                                "(the reference's CPU executor is single-threaded)"}
            except ImportError:
                pass
        if world == 1 and not args.no_library_proxy:
            ex.close()
            try:
                line["config"]["library_proxy"] = library_proxy(make_inputs)
            except Exception as e:   # information only: never fails the bench
                line["config"]["library_proxy"] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        print(json.dumps(line), flush=True)

    ex.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
