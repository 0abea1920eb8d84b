"""Throughput and per-step profile of an ONNX model on the CUDA executor: the reference's `profile_net`
tool (kn-cuda-eval/src/bin/profile_net.rs) with the same flags and the same timing method.

    python -m kyanite_b200.profile_net model.onnx --optimize --batch-size 256 [-n 100] [--skip-io]
    python -m kyanite_b200.profile_net model.onnx --optimize            # sweep over batch sizes 1..2048
    python -m kyanite_b200.profile_net model.onnx --print --batch-size 8

Timing (profile_net.rs:146-180): max(1, n/10) warm-up calls, then n calls of `evaluate` (with host<->device
copies) or, with --skip-io, of `run_async` followed by one synchronise; throughput = batch_size * n / wall
time.  Inputs are zeros of the graph's input shapes (`Graph::dummy_zero_inputs`).  `--math f32` selects
exact-f32 contractions instead of the default TF32 tensor-core path.
"""
from __future__ import annotations

import argparse
import os
import sys
import time
from typing import List

import numpy as np

from . import graph as ir
from .executor import MATH_F32, MATH_TF32, CudaDevice, CudaExecutor, plan_describe
from .onnx import load_graph_from_onnx_path
from .optimizer import optimize_graph

TEST_BATCH_SIZES = [1, 2, 3, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048]
TEST_BATCH_ITERATIONS = [100, 100, 100, 100, 100, 100, 100, 100, 50, 25, 12, 8, 4]
DEFAULT_ITERATIONS = 100


def dummy_zero_inputs(graph: ir.Graph, batch_size: int) -> List[np.ndarray]:
    return [np.zeros(tuple(d.eval(batch_size) for d in graph[v].shape), dtype=graph[v].dtype.np) for v in graph.inputs]


def profile_single(device: CudaDevice, graph: ir.Graph, batch_size: int, n: int, skip_io: bool, math_mode: int,
                   out=sys.stdout) -> float:
    with CudaExecutor(device, graph, batch_size, math_mode=math_mode) as ex:
        inputs = dummy_zero_inputs(graph, batch_size)
        print("Warmup", file=out)
        for _ in range(max(1, n // 10)):
            ex.evaluate(inputs)
        print("Throughput test", file=out)
        start = time.perf_counter()
        for _ in range(n):
            if skip_io:
                ex.run_async()
            else:
                ex.evaluate(inputs)
        if skip_io:
            ex.synchronize()
        throughput = batch_size * n / (time.perf_counter() - start)
        print("Profiling", file=out)
        ex.set_profile(True)
        ex.evaluate(inputs)
        print(ex.last_profile(), file=out)
    print(f"Throughput: {throughput} evals/s", file=out)
    return throughput


def profile_batch_sizes(device: CudaDevice, graph: ir.Graph, math_mode: int, out=sys.stdout):
    result = []
    for batch_size, iterations in zip(TEST_BATCH_SIZES, TEST_BATCH_ITERATIONS):
        print(f"Testing batch size {batch_size} with {iterations} iterations", file=out)
        with CudaExecutor(device, graph, batch_size, math_mode=math_mode) as ex:
            inputs = dummy_zero_inputs(graph, batch_size)
            for _ in range(max(1, iterations // 10)):
                ex.evaluate(inputs)
            start = time.perf_counter()
            for _ in range(iterations):
                ex.evaluate(inputs)
            throughput = batch_size * iterations / (time.perf_counter() - start)
        print(f"  throughput: {throughput} evals/s", file=out)
        result.append((batch_size, throughput))
    print(result, file=out)
    return result


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="profile_net", description=__doc__.splitlines()[0])
    ap.add_argument("path")
    ap.add_argument("-b", "--batch-size", type=int, default=0)
    ap.add_argument("-o", "--optimize", action="store_true")
    ap.add_argument("-p", "--print", dest="print_graph", action="store_true")
    ap.add_argument("-c", "--cpu", action="store_true")
    ap.add_argument("-d", "--device", type=int, default=None)
    ap.add_argument("-s", "--skip-io", action="store_true")
    ap.add_argument("-n", type=int, default=None)
    ap.add_argument("--math", choices=["tf32", "f32"], default="tf32")
    args = ap.parse_args(argv)

    warnings = []

    def warn(message: str):
        warnings.append(message)
        print(message, file=sys.stderr)

    if args.cpu:
        print("Error: this library has no CPU executor", file=sys.stderr)
        return 2
    n = args.n if args.n is not None else DEFAULT_ITERATIONS
    math_mode = MATH_TF32 if args.math == "tf32" else MATH_F32

    path = os.path.abspath(args.path)
    print(f"Loading graph '{path}'")
    loaded = load_graph_from_onnx_path(path, allow_external=True)
    shapes = [loaded[v].shape for v in loaded.inputs]
    if any(sum(1 for d in s if d == ir.BATCH) != 1 for s in shapes):
        warn("Warning: graph has inputs without exactly one batch dimension. This messes up the evals/s stats.")
        warn(f"    input shapes: {shapes}")
    if args.optimize:
        print("Optimizing graph")
        graph = optimize_graph(loaded)
    else:
        warn("Warning: not optimizing graph")
        graph = loaded

    if args.print_graph:
        print(graph.dump())
        if args.batch_size <= 0:
            print("Error: must set batch size", file=sys.stderr)
            return 2
        print(plan_describe(graph, args.batch_size, math_mode))      # needs no GPU
    else:
        device = CudaDevice(args.device if args.device is not None else 0)
        if args.batch_size < 1:
            profile_batch_sizes(device, graph, math_mode)
        else:
            profile_single(device, graph, args.batch_size, n, args.skip_io, math_mode)
    for w in warnings:
        print(w, file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
