"""The reference's Python module (`kyanite`, kn-python/src/lib.rs:14-78) on top of this library: the same
two classes with the same methods, so scripts written against it run unchanged.

    graph = Graph.from_bytes(onnx_bytes).optimize()
    batch = graph.infer_batch_size(inputs)
    prepared = graph.prepare("cuda:0", batch)
    outputs = prepared.eval(inputs)

Device strings follow kn-python/src/lib.rs:139-164: "best", "cuda", "cuda:<index>" and "cpu".  This library
has no CPU executor, so "cpu" is refused and "best" means the first CUDA device.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from . import graph as ir
from .executor import CudaDevice, CudaDeviceNotAvailable, Device, PreparedGraph
from .onnx import OnnxError, load_graph_from_onnx_bytes
from .optimizer import optimize_graph

__all__ = ["Graph", "Prepared", "infer_batch_size"]


def infer_batch_size(expected: Sequence[ir.Shape], actual: Sequence[Sequence[int]]) -> Optional[int]:
    """The batch size that makes every symbolic shape equal to the concrete one, None if any would do
    (no dimension mentions it); ValueError if none fits (kn-graph/src/shape.rs:352-419)."""
    exp_dims = [d for s in expected for d in s]
    act_dims = [int(d) for s in actual for d in s]
    if len(exp_dims) != len(act_dims):
        raise ValueError("Could not infer batch size: DifferentLength")
    batch = None
    for e, a in zip(exp_dims, act_dims):
        if e.exp == 0:
            if a != e.factor:
                raise ValueError("Could not infer batch size: ConstantMismatch")
        elif batch is not None:
            if a != e.eval(batch):
                raise ValueError("Could not infer batch size: BatchConflict")
        else:
            approx = int((a / e.factor) ** (1.0 / e.exp))
            for delta in (0, 1, -1, 2, -2):
                cand = approx + delta
                if cand >= 0 and e.factor * cand ** e.exp == a:
                    batch = cand
                    break
            else:
                raise ValueError("Could not infer batch size: ImpossibleBatchValue")
    return batch


def parse_device(device: str) -> Device:
    name = device.lower()
    if name == "cpu":
        raise RuntimeError("this library has no CPU executor; use 'cuda' or 'cuda:<index>'")
    if name in ("best", "cuda"):
        if CudaDevice.device_count() == 0:
            raise RuntimeError("No CUDA device found")
        return Device.cuda(0)
    head, sep, index = name.partition(":")
    if head == "cuda" and sep and index.isdigit():
        try:
            return Device.cuda(int(index))
        except CudaDeviceNotAvailable as e:
            raise RuntimeError("Invalid CUDA device index") from e
    raise TypeError(f"Invalid device string: '{device}'")


class Graph:
    def __init__(self, inner: ir.Graph):
        self.inner = inner

    @staticmethod
    def from_bytes(data: bytes) -> "Graph":
        try:
            return Graph(load_graph_from_onnx_bytes(data))
        except OnnxError as e:
            raise RuntimeError(str(e)) from e

    def optimize(self) -> "Graph":
        return Graph(optimize_graph(self.inner))

    def infer_batch_size(self, inputs: Sequence[np.ndarray]) -> Optional[int]:
        try:
            return infer_batch_size(self.inner.input_shapes(), [np.shape(a) for a in inputs])
        except ValueError as e:
            raise RuntimeError(str(e)) from e

    def prepare(self, device: str, batch_size: int) -> "Prepared":
        return Prepared(parse_device(device).prepare(self.inner, batch_size))

    def __str__(self):
        return self.inner.dump()


class Prepared:
    def __init__(self, inner: PreparedGraph):
        self.inner = inner

    def eval(self, inputs: Sequence[np.ndarray]) -> List[np.ndarray]:
        for a in inputs:
            if np.asarray(a).dtype not in ir._OF_NP:
                raise TypeError(f"Unsupported dtype {np.asarray(a).dtype} for input tensor")
        return self.inner.eval([np.asarray(a) for a in inputs])
