"""Batch sharding across devices: the executor's only multi-GPU mode.

Every per-sample tensor of a graph carries the batch size in its shape (`Size(factor, exp)` with
exp > 0), samples never interact in the operations the executor runs, and the reference has no
collective at all (it can only run one executor per device).  So a global batch is split on the host
along each input's batch axis, every rank evaluates its shard with its own executor, and outputs are
concatenated along their batch axis.  Inputs without a batch axis are replicated.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np

from .graph import Graph


def batch_axis(shape) -> Optional[int]:
    """Index of the (single) axis proportional to the batch size, or None."""
    axes = [i for i, d in enumerate(shape) if d.exp > 0]
    if not axes:
        return None
    if len(axes) > 1 or shape[axes[0]].exp != 1:
        raise ValueError(f"shape {shape} is not linear in the batch size along one axis; cannot shard it")
    return axes[0]


def check_shardable(graph: Graph) -> None:
    """Raises ValueError if some operation of `graph` combines different batch entries, so that evaluating
    shards of the batch separately would give other numbers than evaluating the whole batch: a reduction,
    softmax or layernorm along an axis whose size depends on the batch size, a matrix product that contracts
    over one, a convolution with the batch size in its channels or image, a gather, slice, flip or concat
    along one, or an all-reduce (that graph belongs to a tensor-parallel run, not a batch-sharded one)."""
    from .graph import OpKind

    def batchy(shape, axis) -> bool:
        return shape[axis].exp > 0

    for index, info in enumerate(graph.values):
        k = info.kind
        ins = [graph.values[i] for i in info.inputs]
        reason = None
        if k == OpKind.REDUCE and any(batchy(ins[0].shape, a) for a in info.axes):
            reason = "reduces over a batch-sized axis"
        elif k in (OpKind.SOFTMAX, OpKind.LAYERNORM) and batchy(ins[0].shape, info.axis):
            reason = "normalises along a batch-sized axis"
        elif k == OpKind.MATMUL and (batchy(ins[0].shape, 2) or batchy(ins[1].shape, 1)):
            reason = "contracts over a batch-sized axis"
        elif k == OpKind.CONV and (any(batchy(ins[0].shape, a) for a in (1, 2, 3)) or any(d.exp > 0 for d in ins[1].shape)):
            reason = "convolves over a batch-sized axis"
        elif k == OpKind.GATHER and batchy(ins[0].shape, info.axis):
            reason = "gathers along a batch-sized axis"
        elif k in (OpKind.SLICE, OpKind.FLIP) and batchy(ins[0].shape, info.axis):
            reason = "slices or flips a batch-sized axis"
        elif k == OpKind.CONCAT and batchy(info.shape, info.axis):
            reason = "concatenates along a batch-sized axis"
        elif k == OpKind.ALL_REDUCE:
            reason = "is an all-reduce"
        if reason:
            raise ValueError(f"graph cannot be sharded by batch: value {index} ({k.name}) {reason}")
    for v in list(graph.inputs) + list(graph.outputs):
        batch_axis(graph[v].shape)


def shard_sizes(global_batch: int, world: int) -> List[int]:
    """Per-rank batch sizes: as even as possible, earlier ranks take the remainder."""
    base, rem = divmod(global_batch, world)
    return [base + (1 if r < rem else 0) for r in range(world)]


def split_inputs(graph: Graph, inputs: Sequence[np.ndarray], global_batch: int, rank: int, world: int) -> List[np.ndarray]:
    check_shardable(graph)
    sizes = shard_sizes(global_batch, world)
    start = sum(sizes[:rank])
    out = []
    for v, x in zip(graph.inputs, inputs):
        shape = graph[v].shape
        axis = batch_axis(shape)
        if axis is None:
            out.append(x)
            continue
        f = shape[axis].factor
        sl = [slice(None)] * x.ndim
        sl[axis] = slice(start * f, (start + sizes[rank]) * f)
        out.append(np.ascontiguousarray(x[tuple(sl)]))
    return out


def merge_outputs(graph: Graph, per_rank_outputs: Sequence[Sequence[np.ndarray]]) -> List[np.ndarray]:
    merged = []
    for i, v in enumerate(graph.outputs):
        axis = batch_axis(graph[v].shape)
        parts = [outs[i] for outs in per_rank_outputs]
        if axis is None:
            for p in parts[1:]:
                if not np.array_equal(p, parts[0], equal_nan=True):
                    raise ValueError(f"output {i} has no batch axis but differs between ranks")
            merged.append(parts[0])
        else:
            merged.append(np.concatenate(parts, axis=axis))
    return merged


def cpus_from_affinity_words(words: Sequence[int], bits: int = 64) -> List[int]:
    """CPU numbers of an affinity bit mask given as machine words, least significant word first (the form NVML
    returns a device's ideal CPU affinity in)."""
    return [w * bits + b for w, word in enumerate(words) for b in range(bits) if (int(word) >> b) & 1]


def bind_process_near_gpu(gpu_uuid: str, allowed: Optional[Sequence[int]] = None, nvml=None) -> dict:
    """Restricts the calling process to the CPUs the driver names as closest to the GPU (its NUMA node), so that the
    rank's host buffers (first touch) and the threads that fill them are local to the GPU's PCIe root.  With one
    process per GPU and the per-step staging copies of `evaluate`, ranks whose process ran on the far socket took
    twice as long for the same copies.  Changes nothing but this process's own CPU affinity; does nothing (and says
    so) when NVML is missing, when the ideal set and the CPUs this process may use do not overlap, or when the
    process is already inside the ideal set.  `nvml`: the pynvml module or a stand-in (tests)."""
    import os
    if allowed is None:
        allowed = sorted(os.sched_getaffinity(0))
    try:
        if nvml is None:
            import pynvml as nvml
            nvml.nvmlInit()
        handle = nvml.nvmlDeviceGetHandleByUUID(gpu_uuid.encode())
        words = nvml.nvmlDeviceGetCpuAffinity(handle, (max(allowed) // 64 + 1) if allowed else 1)
    except Exception as e:   # no NVML, or the query is not supported here
        return {"bound": False, "why": f"no ideal affinity from NVML ({type(e).__name__})", "cpus": len(allowed)}
    ideal = set(cpus_from_affinity_words(words))
    target = sorted(ideal.intersection(allowed))
    if not target:
        return {"bound": False, "why": "the GPU's ideal CPUs are outside this process's CPU set", "cpus": len(allowed)}
    if len(target) == len(allowed):
        return {"bound": False, "why": "already inside the GPU's ideal CPU set", "cpus": len(allowed)}
    os.sched_setaffinity(0, target)
    return {"bound": True, "cpus": len(target), "of": len(allowed)}


def aggregate_throughput(units_per_rank: Sequence[int], ms_per_rank: Sequence[float]) -> float:
    """Whole-job units per second: all units over the slowest rank's time."""
    return sum(units_per_rank) / (max(ms_per_rank) / 1000.0)
