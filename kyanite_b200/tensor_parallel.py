"""Tensor-parallel execution of the LLaMA-shaped decoder: one process per GPU, NCCL all-reduce after the
row-parallel projections.  This has no counterpart in the reference (which runs one graph on one device).
Every rank runs ONE graph (`llama_rank_graph`) through one `CudaExecutor`; the all-reduce after each
attention block and each feed-forward block is a value of that graph (`Graph.all_reduce`), which the executor
runs as a step of its step list: the arena buffer goes to ncclAllReduce on the executor's stream, between the
kernels before and after it, with nothing crossing host memory.  Only the final all-gather of the logits
(once per prefill, each rank holds a vocabulary slice) is done by the host.

Partitioning (world size W, rank r):
* attention: heads `[r*H/W, (r+1)*H/W)`.  W_q, W_k, W_v are split by output rows (column-parallel), RoPE,
  scores, softmax and the context product are local per head, W_o is split by input columns
  (row-parallel), so each rank produces a partial `[B, seq, d_model]` sum;
* feed-forward: hidden units `[r*F/W, (r+1)*F/W)`: gate and up column-parallel, down row-parallel, again a
  partial sum;
* RMSNorm, the residual stream, the embedding table and the final norm are replicated;
* lm head: vocabulary rows `[r*V/W, (r+1)*V/W)`, logits all-gathered along the vocabulary axis.

`llama_segments` is the same partition cut into `2 * layers + 1` separate graphs at the all-reduce points, so
that the slices of several ranks can be checked on ONE device (the tests play the collective on the host
between segments); it is not the execution path.  Segment k takes the
residual stream `x` and the reduced sum `s` of the previous block, forms `x + s` (replicated arithmetic,
bit-identical on every rank) and returns it together with this rank's partial sum of the next block:

    ids      -> seg[0]   -> x0,   p0 (attention 0)        s0 = all_reduce(p0)
    x0, s0   -> seg[1]   -> x1,   p1 (feed-forward 0)      s1 = all_reduce(p1)
    ...
    x, s     -> seg[2L]  -> logits[:, :, vocab slice]      logits = all_gather(...)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import numpy as np

from .configs import LlamaBlocks, llama_weights
from .graph import BATCH, DType, Graph, shape

__all__ = ["LlamaShape", "llama_rank_graph", "llama_segments", "TorchComm", "LocalComm", "TensorParallelLlama",
           "cuda_prepare"]


@dataclass(frozen=True)
class LlamaShape:
    layers: int = 32
    d_model: int = 4096
    heads: int = 32
    ffn: int = 11008
    vocab: int = 32000
    seq: int = 2048
    eps: float = 1e-6
    rope_base: float = 10000.0
    seed: int = 10


def _even_slice(total: int, rank: int, world: int, what: str) -> slice:
    if total % world != 0:
        raise ValueError(f"{what} ({total}) is not divisible by the tensor-parallel size {world}")
    step = total // world
    return slice(rank * step, (rank + 1) * step)


def llama_rank_graph(cfg: LlamaShape, rank: int, world: int, draw_slices_only: bool = False, dtype="f32") -> Graph:
    """The one graph rank `rank` of `world` runs: token ids [B, seq] -> this rank's vocabulary slice of the
    logits [B, seq, vocab / world], with an all-reduce value after every row-parallel projection
    (2 * layers of them, each [B, seq, d_model]).  `draw_slices_only`: see `llama_weights` (timing runs).
    `dtype`: "f32", or "f16" for half storage (weights, activations, all-reduce buffers and logits f16)."""
    dt = DType.F16 if str(dtype).lower() in ("f16", "dtype.f16") or dtype == DType.F16 else DType.F32
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of size {world}")
    head_slice = _even_slice(cfg.heads, rank, world, "head count")
    ffn_slice = _even_slice(cfg.ffn, rank, world, "feed-forward width")
    vocab_slice = _even_slice(cfg.vocab, rank, world, "vocabulary")
    w = llama_weights(cfg.layers, cfg.d_model, cfg.heads, cfg.ffn, cfg.vocab, cfg.seed, head_slice=head_slice,
                      ffn_slice=ffn_slice, vocab_slice=vocab_slice, draw_slices_only=draw_slices_only)
    local_heads = head_slice.stop - head_slice.start
    g = Graph()
    blocks = LlamaBlocks(g, cfg.d_model, cfg.d_model // cfg.heads, cfg.seq, cfg.eps, cfg.rope_base, dt)
    ids = g.input(shape(BATCH, cfg.seq), DType.I32)
    x = g.view(g.gather(g.constant_tensor(w["table"].astype(dt.np)), 0, g.flatten(ids, 0)), shape(BATCH, cfg.seq, cfg.d_model))
    for layer in w["layers"]:
        x = g.add(x, g.all_reduce(blocks.attention_partial(x, layer, head_slice, local_heads)))
        x = g.add(x, g.all_reduce(blocks.ffn_partial(x, layer, ffn_slice)))
    g.output(blocks.logits(x, w["norm_f"], w["lm_head"]))
    return g


def llama_segments(cfg: LlamaShape, rank: int, world: int) -> List[Graph]:
    """The graphs rank `rank` of `world` runs, in order (see the module docstring)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of size {world}")
    w = llama_weights(cfg.layers, cfg.d_model, cfg.heads, cfg.ffn, cfg.vocab, cfg.seed)
    head_slice = _even_slice(cfg.heads, rank, world, "head count")
    ffn_slice = _even_slice(cfg.ffn, rank, world, "feed-forward width")
    vocab_slice = _even_slice(cfg.vocab, rank, world, "vocabulary")
    local_heads = head_slice.stop - head_slice.start
    hd = cfg.d_model // cfg.heads
    stream = shape(BATCH, cfg.seq, cfg.d_model)

    def begin():
        g = Graph()
        return g, LlamaBlocks(g, cfg.d_model, hd, cfg.seq, cfg.eps, cfg.rope_base)

    segments: List[Graph] = []
    # segment 0: embedding, attention of layer 0
    g, blocks = begin()
    ids = g.input(shape(BATCH, cfg.seq), DType.I32)
    x = g.view(g.gather(g.constant_tensor(w["table"]), 0, g.flatten(ids, 0)), stream)
    g.output(x)
    g.output(blocks.attention_partial(x, w["layers"][0], head_slice, local_heads))
    segments.append(g)
    for li, layer in enumerate(w["layers"]):
        # feed-forward of layer li
        g, blocks = begin()
        x = g.add(g.input(stream), g.input(stream))
        g.output(x)
        g.output(blocks.ffn_partial(x, layer, ffn_slice))
        segments.append(g)
        if li + 1 < cfg.layers:
            # attention of layer li + 1
            g, blocks = begin()
            x = g.add(g.input(stream), g.input(stream))
            g.output(x)
            g.output(blocks.attention_partial(x, w["layers"][li + 1], head_slice, local_heads))
            segments.append(g)
    # last segment: final norm and this rank's slice of the lm head
    g, blocks = begin()
    x = g.add(g.input(stream), g.input(stream))
    g.output(blocks.logits(x, w["norm_f"], w["lm_head"][vocab_slice]))
    segments.append(g)
    return segments


class LocalComm:
    """World of size 1: the collectives are identities."""
    rank, world = 0, 1
    device_comm = None

    def all_reduce_sum(self, a: np.ndarray) -> np.ndarray:
        return a

    def all_gather_last_axis(self, a: np.ndarray) -> np.ndarray:
        return a


class TorchComm:
    """The host side of a rank, over an initialised `torch.distributed` process group (gloo on CPU, NCCL on
    GPUs): carries the communicator id to the ranks, gathers the logits once per prefill, and, for the CPU
    tests, plays the all-reduce for the oracle.  With a CUDA `device`, `device_comm` is the executor's own NCCL
    communicator (kyanite_b200.executor.Communicator), created from an id that rank 0 makes and this process
    group broadcasts."""

    def __init__(self, device: Optional[str] = None):
        import torch
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")
        self.torch, self.dist = torch, dist
        self.rank, self.world = dist.get_rank(), dist.get_world_size()
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        self.device_comm = None
        if self.device.type == "cuda":
            from .executor import Communicator
            box = [Communicator.unique_id() if self.rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            index = self.device.index if self.device.index is not None else torch.cuda.current_device()
            self.device_comm = Communicator(index, self.rank, self.world, box[0])

    def all_reduce_sum(self, a: np.ndarray) -> np.ndarray:
        t = self.torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return t.cpu().numpy()

    def all_gather_last_axis(self, a: np.ndarray) -> np.ndarray:
        t = self.torch.from_numpy(np.ascontiguousarray(a)).to(self.device)
        parts = [self.torch.empty_like(t) for _ in range(self.world)]
        self.dist.all_gather(parts, t)
        return self.torch.cat(parts, dim=-1).cpu().numpy()

    def close(self):
        if self.device_comm is not None:
            self.device_comm.close()
            self.device_comm = None


class TensorParallelLlama:
    """One rank of the tensor-parallel decoder.

    `prepare(graph, batch_size, comm)` returns a callable `inputs -> outputs` for the rank's graph: on a GPU
    `cuda_prepare(device)`, which builds a `CudaExecutor` and attaches `comm.device_comm`; tests on CPU pass an
    evaluator that runs the oracle with `comm.all_reduce_sum` as the collective."""

    def __init__(self, cfg: LlamaShape, batch_size: int, comm, prepare: Callable):
        self.cfg, self.batch_size, self.comm = cfg, batch_size, comm
        self.graph = llama_rank_graph(cfg, comm.rank, comm.world)
        self.run = prepare(self.graph, batch_size, comm)
        self.all_reduces = 2 * cfg.layers

    def forward_local(self, ids: np.ndarray) -> np.ndarray:
        """Token ids [B, seq] (identical on every rank) -> this rank's slice of the logits."""
        (local_logits,) = self.run([np.ascontiguousarray(ids, dtype=np.int32)])
        return local_logits

    def forward(self, ids: np.ndarray) -> np.ndarray:
        """Token ids [B, seq] (identical on every rank) -> logits [B, seq, vocab] (identical on every rank)."""
        return self.comm.all_gather_last_axis(self.forward_local(ids))


def cuda_prepare(device_index: int, **executor_kwargs) -> Callable:
    """`prepare` for `TensorParallelLlama` (and for single segments: `comm` may be omitted) on CUDA device
    `device_index`.  The executor is reachable as `.executor` of the returned callable."""
    from .executor import CudaExecutor

    def prepare(graph: Graph, batch_size: int, comm=None):
        ex = CudaExecutor(device_index, graph, batch_size, **executor_kwargs)
        if comm is not None and getattr(comm, "device_comm", None) is not None:
            ex.set_comm(comm.device_comm)

        def run(inputs):
            return ex.evaluate(inputs)

        run.executor = ex
        return run

    return prepare
