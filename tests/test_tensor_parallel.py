"""Tensor-parallel LLaMA-shaped decoder (kyanite_b200/tensor_parallel.py).

Every rank runs one graph with all-reduce values in it.
CPU: two and four gloo ranks run their graphs through the CPU oracle, whose all-reduce values are played by
torch.distributed, and every rank must end with the logits of the unpartitioned graph.
GPU: one rank with a real NCCL communicator of size one (the executor's ncclAllReduce path on any box); the
rank slices of a two-rank partition run segment by segment on one device; two ranks on two GPUs with the
all-reduce steps going to NCCL from inside the executor (needs two devices; skipped otherwise)."""
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from kyanite_b200.configs import llama_decoder
from kyanite_b200.tensor_parallel import (LlamaShape, LocalComm, TensorParallelLlama, TorchComm, cuda_prepare,
                                          llama_rank_graph, llama_segments)
from oracle.cpu_eval import assert_tensors_match, cpu_eval_graph

CFG = LlamaShape(layers=2, d_model=64, heads=4, ffn=96, vocab=100, seq=16)
BATCH_SIZE = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def oracle_prepare(graph, batch_size, comm=None):
    blob = graph.to_bytes()
    reduce = comm.all_reduce_sum if comm is not None else None
    return lambda inputs: cpu_eval_graph(blob, batch_size, inputs, all_reduce=reduce)


def full_logits(ids):
    graph, _ = llama_decoder(layers=CFG.layers, d_model=CFG.d_model, heads=CFG.heads, ffn=CFG.ffn, vocab=CFG.vocab,
                             seq=CFG.seq, eps=CFG.eps, rope_base=CFG.rope_base, seed=CFG.seed)
    return cpu_eval_graph(graph.to_bytes(), ids.shape[0], [ids])[0]


def token_ids():
    return np.random.Generator(np.random.PCG64(5)).integers(0, CFG.vocab, (BATCH_SIZE, CFG.seq)).astype(np.int32)


def test_segment_count_and_shapes():
    for world in (1, 2, 4):
        segs = llama_segments(CFG, 0, world)
        assert len(segs) == 2 * CFG.layers + 1
        assert len(segs[0].inputs) == 1 and len(segs[0].outputs) == 2
        assert all(len(s.inputs) == 2 and len(s.outputs) == 2 for s in segs[1:-1])
        last = segs[-1]
        assert last[last.outputs[0]].shape[-1].factor == CFG.vocab // world
    with pytest.raises(ValueError, match="not divisible"):
        llama_segments(CFG, 0, 3)
    with pytest.raises(ValueError, match="outside world"):
        llama_segments(CFG, 2, 2)


def test_rank_graph_has_one_all_reduce_per_block():
    from kyanite_b200.executor import plan_describe
    from kyanite_b200.graph import OpKind
    for world in (1, 2, 4):
        g = llama_rank_graph(CFG, world - 1, world)
        assert sum(1 for info in g.values if info.kind == OpKind.ALL_REDUCE) == 2 * CFG.layers
        assert len(g.inputs) == 1 and len(g.outputs) == 1
        assert g[g.outputs[0]].shape[-1].factor == CFG.vocab // world
        steps = [l for l in plan_describe(g, BATCH_SIZE).splitlines() if l.startswith("step")]
        reduces = [l for l in steps if " AllReduce " in l]
        assert len(reduces) == 2 * CFG.layers
        assert all(f"count={BATCH_SIZE * CFG.seq * CFG.d_model} f32" in l for l in reduces)


def test_single_rank_equals_whole_graph():
    ids = token_ids()
    tp = TensorParallelLlama(CFG, BATCH_SIZE, LocalComm(), oracle_prepare)
    assert_tensors_match([full_logits(ids)], [tp.forward(ids)], 1e-5, 1e-5)
    assert tp.all_reduces == 2 * CFG.layers


def _cpu_worker(rank, world, port, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ids = token_ids()
        tp = TensorParallelLlama(CFG, BATCH_SIZE, TorchComm(), oracle_prepare)
        logits = tp.forward(ids)
        np.save(os.path.join(result_dir, f"logits{rank}.npy"), logits)
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_match_whole_graph(tmp_path, world):
    mp.spawn(_cpu_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    expected = full_logits(token_ids())
    for rank in range(world):
        got = np.load(tmp_path / f"logits{rank}.npy")
        # the partial sums are added in a different order than the whole matmul adds its terms
        assert_tensors_match([expected], [got], 1e-4, 1e-4)
    np.testing.assert_array_equal(np.load(tmp_path / "logits0.npy"), np.load(tmp_path / f"logits{world - 1}.npy"))


def _gpu_worker(rank, world, port, result_dir):
    import torch
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from kyanite_b200.executor import MATH_F32
        ids = token_ids()
        comm = TorchComm(f"cuda:{rank}")
        tp = TensorParallelLlama(CFG, BATCH_SIZE, comm, cuda_prepare(rank, math_mode=MATH_F32))
        first = tp.forward(ids)
        second = tp.forward(ids)
        np.testing.assert_array_equal(first, second)
        np.save(os.path.join(result_dir, f"logits{rank}.npy"), first)
        dist.barrier()
        tp.run.executor.close()
        comm.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
def test_two_gpus_nccl(tmp_path):
    from kyanite_b200.executor import CudaDevice
    if CudaDevice.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_gpu_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    expected = full_logits(token_ids())
    for rank in range(2):
        assert_tensors_match([expected], [np.load(tmp_path / f"logits{rank}.npy")], 1e-3, 1e-3)


@pytest.mark.gpu
@pytest.mark.parametrize("with_comm", [False, True], ids=["no_communicator", "nccl_world_of_one"])
def test_one_rank_on_gpu(with_comm):
    """The rank graph of a world of one on cuda:0: without a communicator the all-reduce steps are copies; with
    an NCCL communicator of size one attached they still are (one rank), and the communicator's creation and
    release go through the library's run-time binding of NCCL."""
    from kyanite_b200.executor import Communicator, CudaExecutor, MATH_F32
    ids = token_ids()
    expected = full_logits(ids)
    graph = llama_rank_graph(CFG, 0, 1)
    comm = Communicator(0, 0, 1, Communicator.unique_id()) if with_comm else None
    with CudaExecutor(0, graph, BATCH_SIZE, math_mode=MATH_F32) as ex:
        if comm is not None:
            ex.set_comm(comm)
        for _ in range(2):
            assert_tensors_match([expected], ex.evaluate([ids]), 1e-3, 1e-3)
        ex.set_comm(None)
        assert_tensors_match([expected], ex.evaluate([ids]), 1e-3, 1e-3)
    if comm is not None:
        comm.close()


@pytest.mark.gpu
def test_one_gpu_segments_match_oracle():
    """The segment graphs themselves on one GPU (both ranks' slices run one after the other on cuda:0,
    partial sums added on the host): no second device needed."""
    from kyanite_b200.executor import MATH_F32, MATH_TF32

    class TwoRanksOnOneDevice:
        """Runs rank 0's and rank 1's segments in lock step and plays the collective on the host."""

        def __init__(self, mode):
            prepare = cuda_prepare(0, math_mode=mode)
            self.ranks = [[prepare(g, BATCH_SIZE) for g in llama_segments(CFG, r, 2)] for r in range(2)]

        def forward(self, ids):
            outs = [segs[0]([ids]) for segs in self.ranks]
            for k in range(1, len(self.ranks[0]) - 1):
                s = outs[0][1] + outs[1][1]
                outs = [segs[k]([o[0], s]) for segs, o in zip(self.ranks, outs)]
            s = outs[0][1] + outs[1][1]
            return np.concatenate([segs[-1]([o[0], s])[0] for segs, o in zip(self.ranks, outs)], axis=-1)

    ids = token_ids()
    expected = full_logits(ids)
    assert_tensors_match([expected], [TwoRanksOnOneDevice(MATH_F32).forward(ids)], 1e-3, 1e-3)
    assert_tensors_match([expected], [TwoRanksOnOneDevice(MATH_TF32).forward(ids)], 4e-3, 4e-3, abs_scaled=True)
