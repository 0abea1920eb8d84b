"""Batch sharding on CPU with two gloo ranks: each rank evaluates its shard of a global batch (with
the CPU oracle standing in for a device), rank 0 merges and compares with the unsharded result."""
import os
import socket

import numpy as np
import pytest
import torch.distributed as dist
import torch.multiprocessing as mp

from kyanite_b200.configs import resnet_tower
from kyanite_b200.graph import BATCH, DType, Graph, shape
from kyanite_b200.sharding import (aggregate_throughput, batch_axis, check_shardable, merge_outputs, shard_sizes,
                                   split_inputs)
from oracle.cpu_eval import cpu_eval_graph


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, global_batch, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        graph, make_inputs = resnet_tower(channels=8, blocks=1)
        inputs = make_inputs(global_batch, 3)
        mine = split_inputs(graph, inputs, global_batch, rank, world)
        sizes = shard_sizes(global_batch, world)
        outs = cpu_eval_graph(graph.to_bytes(), sizes[rank], mine)
        gathered = [None] * world
        dist.all_gather_object(gathered, outs)
        times = [None] * world
        dist.all_gather_object(times, 1.0 + rank)   # pretend rank r took (1 + r) ms
        if rank == 0:
            merged = merge_outputs(graph, gathered)
            full = cpu_eval_graph(graph.to_bytes(), global_batch, inputs)
            ok = all(np.allclose(a, b, rtol=1e-5, atol=1e-6) for a, b in zip(merged, full))
            rate = aggregate_throughput(sizes, times)
            with open(result_path, "w") as f:
                f.write(f"{int(ok)} {rate}")
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("global_batch", [8, 7])
def test_two_rank_batch_sharding(tmp_path, global_batch):
    result = tmp_path / "result.txt"
    mp.spawn(_worker, args=(2, _free_port(), global_batch, str(result)), nprocs=2, join=True)
    ok, rate = result.read_text().split()
    assert ok == "1"
    assert float(rate) == pytest.approx(global_batch / 0.002)   # slowest rank: 2 ms


def test_shard_helpers():
    assert shard_sizes(10, 4) == [3, 3, 2, 2]
    assert batch_axis(shape(BATCH, 3)) == 0
    assert batch_axis(shape(4, 3)) is None
    g = Graph()
    a = g.input(shape(BATCH, 2))
    t = g.input(shape(3))
    g.output(g.add(a, g.view(g.slice(t, 0, (0, 2, 1)), shape(1, 2))))
    x = np.arange(8, dtype=np.float32).reshape(4, 2)
    tt = np.ones(3, np.float32)
    s0 = split_inputs(g, [x, tt], 4, 0, 2)
    s1 = split_inputs(g, [x, tt], 4, 1, 2)
    assert np.array_equal(s0[0], x[:2]) and np.array_equal(s1[0], x[2:]) and s0[1] is tt
    with pytest.raises(ValueError):
        batch_axis((BATCH * BATCH,))


def test_graphs_that_mix_batch_entries_are_refused():
    from kyanite_b200 import configs
    from kyanite_b200.graph import ReduceOp
    # every workload graph is per-sample
    for build in (configs.mlp, lambda: configs.resnet_tower(channels=8, blocks=1),
                  lambda: configs.bert_encoder(layers=1, hidden=32, heads=2, ffn=64, vocab=50, seq=8),
                  lambda: configs.unet_step(levels=(32,), res_blocks=1, attention_levels=(0,), heads=2, size=8, ctx_len=3,
                                            ctx_dim=8, groups=8)):
        check_shardable(build()[0])

    def graph_with(f):
        g = Graph()
        g.output(f(g, g.input(shape(BATCH, 6))))
        return g

    bad = {
        "reduces over": lambda g, x: g.reduce(x, [0], ReduceOp.SUM),
        "normalises along": lambda g, x: g.softmax(x, 0),
        "contracts over": lambda g, x: g.mat_mul(g.permute(x, [1, 0]), x),
        "slices or flips": lambda g, x: g.flip(x, 0),
        "is an all-reduce": lambda g, x: g.all_reduce(x),
    }
    for reason, f in bad.items():
        g = graph_with(f)
        with pytest.raises(ValueError, match=reason):
            check_shardable(g)
        with pytest.raises(ValueError, match="cannot be sharded"):
            split_inputs(g, [np.zeros((4, 6), np.float32)], 4, 0, 2)
    # the same operations along a per-sample axis are fine
    check_shardable(graph_with(lambda g, x: g.softmax(g.flip(x, 1), 1)))


def test_affinity_words_and_binding_decisions():
    """Which CPUs a rank is bound to, against a stand-in for NVML (no GPU, and the test leaves the process's own
    affinity as it found it)."""
    import os

    from kyanite_b200.sharding import bind_process_near_gpu, cpus_from_affinity_words

    assert cpus_from_affinity_words([0b1011]) == [0, 1, 3]
    assert cpus_from_affinity_words([0, 1 << 2]) == [66]

    class FakeNvml:
        def __init__(self, words):
            self.words = words

        def nvmlDeviceGetHandleByUUID(self, uuid):
            assert uuid == b"GPU-x"
            return object()

        def nvmlDeviceGetCpuAffinity(self, handle, n_words):
            return self.words[:n_words] + [0] * max(0, n_words - len(self.words))

    before = os.sched_getaffinity(0)
    try:
        allowed = sorted(before)
        # the GPU's CPUs lie outside what this process may use: nothing changes
        far = [0] * (max(allowed) // 64 + 2)
        far[-1] = 1 << 63
        r = bind_process_near_gpu("GPU-x", allowed=allowed, nvml=FakeNvml(far))
        assert r["bound"] is False and os.sched_getaffinity(0) == before
        # every allowed CPU is ideal: nothing to do
        every = [(1 << 64) - 1] * (max(allowed) // 64 + 1)
        r = bind_process_near_gpu("GPU-x", allowed=allowed, nvml=FakeNvml(every))
        assert r["bound"] is False and os.sched_getaffinity(0) == before
        # a query that fails is reported, not raised
        class Broken(FakeNvml):
            def nvmlDeviceGetCpuAffinity(self, handle, n_words):
                raise RuntimeError("not supported")
        assert bind_process_near_gpu("GPU-x", allowed=allowed, nvml=Broken([]))["bound"] is False
        if len(allowed) >= 2:
            # half of the allowed CPUs are ideal: the process is restricted to them
            half = allowed[: len(allowed) // 2]
            words = [0] * (max(allowed) // 64 + 1)
            for c in half:
                words[c // 64] |= 1 << (c % 64)
            r = bind_process_near_gpu("GPU-x", allowed=allowed, nvml=FakeNvml(words))
            assert r == {"bound": True, "cpus": len(half), "of": len(allowed)}
            assert sorted(os.sched_getaffinity(0)) == half
    finally:
        os.sched_setaffinity(0, before)
