"""Times the tensor-parallel LLaMA-shaped prefill: one process per GPU, every rank running its graph through one
executor whose all-reduce steps go to NCCL on the executor's stream.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \
        -m kyanite_b200.tp_bench [--layers 32] [--seq 2048] [--batch 1] [--iters 5]

Rank 0 prints one JSON line: milliseconds per prefill (CUDA events on the executor's stream, max over ranks),
tokens/s, and the share of the step time spent in all-reduce steps (from a step-by-step profiled run, where a
step's time includes waiting for the slowest rank).  Weights are synthetic: every rank draws only its own
slices (`draw_slices_only`), so the numbers are not those of an unpartitioned model; timing does not depend
on them.  torch.distributed is used to launch and to carry the communicator id, not in the data path."""
from __future__ import annotations

import argparse
import json
import os
import time

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--d-model", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--ffn", type=int, default=11008)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16"])
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from .executor import CudaExecutor
    from .tensor_parallel import LlamaShape, TorchComm, llama_rank_graph

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", local_rank))

    cfg = LlamaShape(layers=args.layers, d_model=args.d_model, heads=args.heads, ffn=args.ffn, vocab=args.vocab, seq=args.seq)
    t0 = time.perf_counter()
    graph_kwargs = {"dtype": args.dtype} if args.dtype != "f32" else {}
    graph = llama_rank_graph(cfg, rank, world, draw_slices_only=True, **graph_kwargs)
    t_build = time.perf_counter() - t0
    comm = TorchComm(f"cuda:{local_rank}")
    ex = CudaExecutor(local_rank, graph, args.batch)
    del graph
    ex.set_comm(comm.device_comm)
    ids = np.random.Generator(np.random.PCG64(3)).integers(0, cfg.vocab, (args.batch, cfg.seq)).astype(np.int32)
    ex.host_inputs[0][...] = ids
    stream = torch.cuda.ExternalStream(ex.stream(), device=torch.device("cuda", local_rank))

    ex.upload_inputs()
    for _ in range(2):
        ex.run_async()
    ex.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record(stream)
    for _ in range(args.iters):
        ex.run_async()
    b.record(stream)
    ex.synchronize()
    ms = a.elapsed_time(b) / args.iters

    # step-by-step profile: which share is all-reduce
    ex.set_profile(True)
    ex.run_async()
    ex.set_profile(False)
    totals = {}
    n_reduce = 0
    for line in ex.last_profile().splitlines():
        parts = line.split()
        if parts and parts[0] == "total":
            totals[parts[1]] = float(parts[2])
        elif len(parts) > 2 and parts[0].isdigit() and parts[1] == "AllReduce":
            n_reduce += 1
    step_sum = sum(v for k, v in totals.items() if k != "tensor_core")
    steps, launches = ex.step_count()

    t = torch.tensor([ms, totals.get("AllReduce", 0.0), step_sum], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, reduce_us, step_sum = t.tolist()
    if rank == 0:
        tokens = args.batch * cfg.seq
        # ring all-reduce moves 2 (W-1)/W of the buffer per rank and direction
        bytes_per_reduce = tokens * cfg.d_model * (2 if args.dtype == "f16" else 4)
        line = {"workload": f"llama-shaped prefill, {cfg.layers} layers, d_model {cfg.d_model}, {cfg.heads} heads, ffn {cfg.ffn}, "
                            f"vocab {cfg.vocab}, batch {args.batch} x {cfg.seq} tokens, {args.dtype} storage, tensor-parallel x{world}",
                "n_gpus": world, "ms_per_prefill": ms, "tokens_per_s": tokens / (ms / 1000.0), "steps": steps,
                "all_reduce_steps": n_reduce, "all_reduce_bytes_each": bytes_per_reduce,
                "profiled_step_sum_ms": step_sum / 1000.0, "all_reduce_ms": reduce_us / 1000.0,
                "all_reduce_share_of_steps": reduce_us / step_sum if step_sum else None,
                "all_reduce_bus_gbs": (2.0 * (world - 1) / world * bytes_per_reduce * n_reduce / (reduce_us * 1e-6) / 1e9
                                       if reduce_us > 0 and world > 1 else None),
                "mem": {"arena_bytes": ex.mem_usage.shared_bytes, "const_bytes": ex.mem_usage.dedicated_bytes},
                "graph_build_s": t_build, "per_kind_us": totals}
        print(json.dumps(line), flush=True)
    ex.close()
    comm.close()
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
