"""Forward + backward time of the trainable sequence-parallel MLP.

    python -m kernel_b200.utils.train_bench [--tokens 8192 --hidden 8192 --ffn 29568 --iters 10]
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m kernel_b200.utils.train_bench

Device-timed with CUDA events (max over ranks), L2 flushed between iterations;
prints one JSON line with the step time and the tensor throughput of the six
GEMMs of a step (two forward, two input-gradient, two weight-gradient).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=8192)
    ap.add_argument("--ffn", type=int, default=29568, help="global MLP width; sharded over the ranks")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ns = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from kernel_b200.models import TrainableSequenceParallelMLP
    from kernel_b200.utils.common import clear_l2_cache

    fl = ns.ffn // world
    mlp = TrainableSequenceParallelMLP(ns.tokens, ns.hidden, fl, activation="gelu", device=dev)
    x = torch.randn(ns.tokens // world, ns.hidden, device=dev).to(torch.bfloat16).requires_grad_(True)
    gy = torch.randn(ns.tokens // world, ns.hidden, device=dev).to(torch.bfloat16)

    def step() -> None:
        for p in mlp.parameters():
            p.grad = None
        x.grad = None
        mlp(x).backward(gy)

    for _ in range(ns.warmup):
        step()
    times = []
    for _ in range(ns.iters):
        clear_l2_cache()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        e1.synchronize()
        t = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times.append(float(t))
    ms = sum(times) / len(times)
    flops = 6 * 2.0 * ns.tokens * ns.hidden * ns.ffn  # whole job, all ranks
    if rank == 0:
        print(json.dumps({"op": "sequence-parallel MLP forward+backward", "n_gpus": world, "tokens": ns.tokens, "hidden": ns.hidden,
                          "ffn": ns.ffn, "ms_per_step": round(ms, 3), "min_ms": round(min(times), 3),
                          "tflops_total": round(flops / ms / 1e9, 1), "tflops_per_gpu": round(flops / ms / 1e9 / world, 1)}))
    mlp.close()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
