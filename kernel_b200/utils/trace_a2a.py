"""Per-phase timing of the MoE round trip on N ranks, from the kernel's own
phase stamps (the role of the reference's ``all2all/submission_timed.py``).

    python -m torch.distributed.run --nproc-per-node N -m kernel_b200.utils.trace_a2a [--tokens 1,16,256]

CTA 0 of every rank records the global timer at each phase boundary; the table
shows, per phase, the mean over calls and the maximum over ranks, next to the
CUDA-event time of the whole call (L2 flushed, ranks aligned before the start).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,16,128,256,512")
    ap.add_argument("--experts", type=int, default=256)
    ap.add_argument("--topk", type=int, default=8)
    ap.add_argument("--hidden", type=int, default=7168)
    ap.add_argument("--iters", type=int, default=10)
    ns = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in os.environ:  # single process without a launcher: any free port
        import socket

        with socket.socket() as sock:
            sock.bind(("127.0.0.1", 0))
            os.environ["MASTER_PORT"] = str(sock.getsockname()[1])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from ..tasks.all2all import reference as R
    from ..tasks.all2all import submission as S

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    align = torch.zeros(1, device=dev)
    for T in [int(t) for t in ns.tokens.split(",")]:
        data = R.generate_input(ns.experts, ns.topk, ns.hidden, T, 4, rank, world, dtype="bf16", fixed_tokens=True,
                                weight_mode="softmax", expert_scale="expert")
        ctx = S.get_context(data[0], world, dev)
        ctx.enable_trace()
        rows, events = [], []
        for i in range(3 + ns.iters):
            flush.fill_(1)
            dist.all_reduce(align)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            S.custom_kernel(data)
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                rows.append(ctx.read_trace())
                events.append(e0.elapsed_time(e1) * 1e3)
        keys = list(rows[0].keys())
        t = torch.tensor([[r[k] for k in keys] + [e] for r, e in zip(rows, events)], dtype=torch.float64, device=dev).mean(0)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            out = {k: round(v, 1) for k, v in zip(keys + ["event_us"], t.tolist())}
            print(json.dumps({"tokens": T, "world": world, **out}), flush=True)
    torch.cuda.synchronize()
    S.release_contexts()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
