"""Scaling sweep of the three fused ops against their NCCL + cuBLAS baselines.

    python -m torch.distributed.run --nproc-per-node N -m kernel_b200.utils.sweep \
        [--ops a2a,gemm_rs,ag_gemm] [--quick] [--out sweep_N.json]

Every number is a device time (CUDA events on the launching stream, L2 flushed
and ranks aligned by an in-stream all-reduce before the start event), MAX over
ranks, mean of ``--iters`` calls after ``--warmup``.  Rank 0 prints a table with
the achieved fraction of the roofline (slower of FLOPs at the GEMM peak and
NVLink bytes at the link bandwidth) and writes the rows as JSON.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

from . import roofline as rf

A2A_SHAPES = [  # tokens per rank, hidden, top-k, experts
    (1, 7168, 8, 256), (16, 7168, 8, 256), (128, 7168, 8, 256), (256, 7168, 8, 256), (512, 7168, 8, 256),
    (1024, 7168, 8, 256), (128, 2048, 4, 64), (256, 4096, 8, 256), (1024, 2048, 8, 64),
]
GEMM_RS_SHAPES = [  # m, n, k (k sharded); the first three are the small-M cases the reference ranks (gemm_rs/task.yml:79-81)
    (64, 7168, 18432), (512, 4096, 12288), (2048, 2880, 2880),
    (1024, 4096, 4096), (4096, 4096, 4096), (8192, 4096, 14336), (8192, 8192, 29568), (16384, 8192, 8192),
]
AG_GEMM_SHAPES = [  # m, n (n sharded), k
    (1024, 4096, 4096), (4096, 14336, 4096), (8192, 29568, 8192), (16384, 29568, 4096),
]
QUICK = {"a2a": [0, 3], "gemm_rs": [4, 6], "ag_gemm": [0, 2]}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", default="a2a,gemm_rs,ag_gemm")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--out", default=None)
    ap.add_argument("--timing-words", action="store_true",
                    help="GEMM ops: also report the kernel's timing words (us waited on peers, us until pushes were out, "
                         "us until the last epilogue or reduction; maximum over CTAs, calls and ranks)")
    ns = ap.parse_args()

    if ns.timing_words:
        os.environ["KB200_GEMM_TIMING"] = "1"  # read once, by the library's first GEMM launch
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

    from ..baseline import ag_gemm as ag_base
    from ..baseline import all2all as a2a_base
    from ..baseline import gemm_rs as rs_base
    from ..tasks.ag_gemm import reference as ag_ref
    from ..tasks.ag_gemm import submission as ag_sub
    from ..tasks.all2all import reference as a2a_ref
    from ..tasks.all2all import submission as a2a_sub
    from ..tasks.gemm_rs import reference as rs_ref
    from ..tasks.gemm_rs import submission as rs_sub

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    align = torch.zeros(1, device=dev)

    def timed(fn) -> float:
        ts = []
        for i in range(ns.warmup + ns.iters):
            flush.fill_(1)
            dist.all_reduce(align)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= ns.warmup:
                ts.append(e0.elapsed_time(e1) * 1e3)
        t = torch.tensor(ts, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        timed.last_min = float(t.min())
        timed.last_median = float(t.median())
        return float(t.mean())

    nominal = rf.Peaks()
    measured = rf.measured_peaks() or rf.Peaks(1642.6, rf.MEASURED_NVLINK_GBS, "measured")
    rows = []

    def timing_words(ctx):
        if not ns.timing_words or ctx is None:
            return None
        w = ctx.status[5:8].to(torch.int64).clone()
        dist.all_reduce(w, op=dist.ReduceOp.MAX)
        ctx.status.zero_()
        return w.tolist()

    def record(op, shape, fused_us, base_us, ok, roof_nom, roof_meas, fused_min=None, msg="", words=None):
        row = {"op": op, "shape": shape, "world": world, "fused_us": round(fused_us, 2),
               "fused_min_us": round(fused_min, 2) if fused_min is not None else None, "check": msg[:160],
               "baseline_us": round(base_us, 2),
               "speedup": round(base_us / fused_us, 3), "correct": bool(ok),
               "roofline_nominal_us": round(roof_nom["roofline_us"], 2), "frac_nominal": round(roof_nom["roofline_us"] / fused_us, 3),
               "roofline_measured_us": round(roof_meas["roofline_us"], 2), "frac_measured": round(roof_meas["roofline_us"] / fused_us, 3)}
        if words is not None:
            row["timing_words_us"] = {"waited_on_peers": words[0], "pushes_out": words[1], "last_epilogue": words[2]}
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    ops = ns.ops.split(",")
    pick = (lambda name, lst: [lst[i] for i in QUICK[name]]) if ns.quick else (lambda name, lst: lst)
    if "a2a" in ops:
        for (T, H, k, E) in pick("a2a", A2A_SHAPES):
            if E % world:
                continue
            data = a2a_ref.generate_input(E, k, H, T, 7, rank, world, dtype="bf16", fixed_tokens=True, weight_mode="softmax",
                                          expert_scale="expert")
            out = a2a_sub.custom_kernel(data)
            ok, msg = a2a_ref.check_implementation(data, out)
            f = timed(lambda: a2a_sub.custom_kernel(data))
            fmin = timed.last_min
            b = timed(lambda: a2a_base.custom_kernel(data))
            record("a2a", {"tokens": T, "hidden": H, "topk": k, "experts": E}, f, b, ok,
                   rf.a2a_roofline_us(T, k, H, 2, world, nominal), rf.a2a_roofline_us(T, k, H, 2, world, measured), fmin, msg)
        a2a_sub.release_contexts()
    if "gemm_rs" in ops:
        for (m, n, k) in pick("gemm_rs", GEMM_RS_SHAPES):
            if m % world or k % world or (k // world) % 8:
                continue
            data = rs_ref.generate_input(rank, world, m, n, k, True, 3, dist="normal", bias_mode="once")
            out = rs_sub.custom_kernel(data)
            ok, msg = rs_ref.check_implementation(data, out)
            ctx = rs_sub.get_context(m, n, dev)
            ctx.status.zero_()
            f = timed(lambda: rs_sub.custom_kernel(data))
            fmin = timed.last_min
            words = timing_words(ctx)
            b = timed(lambda: rs_base.custom_kernel(data))
            record("gemm_rs", {"m": m, "n": n, "k": k}, f, b, ok, rf.gemm_rs_roofline_us(m, n, k, world, nominal),
                   rf.gemm_rs_roofline_us(m, n, k, world, measured), fmin, msg, words)
        rs_sub.release_contexts()
    if "ag_gemm" in ops:
        for (m, n, k) in pick("ag_gemm", AG_GEMM_SHAPES):
            if m % world or n % world or (n // world) % 8:
                continue
            data = ag_ref.generate_input(rank, world, m, n, k, True, 5)
            out = ag_sub.custom_kernel(data)
            ok, msg = ag_ref.check_implementation(data, out)
            ctx = ag_sub.get_context(m, k, dev)
            ctx.status.zero_()
            f = timed(lambda: ag_sub.custom_kernel(data))
            fmin = timed.last_min
            words = timing_words(ctx)
            b = timed(lambda: ag_base.custom_kernel(data))
            record("ag_gemm", {"m": m, "n": n, "k": k}, f, b, ok, rf.ag_gemm_roofline_us(m, n, k, world, nominal),
                   rf.ag_gemm_roofline_us(m, n, k, world, measured), fmin, msg, words)
        ag_sub.release_contexts()
    if rank == 0 and ns.out:
        with open(ns.out, "w") as fh:
            json.dump(rows, fh, indent=1)
    torch.cuda.synchronize()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
