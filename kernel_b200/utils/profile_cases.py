"""Small single-GPU cases of each hand-written kernel, for profilers.

    python -m kernel_b200.utils.profile_cases gemm   [--m 8192 --n 8192 --k 2048] [--iters 3]
    python -m kernel_b200.utils.profile_cases a2a    [--tokens 256] [--iters 3]
    python -m kernel_b200.utils.profile_cases a2a3   (the three-launch variant)

Each case holds a few hundred MB on the device (more than the L2, far less than
a full-size workload), runs a handful of launches and exits, so that a capture
ends by itself.  On one GPU the reduce-scatter and all-gather variants of the
GEMM reduce to the plain kernel; their communication paths need several ranks
and are measured with CUDA events instead (``kernel_b200.utils.sweep``).
"""
from __future__ import annotations

import argparse
import os

import torch


def run_gemm(m: int, n: int, k: int, iters: int, pair=None) -> None:
    from ..ops.gemm import gemm

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    a = torch.randn(m, k, device=dev).to(torch.bfloat16)
    b = (torch.randn(n, k, device=dev) / k ** 0.5).to(torch.bfloat16)
    bias = (torch.randn(n, device=dev) * 0.02).to(torch.bfloat16)
    out = torch.empty(m, n, device=dev, dtype=torch.bfloat16)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for i in range(iters):
        if i == iters - 1:
            ev[0].record()
        gemm(a, b, bias, out=out, pair=pair)
    ev[1].record()
    torch.cuda.synchronize()
    us = ev[0].elapsed_time(ev[1]) * 1e3
    ref = a[:256].float() @ b.float().t() + bias.float()
    err = (out[:256].float() - ref).abs().max().item()
    print(f"gemm {m}x{n}x{k}: {us:.1f} us, {2 * m * n * k / us / 1e6:.1f} TFLOP/s, max err {err:.4f}")


def run_a2a(tokens: int, iters: int, fused: bool) -> None:
    os.environ["KB200_A2A_FUSED"] = "1" if fused else "0"
    from ..ops.dispatch_combine import SCALE_EXPERT, MoEAllToAll

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    E, k, H = 256, 8, 7168
    ctx = MoEAllToAll(E, k, H, tokens, dtype=torch.bfloat16, device=dev)
    x = torch.randn(tokens, H, device=dev).to(torch.bfloat16)
    idx = torch.rand(tokens, E, device=dev).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(tokens, k, device=dev), -1)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    for i in range(iters):
        if i == iters - 1:
            ev[0].record()
        out = ctx.dispatch_scale_combine(x, idx, w, SCALE_EXPERT)
    ev[1].record()
    torch.cuda.synchronize()
    ctx.heap.check_status()
    print(f"a2a T={tokens} fused={fused}: {ev[0].elapsed_time(ev[1]) * 1e3:.1f} us, out mean {out.float().abs().mean().item():.4f}")


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=["gemm", "a2a", "a2a3"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--iters", type=int, default=3)
    ap.add_argument("--pair", type=int, default=None, help="gemm: 1 = CTA-pair kernel, 0 = single-CTA kernel, default: the faster of the two")
    ns = ap.parse_args()
    if ns.case == "gemm":
        run_gemm(ns.m, ns.n, ns.k, ns.iters, None if ns.pair is None else bool(ns.pair))
    else:
        run_a2a(ns.tokens, ns.iters, fused=ns.case == "a2a")


if __name__ == "__main__":
    main()
