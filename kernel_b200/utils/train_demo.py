"""A few optimisation steps on the trainable blocks: a student sequence-parallel
MLP (optionally followed by the expert-parallel MoE block) is fitted to a fixed
random teacher.  Shows what a training loop around the fused ops looks like:
fp32 master weights, bf16 parameters, gradients of replicated parameters summed
over the ranks.

    python -m kernel_b200.utils.train_demo --steps 30
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m kernel_b200.utils.train_demo --moe

Runs on CPU ranks (gloo) as well as on GPUs (nccl).
"""
from __future__ import annotations

import argparse
import os
from typing import List

import torch
import torch.distributed as dist


class MasterSGD:
    """SGD with momentum on fp32 master copies of bf16 parameters."""

    def __init__(self, params, lr: float, momentum: float = 0.9):
        self.params = [p for p in params if p.requires_grad]
        self.master = [p.detach().float().clone() for p in self.params]
        self.buf = [torch.zeros_like(m) for m in self.master]
        self.lr, self.momentum = lr, momentum

    @torch.no_grad()
    def step(self) -> None:
        for p, m, b in zip(self.params, self.master, self.buf):
            if p.grad is None:
                continue
            b.mul_(self.momentum).add_(p.grad.float())
            m.add_(b, alpha=-self.lr)
            p.copy_(m)
            p.grad = None


def train(steps: int = 30, tokens: int = 256, hidden: int = 128, ffn: int = 256, moe: bool = False, lr: float = 0.05,
          device: str = "auto", seed: int = 0) -> List[float]:
    """Returns the global loss of every step."""
    from kernel_b200.models import TrainableMoELayer, TrainableSequenceParallelMLP

    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if device == "auto":
        device = f"cuda:{int(os.environ.get('LOCAL_RANK', '0'))}" if torch.cuda.is_available() else "cpu"
    dev = torch.device(device)
    g = torch.Generator().manual_seed(seed)  # identical on every rank; slices are taken below
    x_full = torch.randn(tokens, hidden, generator=g)
    teacher = torch.randn(hidden, hidden, generator=g) / hidden ** 0.5
    y_full = torch.tanh(x_full @ teacher)
    tl = tokens // world
    x = x_full[rank * tl:(rank + 1) * tl].to(dev).to(torch.bfloat16)
    y = y_full[rank * tl:(rank + 1) * tl].to(dev)

    torch.manual_seed(seed + 1 + rank)  # different shards on different ranks
    mlp = TrainableSequenceParallelMLP(tokens, hidden, ffn // world, activation="silu", device=dev)
    blocks = [mlp]
    replicated = [mlp.down.bias]
    if moe:
        experts, topk = 4 * world, 2
        layer = TrainableMoELayer(experts, topk, hidden, ffn, tl, device=dev)
        router = torch.nn.Parameter((torch.randn(hidden, experts, generator=g) / hidden ** 0.5).to(dev))  # replicated, fp32
        blocks.append(layer)
        replicated.append(router)
    params = [p for b in blocks for p in b.parameters()] + ([router] if moe else [])
    opt = MasterSGD(params, lr)

    losses = []
    for _ in range(steps):
        h = mlp(x)
        if moe:
            logits = h.float() @ router
            top = logits.topk(topk, dim=-1)
            weights = torch.softmax(top.values, dim=-1)
            h = h + layer(h, top.indices.to(torch.int32).contiguous(), weights.contiguous())
        loss_local = (h.float() - y).square().sum() / (tokens * hidden)   # this rank's share of the global mean
        loss_local.backward()
        total = loss_local.detach().clone()
        if world > 1:
            dist.all_reduce(total)
            for p in replicated:  # every rank holds these whole: their gradients are partial sums
                if p.grad is not None:
                    g32 = p.grad.float()
                    dist.all_reduce(g32)
                    p.grad.copy_(g32)
        losses.append(float(total))
        opt.step()
    for b in blocks:
        b.close()
    return losses


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--hidden", type=int, default=128)
    ap.add_argument("--ffn", type=int, default=256)
    ap.add_argument("--moe", action="store_true")
    ap.add_argument("--lr", type=float, default=0.05)
    ns = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        kwargs = {}
        if torch.cuda.is_available():
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group("nccl" if torch.cuda.is_available() else "gloo", **kwargs)
    losses = train(ns.steps, ns.tokens, ns.hidden, ns.ffn, ns.moe, ns.lr)
    if not dist.is_initialized() or dist.get_rank() == 0:
        print(" ".join(f"{v:.4f}" for v in losses))
    if dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
