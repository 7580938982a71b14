"""Sequence-parallel tensor-parallel MLP: the region that the reference's two
collectives bracket (``gemm_rs/task.yml:16-22`` describes the exit GEMM).

Activations enter and leave sharded along the token dimension.  The up
projection is column-parallel and needs every token: all-gather fused with the
GEMM.  The down projection is row-parallel (its K dimension is the sharded
hidden dimension of the MLP) and produces partial sums for every token: GEMM
fused with the reduce-scatter.  ``SequenceParallelMLP`` is the forward-only block over
given weights; ``TrainableSequenceParallelMLP`` owns parameters and has a backward pass.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops.gemm import AGGemm, GemmRS
from ..parallel.symm import _dist_info


class SequenceParallelMLP:
    """``y_local = RS( act( AG(x_local) @ W1_shard^T + b1_shard ) @ W2_shard^T ) + b2``.

    ``w1`` is this rank's ``[ffn/world, hidden]`` shard, ``w2`` its ``[hidden,
    ffn/world]`` shard; ``tokens`` is the global token count (a multiple of the
    world size).
    """

    def __init__(self, tokens: int, hidden: int, w1: torch.Tensor, w2: torch.Tensor, b1: Optional[torch.Tensor] = None,
                 b2: Optional[torch.Tensor] = None, activation: str = "gelu", group=None):
        self.rank, self.world = _dist_info(group)
        if w1.shape[1] != hidden or w2.shape[0] != hidden or w2.shape[1] != w1.shape[0]:
            raise ValueError("w1 must be [ffn/world, hidden] and w2 [hidden, ffn/world]")
        self.w1, self.w2, self.b1, self.b2 = w1.contiguous(), w2.contiguous(), b1, b2
        self.activation = activation
        dev = w1.device
        self.up = AGGemm(tokens, hidden, group=group, device=dev)
        self.down = GemmRS(tokens, hidden, group=group, device=dev)

    def _act(self, h: torch.Tensor) -> torch.Tensor:
        if self.activation == "gelu":
            return torch.nn.functional.gelu(h, approximate="tanh")
        if self.activation == "relu":
            return torch.relu(h)
        if self.activation == "silu":
            return torch.nn.functional.silu(h)
        raise ValueError(f"unknown activation {self.activation!r}")

    def __call__(self, x_local: torch.Tensor) -> torch.Tensor:
        h = self.up(x_local, self.w1, self.b1)           # [tokens, ffn/world]
        h = self._act(h)
        return self.down(h, self.w2, self.b2)            # [tokens/world, hidden]

    def reference(self, x_full: torch.Tensor, w1_full: torch.Tensor, w2_full: torch.Tensor, b1_full=None, b2=None) -> torch.Tensor:
        """Unsharded fp32 result for all tokens (tests)."""
        h = x_full.float() @ w1_full.float().t()
        if b1_full is not None:
            h = h + b1_full.float()
        h = self._act(h.to(torch.bfloat16)).float()
        y = h @ w2_full.float().t()
        if b2 is not None:
            y = y + b2.float()
        return y

    def close(self) -> None:
        for ctx in (self.up, self.down):
            if ctx.heap is not None:
                ctx.heap.close()


class TrainableSequenceParallelMLP(torch.nn.Module):
    """The same block as ``SequenceParallelMLP`` with parameters and a backward
    pass: ``ColumnParallelLinear`` (all-gather fused forward, reduce-scatter fused
    input gradient) -> activation -> ``RowParallelLinear`` (the mirror image).
    ``ffn_local`` is this rank's share of the MLP's hidden dimension."""

    def __init__(self, tokens: int, hidden: int, ffn_local: int, bias: bool = True, activation: str = "gelu", group=None,
                 device: Optional[torch.device] = None):
        super().__init__()
        from ..ops.autograd import ColumnParallelLinear, RowParallelLinear

        self.up = ColumnParallelLinear(tokens, hidden, ffn_local, bias=bias, group=group, device=device)
        self.down = RowParallelLinear(tokens, ffn_local, hidden, bias=bias, group=group, device=device)
        self.activation = activation

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        h = self.up(x_local)
        if self.activation == "gelu":
            h = torch.nn.functional.gelu(h, approximate="tanh")
        elif self.activation == "relu":
            h = torch.relu(h)
        elif self.activation == "silu":
            h = torch.nn.functional.silu(h)
        else:
            raise ValueError(f"unknown activation {self.activation!r}")
        return self.down(h)

    def close(self) -> None:
        self.up.close()
        self.down.close()
