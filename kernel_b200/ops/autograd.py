"""Differentiable front-ends of the two fused GEMM+collective ops.

The two ops are each other's transpose, which makes training a sequence-parallel
tensor-parallel block need nothing new on the device:

* ``y = AG(x_local) @ W^T``  (column-parallel; ``AGGemm``)
  has ``dx_local = RS(dy @ W)``, a GEMM fused with reduce-scatter;
* ``y_local = RS(x @ W^T)``  (row-parallel; ``GemmRS``)
  has ``dx = AG(dy_local) @ W``, an all-gather fused with a GEMM.

The weight gradients contract over the token dimension and need the gathered
operand (``x`` resp. ``dy``); it is gathered with one library collective and the
product is the plain tcgen05 GEMM.  The gather runs on the same stream as the fused
kernel, before it: the fused kernels are persistent, fill every SM and wait (with a
limit) for their peers, so a collective kernel of another stream that is scheduled
behind them on one rank and ahead of them on another could make the ranks wait on
each other until the limit expires.  CPU tensors take the torch paths of the ops, so the wiring
is testable on gloo ranks.

The reference has forward-only kernels (``gemm_rs/submission.py:5-29``); nothing
there corresponds to this file.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..parallel.symm import _dist_info
from .gemm import AGGemm, GemmRS, gemm


def _gather_rows(t_local: torch.Tensor, world: int, group) -> torch.Tensor:
    if world == 1:
        return t_local
    full = torch.empty((t_local.shape[0] * world, t_local.shape[1]), dtype=t_local.dtype, device=t_local.device)
    dist.all_gather_into_tensor(full, t_local.contiguous(), group=group)
    return full


def _wgrad(dy_full: torch.Tensor, x_full: torch.Tensor) -> torch.Tensor:
    """``dW[N, K] = dy_full[M, N]^T @ x_full[M, K]``; both operands are made
    M-major (K-major in the kernel's terms) by a transpose copy."""
    return gemm(dy_full.t().contiguous(), x_full.t().contiguous())


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, w, bias, layer):
        ctx.layer = layer
        ctx.save_for_backward(x_local, w)
        ctx.has_bias = bias is not None
        return layer.fwd(x_local.contiguous(), w.contiguous(), bias)

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        x_local, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = db = None
        need_dw = ctx.needs_input_grad[1]
        if need_dw:
            x_full = _gather_rows(x_local, layer.world, layer.group)
        if ctx.needs_input_grad[0]:
            # dx_local[M/world, K] = RS(dy[M, Nl] @ W[Nl, K]): contraction over the sharded Nl
            dx = layer.bwd(dy, w.t().contiguous())
        if need_dw:
            dw = _wgrad(dy, x_full)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy.float().sum(0).to(dy.dtype)
        return dx, dw, db, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, layer):
        ctx.layer = layer
        ctx.save_for_backward(x, w)
        ctx.has_bias = bias is not None
        return layer.fwd(x.contiguous(), w.contiguous(), bias)

    @staticmethod
    def backward(ctx, dy_local):
        layer = ctx.layer
        x, w = ctx.saved_tensors
        dy_local = dy_local.contiguous()
        dx = dw = db = None
        need_dw = ctx.needs_input_grad[1]
        if need_dw:
            dy_full = _gather_rows(dy_local, layer.world, layer.group)
        if ctx.needs_input_grad[0]:
            # dx[M, Kl] = AG(dy_local)[M, N] @ W[N, Kl]
            dx = layer.bwd(dy_local, w.t().contiguous())
        if need_dw:
            dw = _wgrad(dy_full, x)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            # the bias is added once to every output row; this is the sum over this
            # rank's rows, to be summed over ranks with the other replicated parameters
            db = dy_local.float().sum(0).to(dy_local.dtype)
        return dx, dw, db, None


class ColumnParallelLinear(torch.nn.Module):
    """``y[M, out/world] = all_gather(x_local)[M, in] @ W_shard^T + b_shard`` with
    the all-gather fused into the GEMM forward and the reduce-scatter fused into
    the input-gradient GEMM backward.  ``tokens`` is the global row count M."""

    def __init__(self, tokens: int, in_features: int, out_features_local: int, bias: bool = True, group=None,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.group = group
        self.rank, self.world = _dist_info(group)
        self.weight = torch.nn.Parameter(torch.empty(out_features_local, in_features, dtype=dtype, device=dev))
        self.bias = torch.nn.Parameter(torch.zeros(out_features_local, dtype=dtype, device=dev)) if bias else None
        torch.nn.init.normal_(self.weight, std=in_features ** -0.5)
        self.fwd = AGGemm(tokens, in_features, group=group, device=dev)
        self.bwd = GemmRS(tokens, in_features, group=group, device=dev)

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        return _ColumnParallelFn.apply(x_local, self.weight, self.bias, self)

    def close(self) -> None:
        for c in (self.fwd, self.bwd):
            if c.heap is not None:
                c.heap.close()


class RowParallelLinear(torch.nn.Module):
    """``y_local[M/world, out] = reduce_scatter(x[M, in/world] @ W_shard^T) + b`` with
    the reduce-scatter fused into the GEMM forward and the all-gather fused into
    the input-gradient GEMM backward.  The bias is replicated: its gradient here is
    the sum over this rank's rows."""

    def __init__(self, tokens: int, in_features_local: int, out_features: int, bias: bool = True, group=None,
                 device: Optional[torch.device] = None, dtype: torch.dtype = torch.bfloat16):
        super().__init__()
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.group = group
        self.rank, self.world = _dist_info(group)
        self.weight = torch.nn.Parameter(torch.empty(out_features, in_features_local, dtype=dtype, device=dev))
        self.bias = torch.nn.Parameter(torch.zeros(out_features, dtype=dtype, device=dev)) if bias else None
        torch.nn.init.normal_(self.weight, std=(in_features_local * self.world) ** -0.5)
        self.fwd = GemmRS(tokens, out_features, group=group, device=dev)
        self.bwd = AGGemm(tokens, out_features, group=group, device=dev)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _RowParallelFn.apply(x, self.weight, self.bias, self)

    def close(self) -> None:
        for c in (self.fwd, self.bwd):
            if c.heap is not None:
                c.heap.close()
