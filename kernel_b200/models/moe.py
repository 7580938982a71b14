"""Expert-parallel MoE layer: dispatch -> per-expert MLP -> combine.

Where the reference simulates the experts with ``x * (1 + rank)``
(``reference.py:262``), this layer runs a real two-matrix expert MLP on the rows
each local expert received, with the tcgen05 GEMM, and writes the results row
for row into the buffer the combine kernel pulls from.
"""
from __future__ import annotations

import torch

from ..ops.dispatch_combine import MoEAllToAll
from ..ops.gemm import gemm


class MoELayer:
    """``y[t] = sum_k w[t,k] * Expert_{e(t,k)}(x[t])``; expert ``e`` lives on rank
    ``e // (num_experts / world)``.  ``w_up[le]`` is ``[ffn, hidden]`` and
    ``w_down[le]`` is ``[hidden, ffn]`` for local expert ``le``."""

    def __init__(self, num_experts: int, topk: int, hidden: int, max_tokens: int, w_up: torch.Tensor, w_down: torch.Tensor,
                 group=None):
        self.a2a = MoEAllToAll(num_experts, topk, hidden, max_tokens, dtype=torch.bfloat16, group=group, device=w_up.device)
        if w_up.shape[0] != self.a2a.El or w_down.shape[0] != self.a2a.El:
            raise ValueError("need one weight pair per local expert")
        self.w_up, self.w_down = w_up.contiguous(), w_down.contiguous()

    def __call__(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        a2a = self.a2a
        if not x.is_cuda:
            return self._dense(x, indices, weights)
        counts, recv = a2a.dispatch(x, indices)
        y = a2a.expert_output_buffer()
        counts_h = counts.cpu()  # the segment lengths size the GEMMs (one sync per layer call)
        for s in range(a2a.world):
            off = 0
            for le in range(a2a.El):
                c = int(counts_h[s, le])
                if c:
                    h = gemm(recv[s, off:off + c], self.w_up[le])
                    h = torch.nn.functional.silu(h)
                    gemm(h, self.w_down[le], out=y[s, off:off + c])
                off += c
        return a2a.combine(x, indices, weights)

    def _dense(self, x, indices, weights) -> torch.Tensor:
        """Single-process fp32 formulation (CPU tests, world 1 only)."""
        out = torch.zeros_like(x, dtype=torch.float32)
        w_up, w_down = self.w_up.to(x.device), self.w_down.to(x.device)
        for t in range(x.shape[0]):
            for kk in range(indices.shape[1]):
                e = int(indices[t, kk])
                h = torch.nn.functional.silu((x[t].float() @ w_up[e].float().t()).to(torch.bfloat16)).float()
                out[t] += weights[t, kk] * (h @ w_down[e].float().t()).to(torch.bfloat16).float()
        return out.to(x.dtype)

    def close(self) -> None:
        if self.a2a.heap is not None:
            self.a2a.heap.close()
