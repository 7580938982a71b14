"""Expert-parallel MoE layer: dispatch -> per-expert MLP -> combine.

Where the reference simulates the experts with ``x * (1 + rank)``
(``reference.py:262``), this layer runs a real two-matrix expert MLP on the rows
each local expert received, with the tcgen05 GEMM, and writes the results row
for row into the buffer the combine kernel pulls from.  ``MoELayer`` is the
forward-only block over given weights; ``TrainableMoELayer`` owns parameters and
has a backward pass made of the same two exchange kernels.
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
        if not x.is_cuda and not a2a.host_heap:
            return self._dense(x, indices, weights)
        counts, recv = a2a.dispatch(x, indices)
        # the segment lengths size the GEMMs (one sync per layer call); the rows of
        # one expert, from all sources, are gathered into one block per expert
        rows_idx, n_e = _expert_major_rows(counts.cpu(), a2a.cap)
        rows_idx = rows_idx.to(x.device)
        X = recv.view(-1, a2a.H)[rows_idx]
        Y = torch.empty_like(X)
        o = 0
        for le, n in enumerate(n_e):
            if n:
                h = torch.nn.functional.silu(_gemm(X[o:o + n], self.w_up[le]))
                gemm(h, self.w_down[le], out=Y[o:o + n], pair=False)
            o += n
        a2a.expert_output_buffer().view(-1, a2a.H)[rows_idx] = Y
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


def _expert_major_rows(counts_h: torch.Tensor, cap: int):
    """Flat positions (``src * cap + row``) of all valid rows of a receive region,
    ordered by local expert and then by source, and the row count per expert.
    ``counts_h`` is the ``[world, El]`` count matrix on the host; the rows of one
    source are grouped by local expert in expert order."""
    c = counts_h.long()
    off = c.cumsum(1) - c                                              # first row of (src, expert) inside the source's region
    starts = (off + torch.arange(c.shape[0]).unsqueeze(1) * cap).t().reshape(-1)   # expert-major
    lens = c.t().reshape(-1)
    total = int(lens.sum())
    seg_first = lens.cumsum(0) - lens
    idx = torch.repeat_interleave(starts - seg_first, lens) + torch.arange(total)
    return idx, c.sum(0).tolist()


def _pad8_t(rows: torch.Tensor) -> torch.Tensor:
    """``rows[n, A]`` -> contiguous ``[A, n8]`` (n rounded up to a multiple of 8 with
    zero columns): the K-major operand layout of the GEMM kernel, whose K must be a
    multiple of 8."""
    n, A = rows.shape
    n8 = (n + 7) // 8 * 8
    out = rows.new_zeros((A, n8))
    out[:, :n] = rows.t()
    return out


def _gemm(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """GEMMs whose row or reduction count is a per-step token count: a fixed tile
    configuration instead of the per-shape tuning of ``gemm`` (which would time
    both configurations again for every new count)."""
    return gemm(a, b, pair=False)


class _MoEFn(torch.autograd.Function):
    """Expert-parallel MoE block with a backward pass built from the same two
    kernels: the gradient of combine is a dispatch (of ``dy``) and the gradient of
    dispatch is a combine (of the experts' input gradients, with unit weights).
    The routing weight of every received row, which the expert-side gradients
    need, travels through a second, small fp32 context as ``[weights | expert ids]``
    per token; the gradient of the routing weights comes back through the same
    context as one-hot rows."""

    @staticmethod
    def forward(ctx, x, weights, w_up, w_down, layer, indices):
        a2a = layer.a2a
        counts, recv = a2a.dispatch(x, indices)
        rows_idx_h, n_e = _expert_major_rows(counts.cpu(), a2a.cap)
        rows_idx = rows_idx_h.to(x.device)
        X = recv.view(-1, a2a.H)[rows_idx]                              # expert-major copy of the received rows
        pre = torch.empty((X.shape[0], w_up.shape[1]), dtype=x.dtype, device=x.device)
        Y = torch.empty_like(X)
        o = 0
        for le, n in enumerate(n_e):
            if n:
                pre[o:o + n] = _gemm(X[o:o + n], w_up[le])
                Y[o:o + n] = _gemm(torch.nn.functional.silu(pre[o:o + n]), w_down[le])
            o += n
        a2a.expert_output_buffer().view(-1, a2a.H)[rows_idx] = Y
        out = a2a.combine(x, indices, weights)
        ctx.layer, ctx.n_e = layer, n_e
        ctx.save_for_backward(indices, weights, w_up, w_down, X, pre, Y, rows_idx)
        return out

    @staticmethod
    def backward(ctx, dy):
        layer, n_e = ctx.layer, ctx.n_e
        indices, weights, w_up, w_down, X, pre, Y, rows_idx = ctx.saved_tensors
        a2a, meta = layer.a2a, layer.meta
        k, dev = a2a.k, dy.device
        dy = dy.contiguous()
        T = dy.shape[0]
        # routing info to the experts: [w_0..w_{k-1} | e_0..e_{k-1}] per token (expert ids are exact in fp32)
        info = torch.zeros((T, meta.H), dtype=torch.float32, device=dev)
        info[:, :k] = weights
        info[:, k:2 * k] = indices.float()
        _, recv_m = meta.dispatch(info, indices)
        M = recv_m.view(-1, meta.H)[rows_idx]
        _, recv_dy = a2a.dispatch(dy, indices)
        dYr = recv_dy.view(-1, a2a.H)[rows_idx]                         # dy of the row's token, unscaled
        row_expert = torch.repeat_interleave(torch.arange(len(n_e), device=dev), torch.tensor(n_e, device=dev)) + a2a.rank * a2a.El
        j = (M[:, k:2 * k] == row_expert.unsqueeze(1).float()).float().argmax(1)   # which of the token's k choices this row is
        w_row = M.gather(1, j.unsqueeze(1))                                        # its routing weight
        # d weights[t, j] = <dy[t], y_row>: returned as one-hot rows, summed over k by a unit-weight combine
        g = (dYr.float() * Y.float()).sum(1, keepdim=True)
        back = torch.zeros((M.shape[0], meta.H), dtype=torch.float32, device=dev)
        back.scatter_(1, j.unsqueeze(1), g)
        meta.expert_output_buffer().view(-1, meta.H)[rows_idx] = back
        ones = torch.ones((T, k), dtype=torch.float32, device=dev)
        dweights = meta.combine(info, indices, ones)[:, :k].contiguous()
        # expert backward on dY = w_row * dy
        dYs = (dYr.float() * w_row).to(dy.dtype)
        dX = torch.empty_like(X)
        dw_up, dw_down = torch.zeros_like(w_up), torch.zeros_like(w_down)
        o = 0
        for le, n in enumerate(n_e):
            if n:
                sl = slice(o, o + n)
                p32 = pre[sl].float()
                sig = torch.sigmoid(p32)
                h = (p32 * sig).to(dy.dtype)
                dw_down[le] = _gemm(_pad8_t(dYs[sl]), _pad8_t(h))                     # [H, F]
                dh = _gemm(dYs[sl], w_down[le].t().contiguous())                      # [n, F]
                dpre = (dh.float() * (sig * (1 + p32 * (1 - sig)))).to(dy.dtype)
                dw_up[le] = _gemm(_pad8_t(dpre), _pad8_t(X[sl]))                      # [F, H]
                dX[sl] = _gemm(dpre, w_up[le].t().contiguous())                       # [n, H]
            o += n
        a2a.expert_output_buffer().view(-1, a2a.H)[rows_idx] = dX
        dx = a2a.combine(dy, indices, ones)
        return dx, dweights, dw_up, dw_down, None, None


class TrainableMoELayer(torch.nn.Module):
    """``MoELayer`` with parameters and a backward pass (see ``_MoEFn``).  Gradients
    flow to the tokens, the routing weights and both expert matrices; every GEMM of
    both passes is the tcgen05 kernel and every exchange one of the two fused
    all-to-all kernels.  ``forward`` synchronises with the host once (the segment
    lengths size the GEMMs)."""

    def __init__(self, num_experts: int, topk: int, hidden: int, ffn: int, max_tokens: int, group=None, device=None):
        super().__init__()
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.a2a = MoEAllToAll(num_experts, topk, hidden, max_tokens, dtype=torch.bfloat16, group=group, device=dev)
        meta_hidden = max(64, (2 * topk + 63) // 64 * 64)   # 256-byte rows at least
        self.meta = MoEAllToAll(num_experts, topk, meta_hidden, max_tokens, dtype=torch.float32, group=group, device=dev)
        El = self.a2a.El
        self.w_up = torch.nn.Parameter(torch.empty(El, ffn, hidden, dtype=torch.bfloat16, device=dev))
        self.w_down = torch.nn.Parameter(torch.empty(El, hidden, ffn, dtype=torch.bfloat16, device=dev))
        torch.nn.init.normal_(self.w_up, std=hidden ** -0.5)
        torch.nn.init.normal_(self.w_down, std=ffn ** -0.5)

    def forward(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        return _MoEFn.apply(x, weights, self.w_up, self.w_down, self, indices)

    def close(self) -> None:
        for c in (self.a2a, self.meta):
            if c.heap is not None:
                c.heap.close()
