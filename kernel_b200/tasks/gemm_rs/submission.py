"""``custom_kernel`` of the GEMM + reduce-scatter task: one fused sm_100a kernel.

Counterpart of the reference's ``gemm_rs/submission.py:5-29`` (``torch.matmul``,
bias add, ``reduce_scatter_tensor``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...ops.gemm import GemmRS
from . import task
from .task import input_t, output_t

_contexts: dict = {}


def _group():
    return dist.group.WORLD if dist.is_available() and dist.is_initialized() else None


def _group_key():
    g = _group()
    return id(g) if g is not None else None


def get_context(M: int, N: int, device: torch.device) -> GemmRS:
    key = (M, N, device.type, device.index, _group_key())
    ctx = _contexts.get(key)
    if ctx is None:
        ctx = GemmRS(M, N, device=device)
        ctx.process_group = _group()  # kept alive with the entry: the id in the key cannot be reused meanwhile
        _contexts[key] = ctx
    return ctx


def release_contexts(collective: bool = True) -> None:
    """Frees cached workspaces.  Collective for the contexts of the current process
    group (call before destroying it); contexts left over from an earlier group
    are freed locally.  ``collective=False`` frees everything locally (a process that
    is leaving while its peers may be gone)."""
    current = _group() if collective else object()
    for ctx in _contexts.values():
        for sub, _ in getattr(ctx, "_stream_state", {}).values():  # chunk-sized contexts of run_from_host
            if sub is not ctx and sub.heap is not None:
                sub.heap.close(collective=ctx.process_group is current)
        if ctx.heap is not None:
            ctx.heap.close(collective=ctx.process_group is current)
    _contexts.clear()


def custom_kernel(data: input_t) -> output_t:
    a, w, bias = data
    ctx = get_context(a.shape[0], w.shape[0], a.device)
    scale = float(ctx.world) if task.bias_mode_of(data) == "per_rank" else 1.0
    return ctx(a, w, bias, bias_scale=scale)
