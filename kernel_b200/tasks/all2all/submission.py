"""``custom_kernel`` of the MoE all-to-all task: the fused sm_100a path.

Counterpart of the reference's ``submission.py:192-219``.  The symmetric
workspace is built once per (configuration, process group) and reused; a call
launches three kernels and performs no host synchronisation.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ...ops.dispatch_combine import MoEAllToAll
from .task import input_t, output_t

_contexts: dict = {}


def _group():
    return dist.group.WORLD if dist.is_available() and dist.is_initialized() else None


def _group_key():
    g = _group()
    return id(g) if g is not None else None


def get_context(cfg, world_size: int, device: torch.device) -> MoEAllToAll:
    key = (cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens, cfg.in_dtype, world_size,
           device.type, device.index, _group_key())
    ctx = _contexts.get(key)
    if ctx is None:
        ctx = MoEAllToAll(cfg.num_experts, cfg.experts_per_token, cfg.hidden_dim, cfg.max_num_tokens,
                          dtype=cfg.in_dtype, device=device)
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
        if ctx.heap is not None:
            ctx.heap.close(collective=ctx.process_group is current)
    _contexts.clear()


def custom_kernel(data: input_t) -> output_t:
    cfg, rank_data, rank, world_size = data
    ctx = get_context(cfg, world_size, rank_data.x.device)
    return ctx.dispatch_scale_combine(rank_data.x, rank_data.indices, rank_data.weights, cfg.expert_scale)
