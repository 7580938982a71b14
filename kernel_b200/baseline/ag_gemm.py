"""All-gather + GEMM on NCCL and cuBLAS: the measured baseline.

``all_gather_into_tensor`` -> ``matmul`` -> bias, the library path the reference's
GEMM + reduce-scatter task would mirror (the reference has no such task).  As for
the other baseline the gathered operand lives in a buffer cached per shape and
the bias goes into the GEMM's epilogue (``torch.addmm``), so the comparison is
with the library path at its best, not with an allocation and an extra pass.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch
import torch.distributed as dist

_buffers: Dict[Tuple, torch.Tensor] = {}


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def release_contexts() -> None:
    _buffers.clear()


def custom_kernel(data):
    a_local, w, bias = data
    world = _world()
    rows, k = a_local.shape
    if world > 1:
        key = (rows, k, world, a_local.device.type, a_local.device.index, a_local.dtype)
        full = _buffers.get(key)
        if full is None:
            full = _buffers[key] = torch.empty((rows * world, k), dtype=a_local.dtype, device=a_local.device)
        dist.all_gather_into_tensor(full, a_local.contiguous())
    else:
        full = a_local
    if not full.is_cuda:
        out = full.float() @ w.float().t()
        if bias is not None:
            out = out + bias.float()
        return out.to(torch.bfloat16)
    if bias is not None:
        return torch.addmm(bias, full, w.t())
    return torch.matmul(full, w.t())
