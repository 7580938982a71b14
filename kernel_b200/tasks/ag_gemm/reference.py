"""Oracle of the all-gather + GEMM task (no counterpart in the reference; the
contract is the mirror image of ``gemm_rs/reference.py``).

M is sharded on input, N on the weights: rank r holds ``a_local[M/world, K]``,
``w_local[N/world, K]`` and ``bias[N/world]``; the result is
``all_gather(a_local) @ w_local^T (+ bias)`` of shape ``[M, N/world]``.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .task import input_t, output_t

RTOL, ATOL = 1e-2, 1e-2


def default_device(rank: int) -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", rank % torch.cuda.device_count())
    return torch.device("cpu")


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def generate_input(rank: int, world_size: int, m: int, n: int, k: int, has_bias: bool, seed: int,
                   dist: str = "normal", device=None) -> input_t:
    dev = torch.device(device) if device is not None else default_device(rank)
    if m % world_size or n % world_size:
        raise ValueError("m and n must be divisible by world_size")
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + rank)
    lm, ln = m // world_size, n // world_size
    if dist == "normal":
        a = torch.randn((lm, k), device=dev, generator=gen).to(torch.bfloat16)
        w = (torch.randn((ln, k), device=dev, generator=gen) / k ** 0.5).to(torch.bfloat16)
        bias = (torch.randn((ln,), device=dev, generator=gen) * 0.02).to(torch.bfloat16) if has_bias else None
    elif dist == "uniform":
        a = ((torch.rand((lm, k), device=dev, generator=gen) * 2 - 1) * 0.01).to(torch.bfloat16)
        w = ((torch.rand((ln, k), device=dev, generator=gen) * 2 - 1) * 0.01).to(torch.bfloat16)
        bias = ((torch.rand((ln,), device=dev, generator=gen) * 2 - 1) * 0.01).to(torch.bfloat16) if has_bias else None
    else:
        raise ValueError(f"unknown dist {dist!r}")
    return a, w, bias


def ref_kernel(data: input_t) -> output_t:
    """``all_gather_into_tensor`` -> ``matmul`` -> bias, i.e. the library path."""
    a_local, w, bias = data
    world = _world()
    if world > 1:
        a = torch.empty((a_local.shape[0] * world, a_local.shape[1]), dtype=a_local.dtype, device=a_local.device)
        dist.all_gather_into_tensor(a, a_local.contiguous())
    else:
        a = a_local
    if a.is_cuda:
        out = torch.matmul(a, w.t())
        if bias is not None:
            out = out + bias
        return out
    out = a.float() @ w.float().t()
    if bias is not None:
        out = out + bias.float()
    return out.to(torch.bfloat16)


def ref_kernel_fp32(data: input_t) -> torch.Tensor:
    """Collective oracle computed in fp32."""
    a_local, w, bias = data
    world = _world()
    if world > 1:
        a = torch.empty((a_local.shape[0] * world, a_local.shape[1]), dtype=a_local.dtype, device=a_local.device)
        dist.all_gather_into_tensor(a, a_local.contiguous())
    else:
        a = a_local
    out = a.float() @ w.float().t()
    if bias is not None:
        out = out + bias.float()
    return out


def check_implementation(data: input_t, output: output_t):
    expected = ref_kernel_fp32(data)
    if output.device != expected.device:
        return False, f"Output device mismatch: {output.device} != {expected.device}"
    if output.shape != expected.shape:
        return False, f"Output shape mismatch: {tuple(output.shape)} != {tuple(expected.shape)}"
    if not torch.allclose(output.float(), expected.float(), rtol=RTOL, atol=ATOL):
        diff = (output.float() - expected.float()).abs()
        return False, f"Output values mismatch: max abs diff {diff.max().item():.5g}"
    return True, ""
