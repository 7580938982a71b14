"""Oracle of the GEMM + reduce-scatter task.

Contract of the reference's ``gemm_rs/reference.py`` (``generate_input`` ``:5-33``,
``ref_kernel`` ``:36-60``, ``check_implementation`` ``:63-71``) with the device as a
parameter and two input distributions:

* ``uniform``: input, weight and bias uniform in +-0.01 (the reference's draw);
* ``normal``:  input ~ N(0,1), weight ~ N(0,1)/sqrt(K), bias ~ N(0,0.02).

K is sharded: rank r holds ``input[M, K/world]`` and ``weight[N, K/world]``; the
result ``sum_r input_r @ weight_r^T`` is row-scattered, rank r keeps rows
``[r*M/world, (r+1)*M/world)``.  See ``task.py`` for the bias convention, which
travels with the data tuple.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from . import task
from .task import input_t, output_t

RTOL, ATOL = 1e-2, 1e-2  # gemm_rs/reference.py:67


def default_device(rank: int) -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", rank % torch.cuda.device_count())
    return torch.device("cpu")


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def generate_input(rank: int, world_size: int, m: int, n: int, k: int, has_bias: bool, seed: int,
                   dist: str = "uniform", bias_mode: Optional[str] = None, device=None) -> input_t:
    dev = torch.device(device) if device is not None else default_device(rank)
    if m % world_size or k % world_size:
        raise ValueError("m and k must be divisible by world_size")
    local_k = k // world_size
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + rank)
    if dist == "uniform":
        a = ((torch.rand((m, local_k), device=dev, generator=gen) * 2 - 1) * 0.01).to(torch.bfloat16)
        w = ((torch.rand((n, local_k), device=dev, generator=gen) * 2 - 1) * 0.01).to(torch.bfloat16)
    elif dist == "normal":
        a = torch.randn((m, local_k), device=dev, generator=gen).to(torch.bfloat16)
        w = (torch.randn((n, local_k), device=dev, generator=gen) / k ** 0.5).to(torch.bfloat16)
    else:
        raise ValueError(f"unknown dist {dist!r}")
    bias = None
    if has_bias:
        gen.manual_seed(seed)  # identical on every rank
        if dist == "uniform":
            bias = ((torch.rand((n,), device=dev, generator=gen) * 2 - 1) * 0.01).to(torch.bfloat16)
        else:
            bias = (torch.randn((n,), device=dev, generator=gen) * 0.02).to(torch.bfloat16)
    return task.GemmRSInput((a, w, bias), bias_mode)


def ref_kernel(data: input_t) -> output_t:
    """``matmul`` -> bias -> ``reduce_scatter_tensor``, i.e. the library path."""
    a, w, bias = data
    world = _world()
    M, N = a.shape[0], w.shape[0]
    if a.is_cuda:
        out = torch.matmul(a, w.t())
    else:
        out = (a.float() @ w.float().t()).to(torch.bfloat16)
    per_rank = task.bias_mode_of(data) == "per_rank"
    if bias is not None and per_rank:
        out = out + bias
    if world > 1:
        rs = torch.empty((M // world, N), dtype=out.dtype, device=a.device)
        dist.reduce_scatter_tensor(rs, out.contiguous())
    else:
        rs = out
    if bias is not None and not per_rank:
        rs = (rs.float() + bias.float()).to(rs.dtype)
    return rs


def ref_fp32(all_inputs, all_weights, bias, rank: int, bias_mode: str = "per_rank") -> torch.Tensor:
    """Collective-free fp32 oracle from every rank's shards (tests only)."""
    world = len(all_inputs)
    acc = sum(a.float() @ w.float().t() for a, w in zip(all_inputs, all_weights))
    if bias is not None:
        acc = acc + (world if bias_mode == "per_rank" else 1) * bias.float()
    rows = acc.shape[0] // world
    return acc[rank * rows:(rank + 1) * rows]


def ref_kernel_fp32(data: input_t, with_magnitude: bool = False):
    """Collective oracle with fp32 partial products and an fp32 reduction: the
    value both the fused kernel and the bf16 library path approximate.  With
    ``with_magnitude`` it also returns ``sum_r |partial_r| (+ |bias|)``, the scale
    of the rounding error of any summation of the partials."""
    a, w, bias = data
    world = _world()
    M, N = a.shape[0], w.shape[0]
    part = a.float() @ w.float().t()
    if world > 1:
        rs = torch.empty((M // world, N), dtype=torch.float32, device=a.device)
        dist.reduce_scatter_tensor(rs, part)
    else:
        rs = part
    mag = None
    if with_magnitude:
        if world > 1:
            mag = torch.empty_like(rs)
            dist.reduce_scatter_tensor(mag, part.abs())
        else:
            mag = part.abs()
    if bias is not None:
        scale = world if task.bias_mode_of(data) == "per_rank" else 1
        rs = rs + scale * bias.float()
        if mag is not None:
            mag = mag + scale * bias.float().abs()
    return (rs, mag) if with_magnitude else rs


MEAN_ERROR_FACTOR = 1.5  # allowed mean |error| relative to the bf16 library path's


def check_implementation(data: input_t, output: output_t):
    """Collective.  Two conditions against the fp32 oracle:

    * every element: ``|output - exact| <= atol + rtol * sum_r |partial_r|``;
    * on average: ``mean |output - exact| <= 1.5 * mean |ref_kernel - exact|`` (plus a
      floor of a thousandth of the mean magnitude), i.e. the implementation is not
      allowed to be noticeably less accurate than the bf16 library path.

    The reference compares with its bf16 library path at ``rtol = atol = 1e-2``
    relative to the result (``gemm_rs/reference.py:67``), which its own +-0.01
    inputs never stress.  With O(1) values every rank's partial is rounded to bf16
    before the sum, so the error of a correct implementation scales with the
    partials, not with the (possibly cancelling) result: measured against fp32 the
    library path misses the result-relative bound on tens of elements per rank.
    The element-wise bound used here is the standard forward-error bound of a
    summation with the same two constants; for one rank it is the reference's
    bound exactly.  It is loose for a single element, so the second condition
    guards the typical error: a wrong partial, a dropped tile or a bias applied
    with the wrong factor moves the mean error far beyond the library path's."""
    expected, magnitude = ref_kernel_fp32(data, with_magnitude=True)
    # The library path is a collective too: it runs before any rank can leave with a
    # verdict of its own, or the ranks whose shards pass would wait in it for a rank
    # that has already returned.
    library = (ref_kernel(data).float() - expected).abs().mean().item()
    if output.device != expected.device:
        return False, f"Output device mismatch: {output.device} != {expected.device}"
    if output.shape != expected.shape:
        return False, f"Output shape mismatch: {tuple(output.shape)} != {tuple(expected.shape)}"
    diff = (output.float() - expected).abs()
    bad = ~(diff <= ATOL + RTOL * magnitude)  # also catches NaN
    if bool(bad.any()):
        i = int(diff.argmax())
        return False, (f"Output values mismatch: {int(bad.sum())} of {bad.numel()} elements, max abs diff "
                       f"{diff.max().item():.5g} at flat index {i} (expected {expected.flatten()[i].item():.5g})")
    mine = diff.mean().item()
    floor = 1e-3 * expected.abs().mean().item()
    if not mine <= MEAN_ERROR_FACTOR * library + floor:
        return False, (f"Output less accurate than the library path: mean abs error {mine:.5g} against "
                       f"{library:.5g} (allowed {MEAN_ERROR_FACTOR} x + {floor:.3g})")
    return True, ""
