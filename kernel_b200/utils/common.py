"""Shared helpers of the harness and the task oracles.

Same public names and behaviour as the reference's ``utils.py`` (``set_seed``
``utils.py:8``, ``get_device`` ``:17``, ``verbose_allclose`` ``:31``,
``verbose_allequal`` ``:99``, ``match_reference`` ``:135``,
``make_match_reference`` ``:148``, ``DisableCuDNNTF32`` ``:155``,
``clear_l2_cache`` ``:169``), written for this code base: everything is
device-agnostic so the CPU/gloo tests can use it, and the L2 flush reuses one
buffer instead of allocating 256 MB per call.
"""
from __future__ import annotations

import random
from typing import Callable, List, Tuple

import numpy as np
import torch

_L2_FLUSH_BYTES = 256 << 20  # larger than B200's 126 MB L2
_flush_buffers: dict = {}


def set_seed(seed: int = 42) -> None:
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


def get_device(use_cuda: bool = True) -> torch.device:
    if use_cuda and torch.cuda.is_available():
        return torch.device("cuda")
    if use_cuda:
        print("No CUDA device found; using the CPU.")
    return torch.device("cpu")


def _describe(received: torch.Tensor, expected: torch.Tensor, bad: torch.Tensor, max_print: int) -> List[str]:
    count = int(bad.count_nonzero().item())
    lines = [f"Number of mismatched elements: {count}"]
    for index in torch.nonzero(bad)[:max_print]:
        i = tuple(index.tolist())
        lines.append(f"ERROR at {i}: {received[i]} {expected[i]}")
    if count > max_print:
        lines.append(f"... and {count - max_print} more mismatched elements.")
    return lines


@torch.no_grad()
def verbose_allclose(received: torch.Tensor, expected: torch.Tensor, rtol: float = 1e-5, atol: float = 1e-8,
                     max_print: int = 5) -> Tuple[bool, List[str]]:
    """``|received - expected| <= atol + rtol * |expected|`` with NaN/inf positions
    required to coincide; returns (ok, report lines)."""
    if received.shape != expected.shape:
        return False, ["SIZE MISMATCH"]
    r32, e32 = received.to(torch.float32), expected.to(torch.float32)
    diff = (r32 - e32).abs()
    bad = diff > (atol + rtol * e32.abs())
    bad |= torch.isnan(r32) ^ torch.isnan(e32)
    bad |= torch.isposinf(r32) ^ torch.isposinf(e32)
    bad |= torch.isneginf(r32) ^ torch.isneginf(e32)
    if bool(bad.any()):
        return False, _describe(received, expected, bad, max_print)
    finite = diff[torch.isfinite(diff)]
    return True, [f"Maximum error: {finite.max().item() if finite.numel() else 0.0}"]


@torch.no_grad()
def verbose_allequal(received: torch.Tensor, expected: torch.Tensor, max_print: int = 5) -> Tuple[bool, List[str]]:
    if received.shape != expected.shape:
        return False, ["SIZE MISMATCH"]
    bad = received != expected
    if bool(bad.any()):
        return False, _describe(received, expected, bad, max_print)
    return True, []


def match_reference(data, output, reference: Callable, rtol: float = 1e-5, atol: float = 1e-8) -> Tuple[bool, str]:
    good, lines = verbose_allclose(output, reference(data), rtol=rtol, atol=atol)
    return good, "\\n".join(lines)


def make_match_reference(reference: Callable, **kwargs) -> Callable:
    def check(data, output):
        return match_reference(data, output, reference=reference, **kwargs)

    return check


class DisableCuDNNTF32:
    """Context manager: cuDNN TF32 off and deterministic algorithms on."""

    def __enter__(self):
        self._saved = (torch.backends.cudnn.allow_tf32, torch.backends.cudnn.deterministic)
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cudnn.deterministic = True
        return self

    def __exit__(self, *exc):
        torch.backends.cudnn.allow_tf32, torch.backends.cudnn.deterministic = self._saved


def clear_l2_cache(device=None) -> None:
    """Overwrites a buffer larger than the L2 so the next kernel starts cold."""
    if not torch.cuda.is_available():
        return
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    buf = _flush_buffers.get(dev)
    if buf is None:
        buf = torch.empty(_L2_FLUSH_BYTES // 8, dtype=torch.int64, device=dev)
        _flush_buffers[dev] = buf
    buf.fill_(42)
