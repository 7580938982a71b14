"""Types and the bias convention of the GEMM + reduce-scatter task
(counterpart of the reference's ``gemm_rs/task.py:4-14``).

Bias convention.  The reference adds the bias on every rank before the
reduce-scatter (``gemm_rs/reference.py:54-59``), so its result contains
``world_size * bias``.  ``per_rank`` reproduces that; ``once`` (default) adds the
bias a single time.  The mode is process-wide state of the task (the data tuple
keeps the reference's three elements); a test case may select it with the
``bias_mode`` key, the environment with ``KB200_GEMM_RS_BIAS_MODE``.
"""
import os
from typing import Optional, Tuple, TypedDict, TypeVar

import torch

input_t = TypeVar("input_t", bound=Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]])
output_t = TypeVar("output_t", bound=torch.Tensor)

_bias_mode = os.environ.get("KB200_GEMM_RS_BIAS_MODE", "once")


def set_bias_mode(mode: str) -> None:
    global _bias_mode
    if mode not in ("once", "per_rank"):
        raise ValueError(f"bias_mode must be 'once' or 'per_rank', got {mode!r}")
    _bias_mode = mode


def get_bias_mode() -> str:
    return _bias_mode


class TestSpec(TypedDict, total=False):
    world_size: int
    m: int
    n: int
    k: int
    has_bias: bool
    seed: int
    dist: str
    bias_mode: str
