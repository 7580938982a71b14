"""Types and the bias convention of the GEMM + reduce-scatter task
(counterpart of the reference's ``gemm_rs/task.py:4-14``).

Bias convention.  The reference adds the bias on every rank before the
reduce-scatter (``gemm_rs/reference.py:54-59``), so its result contains
``world_size * bias``.  ``per_rank`` reproduces that and is the default, so that a
submission written against the reference passes unchanged; ``once`` adds the bias
a single time.  The mode travels with the data: ``generate_input`` returns a
``GemmRSInput``, a 3-tuple ``(input, weight, bias)`` like the reference's that also
carries ``bias_mode``.  A plain tuple means the default, which the environment can
set with ``KB200_GEMM_RS_BIAS_MODE``; nothing is kept in process-wide state.
"""
import os
from typing import Optional, Tuple, TypedDict, TypeVar

import torch

input_t = TypeVar("input_t", bound=Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]])
output_t = TypeVar("output_t", bound=torch.Tensor)

BIAS_MODES = ("once", "per_rank")


def default_bias_mode() -> str:
    mode = os.environ.get("KB200_GEMM_RS_BIAS_MODE", "per_rank")
    if mode not in BIAS_MODES:
        raise ValueError(f"KB200_GEMM_RS_BIAS_MODE must be one of {BIAS_MODES}, got {mode!r}")
    return mode


class GemmRSInput(tuple):
    """``(input, weight, bias)`` plus the bias convention of this case."""

    def __new__(cls, items, bias_mode: Optional[str] = None):
        self = super().__new__(cls, items)
        if len(self) != 3:
            raise ValueError("GemmRSInput holds (input, weight, bias)")
        mode = bias_mode if bias_mode is not None else default_bias_mode()
        if mode not in BIAS_MODES:
            raise ValueError(f"bias_mode must be one of {BIAS_MODES}, got {mode!r}")
        self.bias_mode = mode
        return self

    def rebuilt(self, items):
        """The same case around other tensors (clones, tensors on another device)."""
        return GemmRSInput(items, self.bias_mode)


def bias_mode_of(data) -> str:
    """Bias convention of a data tuple; a plain tuple has the default."""
    return getattr(data, "bias_mode", None) or default_bias_mode()


class TestSpec(TypedDict, total=False):
    world_size: int
    m: int
    n: int
    k: int
    has_bias: bool
    seed: int
    dist: str
    bias_mode: str
