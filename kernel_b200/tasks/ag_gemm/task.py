"""Types of the all-gather + GEMM task.  The reference has no such task; the
contract mirrors its GEMM + reduce-scatter task (``gemm_rs/task.py:4-14``)."""
from typing import Optional, Tuple, TypedDict, TypeVar

import torch

input_t = TypeVar("input_t", bound=Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor]])
output_t = TypeVar("output_t", bound=torch.Tensor)


class TestSpec(TypedDict, total=False):
    world_size: int
    m: int
    n: int
    k: int
    has_bias: bool
    seed: int
    dist: str
