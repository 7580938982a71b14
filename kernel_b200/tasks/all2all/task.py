"""Types of the MoE all-to-all task (counterpart of the reference's ``task.py:8-17``)."""
from typing import TYPE_CHECKING, TypedDict, TypeVar

import torch

if TYPE_CHECKING:
    from .reference import MoEConfig, RankTestData

input_t = TypeVar("input_t", bound=tuple["MoEConfig", "RankTestData", int, int])
output_t = TypeVar("output_t", bound=torch.Tensor)


class TestSpec(TypedDict, total=False):
    num_experts: int
    experts_per_token: int
    hidden_dim: int
    max_num_tokens: int
    seed: int
    world_size: int
    dtype: str
    fixed_tokens: bool
    weight_mode: str
    expert_scale: str
