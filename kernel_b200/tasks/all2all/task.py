"""Types of the MoE all-to-all task.

The data of one rank is the tuple ``(cfg, rank_data, rank, world_size)`` and the
result a ``[num_tokens, hidden_dim]`` tensor, as in the reference's ``task.py:8-17``.
A test case is a mapping with the reference's five keys plus the options of
``reference.generate_input``; ``OPTION_DEFAULTS`` holds the values that reproduce
the reference's behaviour when a case does not mention them.
"""
from __future__ import annotations

from typing import TYPE_CHECKING, Tuple, TypedDict

import torch

if TYPE_CHECKING:  # the classes live next to the oracle
    from .reference import MoEConfig, RankTestData

input_t = Tuple["MoEConfig", "RankTestData", int, int]
output_t = torch.Tensor


class _Shape(TypedDict):
    """What every case names."""

    num_experts: int          # global expert count, divisible by the world size
    experts_per_token: int    # top-k
    hidden_dim: int
    max_num_tokens: int       # per-rank capacity; the token count is drawn below it unless fixed_tokens
    seed: int


class TestSpec(_Shape, total=False):
    """Optional keys: world size and the data options."""

    __test__ = False          # not a pytest class
    world_size: int
    dtype: str                # "fp16" (reference), "bf16", "fp32"
    fixed_tokens: bool        # every rank holds exactly max_num_tokens tokens
    weight_mode: str          # "uniform" (reference) or "softmax"
    expert_scale: str         # simulated expert: "rank" (reference: x * (1 + rank)), "expert", "identity"


OPTION_DEFAULTS = {"dtype": "fp16", "fixed_tokens": False, "weight_mode": "uniform", "expert_scale": "rank"}
