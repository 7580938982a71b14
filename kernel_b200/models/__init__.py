"""Model-level blocks composed from the fused ops.

The reference ships no model; these blocks are the two places its ops occur in a
transformer: the sequence-parallel MLP (all-gather + GEMM on the way in, GEMM +
reduce-scatter on the way out) and the expert-parallel MoE layer (dispatch,
expert MLPs, combine).
"""
from .moe import MoELayer, TrainableMoELayer
from .tp_mlp import SequenceParallelMLP, TrainableSequenceParallelMLP

__all__ = ["MoELayer", "TrainableMoELayer", "SequenceParallelMLP", "TrainableSequenceParallelMLP"]
