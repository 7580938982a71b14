"""kernel_b200: Blackwell-native fused communication kernels and their harness.

Sub-packages: ``ops`` (front-ends of the sm_100a kernels), ``parallel`` (symmetric
memory), ``tasks`` (task specs, oracles, submissions), ``harness`` (evaluator),
``baseline`` (NCCL + cuBLAS paths), ``models`` (blocks built from the ops),
``utils`` (helpers, roofline, sweep, tracing), ``csrc`` (native sources + build).
"""

__version__ = "0.1.0"

__all__ = ["ops", "parallel", "tasks", "harness", "baseline", "models", "utils"]
