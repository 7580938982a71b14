"""Run statistics of a benchmark (counterpart of ``eval.py:96-124`` in the reference)."""
from __future__ import annotations

import dataclasses
import math
from typing import Sequence


@dataclasses.dataclass
class Stats:
    runs: int
    mean: float
    std: float
    err: float
    best: float
    worst: float


def calculate_stats(durations_ns: Sequence[float]) -> Stats:
    """Mean, sample standard deviation (n-1), standard error and extremes of
    durations given in nanoseconds."""
    n = len(durations_ns)
    if n == 0:
        raise ValueError("no durations")
    mean = sum(durations_ns) / n
    if n > 1:
        std = math.sqrt(sum((d - mean) ** 2 for d in durations_ns) / (n - 1))
    else:
        std = 0.0
    return Stats(runs=n, mean=mean, std=std, err=std / math.sqrt(n), best=float(min(durations_ns)),
                 worst=float(max(durations_ns)))


def should_stop(stats: Stats, max_time_ns: float, wall_ns: float, wall_limit_ns: float = 120e9) -> bool:
    """Stop rule of the reference (``eval.py:298-306``): relative standard error
    below 0.1 %, or the measured time budget used up, or two minutes of wall clock."""
    if stats.runs < 3:
        return False
    return (stats.mean > 0 and stats.err / stats.mean < 0.001) or stats.mean * stats.runs > max_time_ns or wall_ns > wall_limit_ns
