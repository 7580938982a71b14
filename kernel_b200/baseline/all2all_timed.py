"""Submission module that runs the collective MoE baseline with per-phase timing.

    POPCORN_FD=3 POPCORN_GPUS=8 python -m kernel_b200.harness.eval benchmark \
        --yaml kernel_b200/tasks/all2all/task.yml --submission kernel_b200.baseline.all2all_timed 3>&1

Every worker process prints its cumulative phase table to stderr every
``KB200_TIMING_EVERY`` calls (default 100) and when it exits normally (the role of
``print_timing_summary`` in the reference's ``all2all/submission_timed.py:225-269``,
which prints after every call).  Pool workers that are terminated run no exit
handlers, hence the periodic print.
"""
from __future__ import annotations

import atexit
import os
import sys

import torch.distributed as dist

from . import all2all as _impl
from ..utils.timing import format_summary

_EVERY = max(1, int(os.environ.get("KB200_TIMING_EVERY", "100")))
_calls = 0


def custom_kernel(data):
    global _calls
    out = _impl.custom_kernel_timed(data)
    _calls += 1
    if _calls % _EVERY == 0:
        _report()
    return out


def _report() -> None:
    for dev, tm in _impl._timers.items():
        if tm.summary():
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else os.environ.get("RANK", dev.index or 0)
            print(format_summary(tm, rank), file=sys.stderr, flush=True)


atexit.register(_report)
