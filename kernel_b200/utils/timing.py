"""Per-phase timing of host-driven pipelines (the collective baselines).

``PhaseTimer`` collects named, possibly nested phases.  On a CUDA device a phase
is bracketed by two events on the current stream and nothing is synchronised
until the numbers are read, so instrumenting a pipeline does not serialise it
(the reference's ``TimingContext``, all2all/submission_timed.py:9-33, calls
``torch.cuda.synchronize()`` at the end of every phase, which adds the host
round trip to every phase it measures).  On CPU tensors a phase is timed with
``time.perf_counter``.  ``summary()`` gives mean/min/max/total/count per phase in
milliseconds and ``format_summary()`` the dispatch/combine and
communication/computation breakdown of ``print_timing_summary``
(all2all/submission_timed.py:225-269).

The fused kernels are timed differently: they stamp ``globaltimer`` per phase on
the device (``MoEAllToAll.enable_trace`` / ``read_trace``).
"""
from __future__ import annotations

import contextlib
import time
from collections import defaultdict
from typing import Dict, Iterable, List, Optional

import torch

COMM_SUFFIXES = ("count_exchange", "data_communication", "meta_communication")


class PhaseTimer:
    def __init__(self, device: Optional[torch.device] = None, enabled: bool = True):
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.cuda = dev.type == "cuda" and torch.cuda.is_available()
        self.enabled = enabled
        self._pending: List[tuple] = []          # (name, start_event, end_event)
        self._ms: Dict[str, List[float]] = defaultdict(list)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            try:
                yield
            finally:
                e1.record()
                self._pending.append((name, e0, e1))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._ms[name].append((time.perf_counter() - t0) * 1e3)

    __call__ = phase

    def resolve(self) -> None:
        """Turns recorded event pairs into milliseconds (one synchronisation)."""
        if not self._pending:
            return
        self._pending[-1][2].synchronize()
        for name, e0, e1 in self._pending:
            e1.synchronize()
            self._ms[name].append(e0.elapsed_time(e1))
        self._pending.clear()

    def reset(self) -> None:
        self._pending.clear()
        self._ms.clear()

    def samples(self, name: str) -> List[float]:
        self.resolve()
        return list(self._ms.get(name, []))

    def summary(self) -> Dict[str, Dict[str, float]]:
        self.resolve()
        out = {}
        for name, vals in self._ms.items():
            if vals:
                out[name] = {"mean": sum(vals) / len(vals), "min": min(vals), "max": max(vals),
                             "total": sum(vals), "count": len(vals)}
        return out

    def merge(self, other: "PhaseTimer") -> None:
        other.resolve()
        for name, vals in other._ms.items():
            self._ms[name].extend(vals)


def _split(summary: Dict[str, Dict[str, float]], prefix: str):
    comm = comp = 0.0
    for name, st in summary.items():
        if not name.startswith(prefix + "_") or name == prefix + "_total":
            continue
        if name[len(prefix) + 1:] in COMM_SUFFIXES:
            comm += st["total"]
        else:
            comp += st["total"]
    return comm, comp


def breakdown(summary: Dict[str, Dict[str, float]], prefixes: Iterable[str] = ("dispatch", "combine")) -> Dict[str, Dict[str, float]]:
    """Communication / computation totals (ms) per prefix and overall.  A phase
    counts as communication when its name ends in one of ``COMM_SUFFIXES``; the
    ``<prefix>_total`` phase, which encloses the others, is left out."""
    out = {}
    tc = tp = 0.0
    for p in prefixes:
        comm, comp = _split(summary, p)
        out[p] = {"communication": comm, "computation": comp}
        tc, tp = tc + comm, tp + comp
    tot = tc + tp
    out["overall"] = {"communication": tc, "computation": tp,
                      "communication_frac": tc / tot if tot > 0 else 0.0}
    return out


def format_summary(timer: PhaseTimer, rank: int = 0) -> str:
    s = timer.summary()
    lines = [f"=== timing summary, rank {rank} ==="]
    for title, pref in (("DISPATCH", "dispatch"), ("EXPERT", "expert"), ("COMBINE", "combine")):
        names = sorted(n for n in s if n.startswith(pref))
        if not names:
            continue
        lines.append(f"{title}:")
        for n in names:
            st = s[n]
            lines.append(f"  {n:32s} {st['mean']:9.3f} ms  (min {st['min']:.3f}, max {st['max']:.3f}, n={st['count']})")
    b = breakdown(s)
    for p in ("dispatch", "combine"):
        lines.append(f"{p:8s} communication {b[p]['communication']:9.3f} ms   computation {b[p]['computation']:9.3f} ms")
    o = b["overall"]
    lines.append(f"overall  communication {o['communication']:9.3f} ms ({100 * o['communication_frac']:.1f} %)   "
                 f"computation {o['computation']:9.3f} ms")
    return "\n".join(lines)


def print_timing_summary(timer: PhaseTimer, rank: int = 0) -> None:
    print(format_summary(timer, rank), flush=True)
