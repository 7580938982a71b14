"""Roofline arithmetic for the three fused ops.

The target time of a fused compute + collective kernel is the slower of its
FLOPs at the GEMM peak and of the bytes that must cross NVLink at the link
bandwidth.  Peaks default to the B200 nominal figures and can be replaced by
measured ones (a JSON file with ``bf16_tflops`` / ``bf16_tflops_sustained``).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Optional

NOMINAL_BF16_TFLOPS = 2250.0
NOMINAL_NVLINK_GBS = 900.0   # per direction per GPU
MEASURED_NVLINK_GBS = 770.0  # peer copy, per direction
NOMINAL_HBM_GBS = 7700.0
PEAKS_FILE = "MEASURED_PEAKS.json"


@dataclass
class Peaks:
    tflops: float = NOMINAL_BF16_TFLOPS
    nvlink_gbs: float = NOMINAL_NVLINK_GBS
    label: str = "nominal"
    hbm_gbs: float = NOMINAL_HBM_GBS


def measured_peaks(path: Optional[str] = None, sustained: bool = False) -> Optional[Peaks]:
    """Peaks from a measurement file (``bf16_tflops``, ``bf16_tflops_sustained``,
    ``hbm_gbs``): ``path``, else ``$KB200_PEAKS_FILE``, else ``MEASURED_PEAKS.json``
    in the current directory or beside the package."""
    import os

    candidates = [path] if path else [os.environ.get("KB200_PEAKS_FILE"), PEAKS_FILE,
                                      str(Path(__file__).resolve().parents[2] / PEAKS_FILE)]
    for cand in candidates:
        if cand and Path(cand).exists():
            d = json.loads(Path(cand).read_text())
            key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
            return Peaks(tflops=float(d[key]), nvlink_gbs=MEASURED_NVLINK_GBS,
                         label="measured" + ("-sustained" if sustained else ""), hbm_gbs=float(d.get("hbm_gbs", NOMINAL_HBM_GBS)))
    return None


def gemm_rs_roofline_us(m: int, n: int, k: int, world: int, peaks: Peaks = Peaks()) -> dict:
    flops = 2.0 * m * n * (k / world)
    link_bytes = (world - 1) / world * m * n * 2  # bf16 partial tiles leaving each rank
    t_c = flops / (peaks.tflops * 1e12) * 1e6
    t_l = link_bytes / (peaks.nvlink_gbs * 1e9) * 1e6
    return {"compute_us": t_c, "link_us": t_l, "roofline_us": max(t_c, t_l), "flops": flops, "link_bytes": link_bytes}


def ag_gemm_roofline_us(m: int, n: int, k: int, world: int, peaks: Peaks = Peaks()) -> dict:
    flops = 2.0 * m * (n / world) * k
    link_bytes = (world - 1) / world * m * k * 2  # remote row blocks of A arriving at each rank
    t_c = flops / (peaks.tflops * 1e12) * 1e6
    t_l = link_bytes / (peaks.nvlink_gbs * 1e9) * 1e6
    return {"compute_us": t_c, "link_us": t_l, "roofline_us": max(t_c, t_l), "flops": flops, "link_bytes": link_bytes}


def a2a_roofline_us(tokens: int, topk: int, hidden: int, elem_bytes: int, world: int, peaks: Peaks = Peaks()) -> dict:
    """Link term: the rows that leave a rank and come back.  Memory term: the six
    passes over the rows (dispatch reads T rows and writes T*k, the expert reads and
    writes T*k, the combine reads T*k and writes T) at the memory bandwidth, which is
    what bounds the op on one GPU."""
    one_way = (world - 1) / world * tokens * topk * hidden * elem_bytes
    t = one_way / (peaks.nvlink_gbs * 1e9) * 1e6
    mem_bytes = (2 * tokens + 4 * tokens * topk) * hidden * elem_bytes
    t_m = mem_bytes / (peaks.hbm_gbs * 1e9) * 1e6
    return {"compute_us": 0.0, "link_us": 2 * t, "memory_us": t_m, "roofline_us": max(2 * t, t_m), "flops": 0.0,
            "link_bytes": 2 * one_way, "memory_bytes": mem_bytes}
