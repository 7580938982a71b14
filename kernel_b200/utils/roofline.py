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


@dataclass
class Peaks:
    tflops: float = NOMINAL_BF16_TFLOPS
    nvlink_gbs: float = NOMINAL_NVLINK_GBS
    label: str = "nominal"


def measured_peaks(path="MEASURED_PEAKS.json", sustained: bool = False) -> Optional[Peaks]:
    p = Path(path)
    if not p.exists():
        return None
    d = json.loads(p.read_text())
    key = "bf16_tflops_sustained" if sustained else "bf16_tflops"
    return Peaks(tflops=float(d[key]), nvlink_gbs=MEASURED_NVLINK_GBS, label="measured" + ("-sustained" if sustained else ""))


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
    one_way = (world - 1) / world * tokens * topk * hidden * elem_bytes
    t = one_way / (peaks.nvlink_gbs * 1e9) * 1e6
    return {"compute_us": 0.0, "link_us": 2 * t, "roofline_us": 2 * t, "flops": 0.0, "link_bytes": 2 * one_way}
