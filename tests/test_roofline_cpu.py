"""Roofline arithmetic against the hand-derived figures for the flagship shapes."""
import math

from kernel_b200.utils import roofline as rf


def test_gemm_rs_flagship_roofline():
    r = rf.gemm_rs_roofline_us(8192, 8192, 29568, 8)
    assert math.isclose(r["flops"], 4.961e11, rel_tol=1e-3)
    assert math.isclose(r["link_bytes"], 117.4e6, rel_tol=1e-3)
    assert math.isclose(r["compute_us"], 220.5, rel_tol=1e-3)
    assert math.isclose(r["link_us"], 130.5, rel_tol=1e-3)
    assert r["roofline_us"] == r["compute_us"]
    measured = rf.Peaks(1642.6, 770.0, "measured")
    assert math.isclose(rf.gemm_rs_roofline_us(8192, 8192, 29568, 8, measured)["compute_us"], 302.0, rel_tol=1e-3)


def test_ag_gemm_flagship_roofline():
    r = rf.ag_gemm_roofline_us(8192, 29568, 8192, 8)
    assert math.isclose(r["flops"], 4.961e11, rel_tol=1e-3)
    assert math.isclose(r["link_bytes"], 117.4e6, rel_tol=1e-3)
    assert math.isclose(r["roofline_us"], 220.5, rel_tol=1e-3)


def test_a2a_roofline_and_single_rank():
    r = rf.a2a_roofline_us(256, 8, 7168, 2, 8)
    assert math.isclose(r["link_bytes"], 2 * 25.69e6, rel_tol=1e-3)
    assert math.isclose(r["roofline_us"], 57.1, rel_tol=2e-3)
    one = rf.a2a_roofline_us(256, 8, 7168, 2, 1)
    assert one["link_us"] == 0.0  # nothing crosses a link on one rank: the six passes over the rows bound the op
    assert math.isclose(one["memory_bytes"], (2 * 256 + 4 * 2048) * 7168 * 2) and one["roofline_us"] == one["memory_us"] > 0


def test_small_gemm_is_link_bound():
    r = rf.gemm_rs_roofline_us(4096, 4096, 4096, 8)
    assert r["roofline_us"] == r["link_us"] > r["compute_us"]
