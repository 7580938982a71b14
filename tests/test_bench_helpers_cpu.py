"""Helpers of bench.py that need no GPU: the read-only clock sampler against a fake
NVML, the geometric mean, the refusal of a mismatching launch."""
import sys
import time
import types
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def _fake_nvml(clocks, powers_mw, mask):
    m = types.ModuleType("pynvml")
    state = {"i": 0, "calls": []}
    m.NVML_CLOCK_SM = 1
    m.nvmlInit = lambda: state["calls"].append("init")
    m.nvmlDeviceGetHandleByIndex = lambda i: ("handle", i)
    m.nvmlDeviceGetMaxClockInfo = lambda h, kind: 1965

    def clock(h, kind):
        state["i"] += 1
        return clocks[min(state["i"] - 1, len(clocks) - 1)]

    m.nvmlDeviceGetClockInfo = clock
    m.nvmlDeviceGetPowerUsage = lambda h: powers_mw[min(state["i"] - 1, len(powers_mw) - 1)]
    m.nvmlDeviceGetCurrentClocksEventReasons = lambda h: mask
    m._state = state
    return m


def test_clock_sampler_reads_only_and_reports_the_loaded_median(monkeypatch):
    import bench

    # idle at 1965 MHz / 150 W, then load at 1300 MHz / 900 W with the power cap active
    fake = _fake_nvml([1965] * 3 + [1300] * 50, [150_000] * 3 + [900_000] * 50, 0x4)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    s = bench.ClockSampler(0, period_s=0.001)
    s.start()
    time.sleep(0.08)
    out = s.stop()
    assert out["sm_max_mhz"] == 1965 and out["sm_mhz"] == 1300          # median of the samples taken under load
    assert out["sm_mhz_min"] == 1300 and out["power_w_max"] == 900.0
    assert out["reasons"] == ["sw_power_cap"] and out["samples"] >= 5
    # nothing but queries was called on the fake: the sampler has no way to change a setting
    assert set(n for n in dir(fake) if n.startswith("nvmlDevice")) == {
        "nvmlDeviceGetHandleByIndex", "nvmlDeviceGetMaxClockInfo", "nvmlDeviceGetClockInfo", "nvmlDeviceGetPowerUsage",
        "nvmlDeviceGetCurrentClocksEventReasons"}


def test_clock_sampler_window_falls_back_to_the_warm_up(monkeypatch):
    """A timed region shorter than three sampling periods is summarised together with
    its warm-up steps, not with whatever ran since the sampler started."""
    import bench

    fake = _fake_nvml([1965] * 10 + [1300] * 500, [150_000] * 10 + [900_000] * 500, 0x4)
    monkeypatch.setitem(sys.modules, "pynvml", fake)
    s = bench.ClockSampler(0, period_s=0.002)
    s.start()
    time.sleep(0.06)           # set-up: idle samples at the maximum clock
    s.mark(2)
    time.sleep(0.05)           # warm-up
    s.mark(0)
    s.mark(1)                  # a timed region without a single sample
    out = s.stop()
    assert out["samples"] >= 3 and out["sm_mhz_all_samples_median"] == 1300   # no idle sample in the summary


def test_clock_sampler_without_nvml(monkeypatch):
    import bench

    monkeypatch.setitem(sys.modules, "pynvml", None)     # import fails
    s = bench.ClockSampler(0)
    s.start()
    out = s.stop()
    assert out["sm_mhz"] is None and out["samples"] == 0 and out["reasons"] == []


def test_geomean_and_launch_check(monkeypatch):
    import bench

    assert abs(bench.geomean([1.0, 10.0, 100.0]) - 10.0) < 1e-9
    monkeypatch.setenv("WORLD_SIZE", "2")
    with pytest.raises(SystemExit) as e:
        bench.init_dist(4)
    assert "nproc-per-node 4" in str(e.value)
