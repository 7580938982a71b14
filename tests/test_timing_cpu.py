"""Phase timer and the timed collective baseline (CPU, gloo)."""
import time

import torch

from kernel_b200.utils.timing import PhaseTimer, breakdown, format_summary

from _mp import run_ranks


def test_phase_timer_nests_and_accumulates():
    tm = PhaseTimer()
    for _ in range(3):
        with tm("dispatch_total"):
            with tm("dispatch_count_exchange"):
                time.sleep(0.002)
            with tm("dispatch_data_preparation"):
                time.sleep(0.001)
    s = tm.summary()
    assert s["dispatch_total"]["count"] == 3
    assert s["dispatch_total"]["min"] >= s["dispatch_count_exchange"]["min"]
    assert s["dispatch_total"]["total"] >= s["dispatch_count_exchange"]["total"] + s["dispatch_data_preparation"]["total"] - 1e-6
    b = breakdown(s)
    assert b["dispatch"]["communication"] == s["dispatch_count_exchange"]["total"]
    assert b["dispatch"]["computation"] == s["dispatch_data_preparation"]["total"]  # the enclosing total is not counted twice
    assert 0.0 < b["overall"]["communication_frac"] < 1.0
    text = format_summary(tm, rank=1)
    assert "rank 1" in text and "dispatch_count_exchange" in text and "overall" in text


def test_disabled_timer_records_nothing_and_reset():
    off = PhaseTimer(enabled=False)
    with off("x"):
        pass
    assert off.summary() == {}
    tm = PhaseTimer()
    with tm("combine_aggregation"):
        pass
    other = PhaseTimer()
    with other("combine_aggregation"):
        pass
    tm.merge(other)
    assert tm.summary()["combine_aggregation"]["count"] == 2
    tm.reset()
    assert tm.summary() == {}


def test_phase_recorded_when_body_raises():
    tm = PhaseTimer()
    try:
        with tm("expert_computation"):
            raise RuntimeError("boom")
    except RuntimeError:
        pass
    assert tm.summary()["expert_computation"]["count"] == 1


def _timed_baseline(rank, world):
    from kernel_b200.baseline import all2all as B
    from kernel_b200.tasks.all2all import reference as R

    data = R.generate_input(8, 2, 32, 12, 5, rank, world, dtype="fp32", fixed_tokens=True, device="cpu")
    for _ in range(2):
        out = B.custom_kernel_timed(data)
    ok, msg = R.check_implementation(data, out)
    plain = B.custom_kernel(data)
    s = B.timing_summary(reset=True)
    return bool(ok), msg, bool(torch.equal(plain, out)), sorted(s), s.get("dispatch_total", {}).get("count"), B.timing_summary()


def test_timed_baseline_gloo_world2():
    res = run_ranks(_timed_baseline, 2)
    for ok, msg, same, names, count, after in res:
        assert ok, msg
        assert same
        assert count == 2
        assert after == {}
        for n in ("dispatch_count_exchange", "dispatch_data_communication", "dispatch_meta_communication", "expert_computation",
                  "combine_count_exchange", "combine_data_communication", "combine_meta_communication", "combine_aggregation",
                  "combine_total", "dispatch_total"):
            assert n in names


def test_timed_submission_module_reports_periodically(capsys, monkeypatch):
    from kernel_b200.baseline import all2all_timed
    from kernel_b200.tasks.all2all import reference as R

    monkeypatch.setattr(all2all_timed, "_EVERY", 2)
    monkeypatch.setattr(all2all_timed, "_calls", 0)
    data = R.generate_input(4, 2, 16, 5, 3, 0, 1, dtype="fp32", fixed_tokens=True, device="cpu")
    out = all2all_timed.custom_kernel(data)
    assert "timing summary" not in capsys.readouterr().err
    all2all_timed.custom_kernel(data)
    assert "timing summary" in capsys.readouterr().err
    ok, msg = R.check_implementation(data, out)
    assert ok, msg
    all2all_timed._impl._timers.clear()  # nothing left for the exit handler to print
