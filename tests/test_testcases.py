"""Tests-file grammar, task.yml loading, seed mixing and run statistics."""
import math
from pathlib import Path

import pytest

from kernel_b200.harness import testcases as tc
from kernel_b200.harness.stats import calculate_stats, should_stop

TASKS = Path(__file__).resolve().parents[1] / "kernel_b200" / "tasks"


def test_parse_line_types_and_bool_fix():
    case = tc.parse_line("world_size: 8; m: 64; n: 2880; k: 2880; has_bias: False; seed: 2035")
    assert case.args == {"world_size": 8, "m": 64, "n": 2880, "k": 2880, "has_bias": False, "seed": 2035}
    assert tc.parse_line("has_bias: True").args["has_bias"] is True
    assert tc.parse_line("dtype: bf16; x: -3").args == {"dtype": "bf16", "x": -3}


@pytest.mark.parametrize("bad", ["m 64", "m: 6.4", "m: 64; ; n: 3", "1m: 3"])
def test_parse_rejects_malformed(bad):
    with pytest.raises(tc.SpecError):
        tc.parse_line(bad)


def test_cantor_seed_mixing():
    assert tc.combine_seeds(0, 0) == 0
    assert tc.combine_seeds(3, 4) == 3 + (7 * 8) // 2
    cases = tc.parse_tests("m: 1; seed: 5\nm: 2", seed=1000)
    assert cases[0].args["seed"] == tc.combine_seeds(5, 1000) and "seed" not in cases[1].args
    assert tc.combine_seeds(5, 10**9) > 10**17  # large secret seed -> large seed


@pytest.mark.parametrize("task,n_tests,n_bench", [("all2all", 11, 10), ("gemm_rs", 13, 7), ("ag_gemm", 7, 5)])
def test_task_yaml_loads_and_round_trips(task, n_tests, n_bench):
    path = TASKS / task / "task.yml"
    tests = tc.cases_from_yaml(path, "tests")
    bench = tc.cases_from_yaml(path, "benchmarks")
    assert len(tests) == n_tests and len(bench) == n_bench
    for case in tests + bench:
        assert tc.parse_line(case.spec).args == case.args  # yaml -> tests-file line -> same dict
        assert case.args["world_size"] == 8


def test_reference_shapes_are_kept():
    rs = [c.args for c in tc.cases_from_yaml(TASKS / "gemm_rs" / "task.yml", "benchmarks")]
    assert {"world_size": 8, "m": 8192, "n": 8192, "k": 29568, "has_bias": False, "seed": 42} in rs
    a2a = [c.args for c in tc.cases_from_yaml(TASKS / "all2all" / "task.yml", "benchmarks")]
    assert {"num_experts": 256, "experts_per_token": 8, "hidden_dim": 7168, "max_num_tokens": 256, "seed": 4, "world_size": 8} in a2a


def test_stats_and_stop_rule():
    s = calculate_stats([100.0, 110.0, 90.0])
    assert s.runs == 3 and s.mean == 100.0 and s.best == 90.0 and s.worst == 110.0
    assert math.isclose(s.std, 10.0) and math.isclose(s.err, 10.0 / math.sqrt(3))
    assert calculate_stats([5.0]).std == 0.0
    assert not should_stop(calculate_stats([1.0, 1.0]), 1e9, 0)            # fewer than 3 runs
    assert should_stop(calculate_stats([100.0, 100.0, 100.0]), 1e9, 0)     # converged
    assert not should_stop(calculate_stats([100.0, 150.0, 50.0]), 1e9, 0)
    assert should_stop(calculate_stats([100.0, 150.0, 50.0]), 200.0, 0)    # time budget
    assert should_stop(calculate_stats([100.0, 150.0, 50.0]), 1e9, 121e9)  # wall clock
