"""The evaluator's command line, protocol and exit codes, on CPU/gloo ranks."""
import base64
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]

A2A = ("num_experts: 8; experts_per_token: 2; hidden_dim: 256; max_num_tokens: 64; seed: 5; world_size: 2; "
       "dtype: fp32; fixed_tokens: True; weight_mode: softmax; expert_scale: identity")
RS = "world_size: 2; m: 64; n: 128; k: 256; has_bias: False; seed: 3"
AG = "world_size: 2; m: 64; n: 128; k: 256; has_bias: True; seed: 3; op: ag_gemm"


def _run(args, tests_text, tmp_path, env_extra=None, with_fd=True):
    tests = tmp_path / "tests.txt"
    tests.write_text(tests_text)
    r, w = os.pipe()
    env = dict(os.environ, POPCORN_GPUS="2", PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1")
    env.pop("POPCORN_FD", None)
    env.pop("MASTER_PORT", None)
    if with_fd:
        env["POPCORN_FD"] = str(w)
    env.update(env_extra or {})
    argv = [sys.executable, "-m", "kernel_b200.harness.eval"] + [a if a != "@tests" else str(tests) for a in args]
    proc = subprocess.run(argv, env=env, pass_fds=(w,), cwd=ROOT, capture_output=True, text=True, timeout=600)
    os.close(w)
    with os.fdopen(r) as f:
        out = f.read()
    log = dict(line.split(": ", 1) for line in out.splitlines() if ": " in line)
    return proc.returncode, log, proc.stderr


def test_test_mode_passes_on_gloo(tmp_path):
    rc, log, err = _run(["test", "@tests", "--backend", "gloo"], "\n".join([A2A, RS, AG]) + "\n", tmp_path)
    assert rc == 0, err
    assert log["test-count"] == "3" and log["check"] == "pass"
    assert [log[f"test.{i}.status"] for i in range(3)] == ["pass"] * 3
    assert log["test.1.spec"] == RS


def test_baseline_impl_and_secret_seed(tmp_path):
    rc, log, err = _run(["test", "@tests", "--backend", "gloo", "--impl", "baseline"], A2A + "\n" + RS + "\n", tmp_path,
                        env_extra={"POPCORN_SEED": "987654321"})
    assert rc == 0, err
    assert log["check"] == "pass"


def test_benchmark_mode_reports_stats(tmp_path):
    rc, log, err = _run(["benchmark", "@tests", "--backend", "gloo"], RS + "\n", tmp_path)
    assert rc == 0, err
    assert log["benchmark-count"] == "1" and log["check"] == "pass"
    for key in ("runs", "mean", "std", "err", "best", "worst", "max_rank_us"):
        assert f"benchmark.0.{key}" in log
    assert 3 <= int(log["benchmark.0.runs"]) <= 100
    assert float(log["benchmark.0.best"]) <= float(log["benchmark.0.mean"]) <= float(log["benchmark.0.worst"])


def test_profile_mode_is_distributed_aware(tmp_path):
    rc, log, err = _run(["profile", "@tests", "--backend", "gloo"], RS + "\n", tmp_path)
    assert rc == 0, err
    table = base64.b64decode(log["benchmark.0.report"], b"+*").decode()
    assert "Self CPU" in table


def test_exit_codes(tmp_path):
    assert _run(["test", "@tests"], RS + "\n", tmp_path, with_fd=False)[0] == 111      # no POPCORN_FD
    assert _run(["test"], RS + "\n", tmp_path)[0] == 2                                  # missing tests file
    assert _run(["frobnicate", "@tests"], RS + "\n", tmp_path)[0] == 2                  # unknown mode
    assert _run(["test", "@tests", "--backend", "gloo"], "m 64\n", tmp_path)[0] == 113  # malformed case
    assert _run(["test", str(tmp_path / "missing.txt")], "", tmp_path)[0] == 113        # unreadable file


def test_world_larger_than_pool_fails_fast(tmp_path):
    rc, log, err = _run(["test", "@tests", "--backend", "gloo"], RS.replace("world_size: 2", "world_size: 4") + "\n", tmp_path)
    assert rc == 112
    assert log["test.0.status"] == "fail" and "exceeds" in log["test.0.error"]


def test_wrong_submission_is_reported(tmp_path):
    (tmp_path / "wrong_sub.py").write_text(
        "from kernel_b200.tasks.gemm_rs.submission import custom_kernel as good\n"
        "def custom_kernel(data):\n    return good(data) + 1.0\n")
    case = "world_size: 2; m: 64; n: 128; k: 256; has_bias: True; seed: 3; dist: normal"
    rc, log, err = _run(["test", "@tests", "--backend", "gloo", "--submission", "wrong_sub"], case + "\n", tmp_path,
                        env_extra={"PYTHONPATH": f"{ROOT}:{tmp_path}"})
    assert rc == 112 and log["check"] == "fail" and "mismatch" in log["test.0.error"]
    assert "rank 0" in log["test.0.error"]


def test_yaml_input_with_world_override(tmp_path):
    yml = tmp_path / "task.yml"
    yml.write_text('tests:\n  - {"world_size": 8, "m": 64, "n": 128, "k": 256, "has_bias": True, "seed": 1}\n')
    rc, log, err = _run(["test", "--yaml", str(yml), "--world", "2", "--backend", "gloo", "--task", "gemm_rs"], "", tmp_path)
    assert rc == 0, err
    assert log["check"] == "pass"


def test_leaderboard_mode_rechecks_with_fresh_seeds(tmp_path):
    rc, log, err = _run(["leaderboard", "@tests", "--backend", "gloo"], RS + "\n", tmp_path)
    assert rc == 0, err
    assert log["benchmark-count"] == "1" and log["check"] == "pass"
    assert int(log["benchmark.0.runs"]) >= 3


def test_leaderboard_mode_reports_failure_exit_code(tmp_path):
    (tmp_path / "wrong_sub2.py").write_text(
        "from kernel_b200.tasks.gemm_rs.submission import custom_kernel as good\n"
        "def custom_kernel(data):\n    return good(data) * 0\n")
    case = "world_size: 2; m: 64; n: 128; k: 256; has_bias: True; seed: 3; dist: normal"
    rc, log, err = _run(["leaderboard", "@tests", "--backend", "gloo", "--submission", "wrong_sub2"], case + "\n", tmp_path,
                        env_extra={"PYTHONPATH": f"{ROOT}:{tmp_path}"})
    assert rc == 112 and log["check"] == "fail"  # the reference falls off main() here and exits 0


def test_benchmark_extra_keys_baseline_and_json(tmp_path):
    import json

    out = tmp_path / "rows.json"
    rc, log, err = _run(["benchmark", "@tests", "--backend", "gloo", "--with-baseline", "--json", str(out)], RS + "\n" + A2A + "\n",
                        tmp_path)
    assert rc == 0, err
    for i in range(2):
        for key in ("max_rank_us", "roofline_us", "roofline_frac", "baseline_us", "speedup"):
            assert f"benchmark.{i}.{key}" in log, (i, key)
    rows = json.loads(out.read_text())
    assert len(rows) == 2 and rows[0]["spec"] == RS and rows[0]["speedup"] > 0
    # gemm_rs 64 x 128 x 256 on two ranks: link term 64*128*2/2 bytes at 900 GB/s
    assert abs(rows[0]["roofline_us"] - 64 * 128 * 2 / 2 / 900e9 * 1e6) < 1e-6


def test_submission_given_as_a_file_path(tmp_path):
    """A submission file next to nothing in particular, named by path (not importable by name)."""
    sub = tmp_path / "my submission.py"   # a name no import statement could spell
    sub.write_text("from kernel_b200.tasks.gemm_rs.submission import custom_kernel\n")
    rc, log, err = _run(["test", "@tests", "--backend", "gloo", "--submission", str(sub)], RS + "\n", tmp_path)
    assert rc == 0, err
    assert log["check"] == "pass"
    rc, log, err = _run(["test", "@tests", "--backend", "gloo", "--submission", str(tmp_path / "absent.py")], RS + "\n", tmp_path)
    assert rc == 112 and "not found" in log["test.0.error"]


def test_a_case_that_runs_out_of_time_does_not_block_the_next_one(tmp_path):
    """The first case never returns on rank 1; its workers are terminated and
    replaced, so the second case still runs (and passes) in fresh processes."""
    (tmp_path / "stuck_sub.py").write_text(
        "import time\n"
        "import torch.distributed as dist\n"
        "from kernel_b200.tasks.gemm_rs.submission import custom_kernel as good\n"
        "def custom_kernel(data):\n"
        "    if data[0].shape[0] == 128 and dist.get_rank() == 1:\n"
        "        time.sleep(600)\n"
        "    return good(data)\n")
    stuck = "world_size: 2; m: 128; n: 128; k: 256; has_bias: False; seed: 3"
    rc, log, err = _run(["test", "@tests", "--backend", "gloo", "--submission", "stuck_sub"], stuck + "\n" + RS + "\n", tmp_path,
                        env_extra={"PYTHONPATH": f"{ROOT}:{tmp_path}", "KB200_EVAL_TEST_TIMEOUT_S": "15",
                                   "KB200_EVAL_KILL_GRACE_S": "5", "KB200_EVAL_SETTLE_S": "0.2",
                                   "KB200_WAIT_LIMIT_MS": "3000"})
    assert rc == 112 and log["check"] == "fail"
    assert log["test.0.status"] == "fail" and "timed out" in log["test.0.error"]
    assert log["test.1.status"] == "pass"


def test_a_rank_that_raises_a_native_error_is_reported_and_the_next_case_runs(tmp_path):
    """Rank 1 raises the native library's error type inside the first case.  The
    error comes back as text (its object would not survive unpickling by default
    and would stop the pool's result thread), rank 0, left alone in a collective,
    is given a short grace period and replaced, and the second case passes."""
    import time

    (tmp_path / "raising_sub.py").write_text(
        "import torch.distributed as dist\n"
        "from kernel_b200 import _native as N\n"
        "from kernel_b200.tasks.gemm_rs.submission import custom_kernel as good\n"
        "def custom_kernel(data):\n"
        "    if data[0].shape[0] == 128 and dist.get_rank() == 1:\n"
        "        raise N.NativeError(N.KB_ERR_ARG, 'made up for the test')\n"
        "    return good(data)\n")
    bad = "world_size: 2; m: 128; n: 128; k: 256; has_bias: False; seed: 3"
    t0 = time.monotonic()
    rc, log, err = _run(["test", "@tests", "--backend", "gloo", "--submission", "raising_sub"], bad + "\n" + RS + "\n", tmp_path,
                        env_extra={"PYTHONPATH": f"{ROOT}:{tmp_path}", "KB200_EVAL_TEST_TIMEOUT_S": "300",
                                   "KB200_EVAL_FAIL_GRACE_S": "5", "KB200_WAIT_LIMIT_MS": "3000"})
    assert time.monotonic() - t0 < 200          # not the 300 s limit of a silent rank
    assert rc == 112 and log["check"] == "fail"
    report = "\n".join(f"{k}: {v}" for k, v in log.items())  # the error has one line per rank
    assert "rank 1 - NativeError" in report and "made up for the test" in report
    assert log["test.1.status"] == "pass"


def test_native_errors_survive_pickling():
    import pickle

    from kernel_b200 import _native as N

    for exc in (N.NativeError(N.KB_ERR_ARG, "bad argument"), N.SymmTimeoutError(N.KB_ERR_TIMEOUT, "late peer")):
        twin = pickle.loads(pickle.dumps(exc))
        assert type(twin) is type(exc) and twin.code == exc.code and str(twin) == str(exc)


def test_sigterm_takes_the_workers_along(tmp_path):
    """An evaluator that is told to stop (a caller's time limit sends SIGTERM)
    terminates its pool: no worker is left holding a rendezvous or a device."""
    import signal
    import time

    import psutil

    (tmp_path / "sleepy_sub.py").write_text(
        "import time\n"
        "def custom_kernel(data):\n"
        "    time.sleep(600)\n")
    tests = tmp_path / "tests.txt"
    tests.write_text(RS + "\n")
    r, w = os.pipe()
    env = dict(os.environ, POPCORN_GPUS="2", PYTHONPATH=f"{ROOT}:{tmp_path}", OMP_NUM_THREADS="1", POPCORN_FD=str(w))
    env.pop("MASTER_PORT", None)
    proc = subprocess.Popen([sys.executable, "-m", "kernel_b200.harness.eval", "test", str(tests), "--backend", "gloo",
                             "--submission", "sleepy_sub"], env=env, pass_fds=(w,), cwd=ROOT,
                            stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    os.close(w)
    try:
        parent = psutil.Process(proc.pid)
        deadline = time.monotonic() + 120
        workers = []
        while time.monotonic() < deadline:  # wait until the ranks are inside the submission
            workers = [c for c in parent.children(recursive=True) if "resource_tracker" not in " ".join(c.cmdline())]
            if len(workers) >= 2 and all(c.cpu_times().user > 0.5 for c in workers):
                break
            time.sleep(0.5)
        assert len(workers) >= 2
        time.sleep(3)
        proc.send_signal(signal.SIGTERM)
        proc.wait(timeout=60)
        gone, alive = psutil.wait_procs(workers, timeout=30)
        assert not alive
    finally:
        if proc.poll() is None:
            proc.kill()
        os.close(r)


def test_a_rank_keeps_its_worker_process_from_case_to_case(tmp_path):
    """Rank r of every case runs in worker r (one process per GPU for the whole run)."""
    (tmp_path / "pid_sub.py").write_text(
        "import os\n"
        "import torch.distributed as dist\n"
        "from kernel_b200.tasks.gemm_rs.submission import custom_kernel as good\n"
        "def custom_kernel(data):\n"
        "    with open(os.environ['PID_LOG'], 'a') as f:\n"
        "        f.write(f'{dist.get_rank()} {os.getpid()}\\n')\n"
        "    return good(data)\n")
    log_path = tmp_path / "pids.txt"
    cases = "\n".join(f"world_size: 2; m: 64; n: 128; k: 256; has_bias: False; seed: {s}" for s in (3, 4, 5)) + "\n"
    rc, log, err = _run(["test", "@tests", "--backend", "gloo", "--submission", "pid_sub"], cases, tmp_path,
                        env_extra={"PYTHONPATH": f"{ROOT}:{tmp_path}", "PID_LOG": str(log_path)})
    assert rc == 0, err
    pids = {0: set(), 1: set()}
    for line in log_path.read_text().split("\n"):
        if line:
            r, pid = line.split()
            pids[int(r)].add(pid)
    assert len(pids[0]) == 1 and len(pids[1]) == 1 and pids[0] != pids[1]


def test_benchmark_mode_reports_a_raising_rank_as_text(tmp_path):
    """Same as the test-mode case above, through the timed loop: the rank that raises
    leaves the others in the loop's barrier; the case is reported as failed with the
    error's text and the evaluator does not wait for its full time limit."""
    import time

    (tmp_path / "raising_sub2.py").write_text(
        "import torch.distributed as dist\n"
        "from kernel_b200 import _native as N\n"
        "from kernel_b200.tasks.gemm_rs.submission import custom_kernel as good\n"
        "calls = 0\n"
        "def custom_kernel(data):\n"
        "    global calls\n"
        "    calls += 1\n"
        "    if calls >= 3 and dist.get_rank() == 1:\n"
        "        raise N.SymmTimeoutError(N.KB_ERR_TIMEOUT, 'made up for the test')\n"
        "    return good(data)\n")
    t0 = time.monotonic()
    rc, log, err = _run(["benchmark", "@tests", "--backend", "gloo", "--submission", "raising_sub2"], RS + "\n", tmp_path,
                        env_extra={"PYTHONPATH": f"{ROOT}:{tmp_path}", "KB200_EVAL_BENCH_TIMEOUT_S": "300",
                                   "KB200_EVAL_FAIL_GRACE_S": "5", "KB200_WAIT_LIMIT_MS": "3000"})
    assert time.monotonic() - t0 < 200
    report = "\n".join(f"{k}: {v}" for k, v in log.items())
    assert rc == 112 and log["check"] == "fail"
    assert "SymmTimeoutError" in report and "made up for the test" in report


def test_replaced_workers_free_their_workspaces_before_they_leave(tmp_path):
    """Rank 1 holds a workspace and never returns.  When the case runs out of time the
    evaluator sends SIGTERM to all workers; the one that can still run Python frees
    its workspace locally (no collective) before it exits, the one blocked inside a
    collective is killed after the grace period; the next case runs in fresh workers."""
    (tmp_path / "holding_sub.py").write_text(
        "import time\n"
        "import torch.distributed as dist\n"
        "from kernel_b200.tasks.gemm_rs.submission import custom_kernel as good\n"
        "def custom_kernel(data):\n"
        "    out = good(data)\n"
        "    if data[0].shape[0] == 128 and dist.get_rank() == 1:\n"
        "        time.sleep(600)\n"
        "    return out\n")
    log_path = tmp_path / "lifecycle.txt"
    stuck = "world_size: 2; m: 128; n: 128; k: 256; has_bias: False; seed: 3"
    rc, log, err = _run(["test", "@tests", "--backend", "gloo", "--submission", "holding_sub"], stuck + "\n" + RS + "\n", tmp_path,
                        env_extra={"PYTHONPATH": f"{ROOT}:{tmp_path}", "KB200_EVAL_TEST_TIMEOUT_S": "15",
                                   "KB200_EVAL_KILL_GRACE_S": "6", "KB200_EVAL_SETTLE_S": "0.2",
                                   "KB200_EVAL_LIFECYCLE_LOG": str(log_path), "KB200_WAIT_LIMIT_MS": "3000"})
    assert rc == 112 and log["test.0.status"] == "fail" and "timed out" in log["test.0.error"]
    assert log["test.1.status"] == "pass"
    assert "1 workspace(s) freed" in log_path.read_text()
