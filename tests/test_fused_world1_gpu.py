"""Task-level paths on one GPU: generate_input -> custom_kernel -> check, for the
three tasks with world_size 1, plus the evaluator's single-GPU flow."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.mark.parametrize("m,n,k,bias", [(256, 512, 1024, True), (64, 2880, 360, True), (2048, 3696, 3696, False)])
def test_gemm_rs_world1(m, n, k, bias):
    from kernel_b200.tasks.gemm_rs import reference as R
    from kernel_b200.tasks.gemm_rs import submission as S

    data = R.generate_input(0, 1, m, n, k, bias, seed=1, dist="normal")
    out = S.custom_kernel(data)
    torch.cuda.synchronize()
    assert R.check_implementation(data, out) == (True, "")
    assert out.shape == (m, n)


@pytest.mark.parametrize("m,n,k,bias", [(256, 512, 1024, True), (1024, 3696, 2048, True)])
def test_ag_gemm_world1(m, n, k, bias):
    from kernel_b200.tasks.ag_gemm import reference as R
    from kernel_b200.tasks.ag_gemm import submission as S

    data = R.generate_input(0, 1, m, n, k, bias, seed=2)
    out = S.custom_kernel(data)
    torch.cuda.synchronize()
    assert R.check_implementation(data, out) == (True, "")


def test_all2all_world1_reference_compatible_mode():
    from kernel_b200.tasks.all2all import reference as R
    from kernel_b200.tasks.all2all import submission as S

    data = R.generate_input(64, 6, 2048, 32, seed=1234, rank=0, world_size=1)
    out = S.custom_kernel(data)
    torch.cuda.synchronize()
    assert R.check_implementation(data, out) == (True, "")
    assert torch.allclose(out.float(), R.ref_closed_form(data).float(), rtol=1e-2, atol=5e-3)
    S.release_contexts()


def test_evaluator_single_gpu_test_and_benchmark(tmp_path):
    tests = tmp_path / "t.txt"
    tests.write_text("m: 256; n: 512; k: 1024; has_bias: True; seed: 1; dist: normal\n"
                     "num_experts: 16; experts_per_token: 2; hidden_dim: 512; max_num_tokens: 32; seed: 2\n")
    r, w = os.pipe()
    env = dict(os.environ, POPCORN_FD=str(w), POPCORN_GPUS="1", PYTHONPATH=str(ROOT))
    for mode in ("test", "benchmark"):
        proc = subprocess.run([sys.executable, "-m", "kernel_b200.harness.eval", mode, str(tests)], env=env, pass_fds=(w,),
                              cwd=ROOT, capture_output=True, text=True, timeout=600)
        assert proc.returncode == 0, proc.stderr[-2000:]
    os.close(w)
    out = os.fdopen(r).read()
    assert out.count("check: pass") == 2 and "benchmark.1.mean" in out
