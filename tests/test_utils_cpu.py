"""Shared utilities (comparison reports, seeding, context managers); counterpart of the reference's ``utils.py``."""
import random

import numpy as np
import torch

from kernel_b200.utils import common as U


def test_verbose_allclose_reports_and_bounds():
    exp = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    ok, lines = U.verbose_allclose(exp + 1e-7, exp)
    assert ok and lines[0].startswith("Maximum error")
    got = exp.clone()
    got[1, 0] += 1.0
    ok, lines = U.verbose_allclose(got, exp, rtol=1e-2, atol=1e-2)
    assert not ok and lines[0] == "Number of mismatched elements: 1" and "(1, 0)" in lines[1]
    assert U.verbose_allclose(exp[:1], exp) == (False, ["SIZE MISMATCH"])
    # the bound is relative to the expected value
    assert U.verbose_allclose(torch.tensor([101.0]), torch.tensor([100.0]), rtol=0.02, atol=0.0)[0]
    assert not U.verbose_allclose(torch.tensor([100.0]), torch.tensor([101.0]), rtol=0.0099, atol=0.0)[0]


def test_verbose_allclose_nan_and_inf_must_coincide():
    nan, inf = float("nan"), float("inf")
    assert U.verbose_allclose(torch.tensor([nan, inf, -inf, 1.0]), torch.tensor([nan, inf, -inf, 1.0]))[0]
    assert not U.verbose_allclose(torch.tensor([nan]), torch.tensor([1.0]))[0]
    assert not U.verbose_allclose(torch.tensor([inf]), torch.tensor([-inf]))[0]
    assert not U.verbose_allclose(torch.tensor([1.0]), torch.tensor([inf]))[0]


def test_report_is_truncated():
    ok, lines = U.verbose_allclose(torch.zeros(20), torch.ones(20), max_print=3)
    assert not ok and len(lines) == 1 + 3 + 1 and lines[-1] == "... and 17 more mismatched elements."


def test_verbose_allequal_and_match_reference():
    a = torch.arange(6).view(2, 3)
    assert U.verbose_allequal(a, a.clone()) == (True, [])
    b = a.clone()
    b[0, 2] = 9
    ok, lines = U.verbose_allequal(b, a)
    assert not ok and "(0, 2)" in lines[1]
    check = U.make_match_reference(lambda d: d * 2, rtol=1e-3, atol=1e-3)
    ok, msg = check(torch.ones(4), torch.full((4,), 2.0))
    assert ok and "Maximum error" in msg
    ok, msg = check(torch.ones(4), torch.zeros(4))
    assert not ok and "\\n" in msg and "\n" not in msg   # one log line: the separator is the two characters \ n


def test_set_seed_seeds_all_generators():
    U.set_seed(123)
    a = (random.random(), float(np.random.rand()), float(torch.rand(1)))
    U.set_seed(123)
    b = (random.random(), float(np.random.rand()), float(torch.rand(1)))
    assert a == b
    U.set_seed(2**40 + 5)   # numpy takes 32 bits


def test_cudnn_context_restores_settings_and_cpu_helpers():
    before = (torch.backends.cudnn.allow_tf32, torch.backends.cudnn.deterministic)
    with U.DisableCuDNNTF32():
        assert torch.backends.cudnn.allow_tf32 is False and torch.backends.cudnn.deterministic is True
    assert (torch.backends.cudnn.allow_tf32, torch.backends.cudnn.deterministic) == before
    assert U.get_device(use_cuda=False).type == "cpu"
    U.clear_l2_cache()   # a no-op without a GPU
