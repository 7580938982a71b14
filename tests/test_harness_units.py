"""Small pieces of the evaluator that need no process group."""
import dataclasses

import torch

from kernel_b200.harness import eval as E
from kernel_b200.harness.testcases import TestCase


def test_guess_task_from_case_keys():
    assert E.guess_task({"num_experts": 8}) == "all2all"
    assert E.guess_task({"m": 1, "n": 2, "k": 3}) == "gemm_rs"
    assert E.guess_task({"m": 1, "op": "ag_gemm"}) == "ag_gemm"


def test_clone_data_descends_into_plain_objects_and_keeps_configs():
    class Bag:
        def __init__(self):
            self.x = torch.arange(4.0)
            self.n = 3

    @dataclasses.dataclass
    class Cfg:
        a: int = 1

    bag, cfg = Bag(), Cfg()
    data = (cfg, bag, [torch.ones(2)], {"t": torch.zeros(1)}, 7)
    out = E.clone_data(data, torch.device("cpu"))
    assert out[0] is cfg and out[4] == 7
    assert out[1] is not bag and out[1].n == 3 and torch.equal(out[1].x, bag.x) and out[1].x is not bag.x
    assert out[2][0] is not data[2][0] and out[3]["t"] is not data[3]["t"]
    out[1].x[0] = 99.0
    assert bag.x[0] == 0.0  # a real copy: the kernel cannot clobber the oracle's inputs


def test_case_args_strip_op_and_add_rank_and_device():
    case = TestCase(args={"m": 4, "op": "ag_gemm", "world_size": 2}, spec="")
    args = E._case_args(case, 1, torch.device("cpu"))
    assert args == {"m": 4, "world_size": 2, "rank": 1, "device": torch.device("cpu")}


def test_free_port_honours_master_port(monkeypatch):
    monkeypatch.setenv("MASTER_PORT", "23456")
    assert E.free_port() == 23456
    monkeypatch.delenv("MASTER_PORT")
    p = E.free_port()
    assert 1024 < p < 65536


def test_case_roofline_keys():
    assert abs(E.case_roofline_us("gemm_rs", {"m": 8192, "n": 8192, "k": 29568, "world_size": 8}) - 220.47) < 0.1
    assert abs(E.case_roofline_us("all2all", {"max_num_tokens": 256, "experts_per_token": 8, "hidden_dim": 7168, "world_size": 8,
                                               "dtype": "bf16"}) - 57.09) < 0.1
    assert E.case_roofline_us("gemm_rs", {"m": 1}) is None


def test_wrap_check_accepts_both_return_styles():
    class Old:
        @staticmethod
        def check_implementation(data, out):
            return ""  # old style: empty string means success

    class New:
        @staticmethod
        def check_implementation(data, out):
            return False, "mismatch"

    assert E.wrap_check(Old, None, None) == (True, "")
    assert E.wrap_check(New, None, None) == (False, "mismatch")


def test_cached_contexts_pin_their_process_group_and_stale_ones_close_locally(monkeypatch):
    """A cached context keeps its process-group object alive (so the id in the cache
    key cannot be reused by a later group) and, once that group is gone, is freed
    without a collective barrier."""
    import torch

    from kernel_b200.tasks.all2all import reference as R
    from kernel_b200.tasks.all2all import submission as S

    S.release_contexts()
    data = R.generate_input(4, 2, 16, 4, 1, 0, 1, dtype="fp32", fixed_tokens=True, device="cpu")
    ctx = S.get_context(data[0], 1, torch.device("cpu"))
    assert S.get_context(data[0], 1, torch.device("cpu")) is ctx            # cached
    assert hasattr(ctx, "process_group") and ctx.process_group is None      # no group in this process
    calls = []
    real_close = ctx.heap.close
    monkeypatch.setattr(ctx.heap, "close", lambda collective=True: (calls.append(collective), real_close(collective=collective)))
    ctx.process_group = object()                                            # as if created under a group that no longer exists
    S.release_contexts()
    assert calls == [False] and S._contexts == {}
    ctx2 = S.get_context(data[0], 1, torch.device("cpu"))
    assert ctx2 is not ctx
    calls2 = []
    real_close2 = ctx2.heap.close
    monkeypatch.setattr(ctx2.heap, "close", lambda collective=True: (calls2.append(collective), real_close2(collective=collective)))
    S.release_contexts()
    assert calls2 == [True]
