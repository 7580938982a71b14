"""Every routing of tiny MoE cases through both host-heap protocols (rows grouped
by expert with flag hand-offs; one row per destination rank with the flags inside
the data), against the closed form ``out[t] = x[t] * sum_k w[t,k] *
scale(expert(t,k))``: the slot arithmetic has no untested combination at these
sizes."""
import itertools

import pytest
import torch

from _mp import run_ranks


def _routings(E, k, T):
    per_token = list(itertools.permutations(range(E), k))      # ordered picks of k distinct experts
    return list(itertools.product(per_token, repeat=T))


def _exhaustive(rank, world, E, k, T):
    from kernel_b200.ops.dispatch_combine import SCALE_EXPERT, MoEAllToAll, expert_scale_vector

    H = 8
    ctx = MoEAllToAll(E, k, H, T, dtype=torch.float32, device="cpu")
    combos = _routings(E, k, T)
    scale = expert_scale_vector(E, world, SCALE_EXPERT)
    g = torch.Generator().manual_seed(rank)
    bad = 0
    for c in range(len(combos)):
        # every rank walks all combinations, each in its own order, so rank pairs see many joint routings
        mine = combos[(c * (2 * rank + 1) + 7 * rank) % len(combos)]
        idx = torch.tensor(mine, dtype=torch.int32).contiguous()
        x = torch.randn(T, H, generator=g)
        w = torch.rand(T, k, generator=g)
        out = ctx.dispatch_scale_combine(x, idx, w, SCALE_EXPERT)
        ref = x * (w * scale[idx.long()]).sum(1, keepdim=True)
        bad += int(not torch.allclose(out, ref, rtol=1e-5, atol=1e-6))
    ctx.heap.close()
    return bad, len(combos)


@pytest.mark.parametrize("low_latency", ["0", "1"])
def test_all_routings_two_ranks_two_tokens(low_latency):
    for E, k in ((2, 1), (2, 2), (4, 1), (4, 2)):
        for bad, n in run_ranks(_exhaustive, 2, E, k, 2, env={"KB200_A2A_LL": low_latency}):
            assert bad == 0, (E, k, bad, n)


@pytest.mark.parametrize("low_latency", ["0", "1"])
def test_all_routings_three_ranks_one_token(low_latency):
    for bad, n in run_ranks(_exhaustive, 3, 6, 2, 1, env={"KB200_A2A_LL": low_latency}):
        assert bad == 0 and n == 30
