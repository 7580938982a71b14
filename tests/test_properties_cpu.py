"""Property tests (hypothesis) of the host-side pieces with index arithmetic in them."""
import math

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from kernel_b200.harness.stats import calculate_stats
from kernel_b200.harness.testcases import combine_seeds, format_spec, parse_line
from kernel_b200.models.moe import _expert_major_rows, _pad8_t

KEY = st.text(alphabet="abcdefghijklmnopqrstuvwxyz_", min_size=1, max_size=12)
VALUE = st.one_of(st.integers(-10**9, 10**9), st.booleans(),
                  st.text(alphabet="abcdefghijklmnopqrstuvwxyz_", min_size=1, max_size=8).filter(lambda s: s not in ("True", "False")))


@given(st.dictionaries(KEY, VALUE, min_size=1, max_size=8))
def test_spec_line_round_trip(args):
    case = parse_line(format_spec(args))
    assert case.args == args
    assert all(type(case.args[k]) is type(v) for k, v in args.items())   # bools stay bools, ints stay ints


@given(st.integers(0, 2**31), st.integers(0, 2**31), st.integers(0, 2**31), st.integers(0, 2**31))
def test_seed_pairing_is_injective(a, b, c, d):
    if (a, b) != (c, d):
        assert combine_seeds(a, b) != combine_seeds(c, d)


@given(st.lists(st.floats(1.0, 1e9), min_size=2, max_size=50))
def test_stats_are_consistent(xs):
    s = calculate_stats(xs)
    assert s.runs == len(xs)
    assert s.best <= s.mean * (1 + 1e-12) and s.mean <= s.worst * (1 + 1e-12)
    assert math.isclose(s.err, s.std / math.sqrt(len(xs)), rel_tol=1e-9, abs_tol=1e-12)


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 5), st.integers(1, 6), st.data())
def test_expert_major_rows_is_a_permutation_of_the_valid_rows(world, El, data):
    cap = 12
    counts = torch.zeros(world, El, dtype=torch.int32)
    for s in range(world):   # any counts whose sum per source fits the capacity
        left = cap
        for le in range(El):
            c = data.draw(st.integers(0, left))
            counts[s, le] = c
            left -= c
    idx, n_e = _expert_major_rows(counts, cap)
    assert n_e == counts.sum(0).tolist()
    valid = sorted(s * cap + r for s in range(world) for r in range(int(counts[s].sum())))
    assert sorted(idx.tolist()) == valid
    # the expert of every listed row, read back from the layout, is non-decreasing and matches n_e
    bounds = counts.long().cumsum(1)
    experts = [int((bounds[p // cap] > (p % cap)).nonzero()[0]) for p in idx.tolist()]
    assert experts == sorted(experts)
    assert [experts.count(e) for e in range(El)] == n_e


@given(st.integers(1, 40), st.integers(1, 9))
def test_pad8_transpose(n, a):
    rows = torch.arange(n * a, dtype=torch.float32).view(n, a)
    t = _pad8_t(rows)
    assert t.shape == (a, (n + 7) // 8 * 8) and t.is_contiguous()
    assert torch.equal(t[:, :n], rows.t()) and bool((t[:, n:] == 0).all())
