"""The low-latency MoE protocol (flags inside the data) on CPU ranks over the host
heap: the same wire format, landing areas and slot arithmetic as the kernel
(``csrc/kernels/a2a_ll.cuh``; host twin ``csrc/symm/a2a_ll_host.cpp``)."""
import pytest
import torch

from _mp import run_ranks


def _sparse_calls(rank, world, low_latency, dtype_name):
    """Many calls on one workspace with a fresh token count and routing every call and
    one expert per token (k = 1, one expert per rank): most peers get no row from
    this rank, so ranks run ahead of each other as far as the protocol allows and
    every slot and count line is reused under a new epoch again and again."""
    import os

    os.environ["KB200_A2A_LL"] = low_latency
    from kernel_b200.ops.dispatch_combine import SCALE_EXPERT, MoEAllToAll, expert_scale_vector

    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16}[dtype_name]
    E, k, H, max_tokens = world, 1, 64, 6
    ctx = MoEAllToAll(E, k, H, max_tokens, dtype=dtype, device="cpu")
    assert ctx.low_latency == (low_latency == "1")
    g = torch.Generator().manual_seed(100 + rank)
    scale = expert_scale_vector(E, world, SCALE_EXPERT)
    ok = True
    for call in range(40):
        T = int(torch.randint(0, max_tokens + 1, (1,), generator=g))
        x = torch.randn(T, H, generator=g).to(dtype)
        idx = torch.randint(0, E, (T, k), generator=g, dtype=torch.int32)
        w = torch.rand(T, k, generator=g)
        out = ctx.dispatch_scale_combine(x, idx, w, SCALE_EXPERT)
        y = (x.float().unsqueeze(1) * scale[idx.long()].unsqueeze(-1)).to(dtype).float()
        ref = (y * w.unsqueeze(-1)).sum(1)
        tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=5e-3)
        ok = ok and tuple(out.shape) == (T, H) and bool(torch.allclose(out.float(), ref, **tol))
    ctx.heap.close()
    return ok


@pytest.mark.parametrize("low_latency", ["1", "0"])
def test_sparse_routing_over_many_epochs(low_latency):
    assert all(run_ranks(_sparse_calls, 4, low_latency, "fp32", timeout=300))


def _one_rank_runs_ahead(rank, world):
    """Rank 0 keeps itself busy with 32 long rows of its own and reads the other
    ranks' counts after them; rank 3 sends one row to rank 2 and is done with a call
    long before that, so its counts of the NEXT call reach rank 0 while rank 0 has
    not read those of the current one.  The count lines alternate with the epoch's
    parity for exactly this case (with one line per source rank 0 would wait for an
    epoch that has been overwritten)."""
    from kernel_b200.ops.dispatch_combine import SCALE_EXPERT, MoEAllToAll, expert_scale_vector

    E, k, H, max_tokens = world, 1, 16384, 32
    ctx = MoEAllToAll(E, k, H, max_tokens, dtype=torch.float32, device="cpu")
    assert ctx.low_latency
    g = torch.Generator().manual_seed(rank)
    T, target = {0: (32, 0), 1: (0, 0), 2: (1, 2), 3: (1, 2)}[rank]
    scale = expert_scale_vector(E, world, SCALE_EXPERT)
    ok = True
    for call in range(8):
        x = torch.randn(T, H, generator=g)
        idx = torch.full((T, k), target, dtype=torch.int32)
        w = torch.rand(T, k, generator=g)
        out = ctx.dispatch_scale_combine(x, idx, w, SCALE_EXPERT)
        ref = x * (w * scale[idx.long()]).sum(-1, keepdim=True)
        ok = ok and bool(torch.allclose(out, ref, rtol=1e-5, atol=1e-6))
    ctx.heap.close()
    return ok


def test_a_rank_may_be_one_call_ahead_of_a_busy_peer():
    assert all(run_ranks(_one_rank_runs_ahead, 4, timeout=300, env={"KB200_WAIT_LIMIT_MS": "5000"}))


def _dense_calls(rank, world, dtype_name):
    """Top-k routing with several experts of a token on one rank: the expert lists
    and weights travel with the row, the partial row is one weighted sum."""
    from kernel_b200.ops.dispatch_combine import SCALE_EXPERT, MoEAllToAll, expert_scale_vector

    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[dtype_name]
    E, k, H, max_tokens = 4 * world, 6, 128, 32
    ctx = MoEAllToAll(E, k, H, max_tokens, dtype=dtype, device="cpu")
    assert ctx.low_latency
    g = torch.Generator().manual_seed(7 + rank)
    scale = expert_scale_vector(E, world, SCALE_EXPERT)
    ok = True
    for call in range(6):
        T = int(torch.randint(1, max_tokens + 1, (1,), generator=g))
        x = torch.randn(T, H, generator=g).to(dtype)
        idx = torch.rand(T, E, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
        w = torch.softmax(torch.randn(T, k, generator=g), -1)
        out = ctx.dispatch_scale_combine(x, idx, w, SCALE_EXPERT)
        y = (x.float().unsqueeze(1) * scale[idx.long()].unsqueeze(-1)).to(dtype).float()
        ref = (y * w.unsqueeze(-1)).sum(1)
        tol = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=1e-2)
        ok = ok and bool(torch.allclose(out.float(), ref, **tol))
    ctx.heap.close()
    return ok


@pytest.mark.parametrize("dtype_name", ["fp32", "bf16", "fp16"])
def test_top_k_routing_with_shared_ranks(dtype_name):
    assert all(run_ranks(_dense_calls, 2, dtype_name, timeout=300))


def test_landing_area_size_matches_the_kernels_layout():
    """The host twin refuses to run when its layout and ``kb_a2a_ll_bytes`` disagree;
    here the closed form of the layout is checked against the exported size."""
    from kernel_b200 import _native as N

    lib = N.lib()
    limit = int(lib.kb_a2a_ll_max_tokens())
    assert limit == 32
    for world, tmax, k, hidden, eb in [(8, 32, 8, 7168, 2), (2, 1, 1, 8, 4), (4, 16, 6, 2048, 2)]:
        row2 = 2 * hidden * eb
        want = 2 * world * tmax * row2 + world * tmax * (2 * k + 2) * 8 + 2 * world * 128
        assert int(lib.kb_a2a_ll_bytes(world, tmax, k, hidden, eb)) == (want + 255) // 256 * 256
    assert int(lib.kb_a2a_ll_bytes(8, limit + 1, 8, 7168, 2)) == 0
