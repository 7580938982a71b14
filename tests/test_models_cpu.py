"""Model blocks on the CPU paths of the ops (single process)."""
import torch


def test_sequence_parallel_mlp_cpu_single_rank():
    from kernel_b200.models import SequenceParallelMLP

    torch.manual_seed(0)
    tokens, hidden, ffn = 32, 64, 128
    x = torch.randn(tokens, hidden).to(torch.bfloat16)
    w1 = (torch.randn(ffn, hidden) / hidden ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn(hidden, ffn) / ffn ** 0.5).to(torch.bfloat16)
    b1 = (torch.randn(ffn) * 0.02).to(torch.bfloat16)
    mlp = SequenceParallelMLP(tokens, hidden, w1, w2, b1, None, activation="silu")
    y = mlp(x)
    ref = mlp.reference(x, w1, w2, b1, None)
    assert y.shape == (tokens, hidden) and torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)


def test_moe_layer_dense_formulation_matches_manual():
    from kernel_b200.models import MoELayer

    torch.manual_seed(1)
    E, k, H, F, T = 4, 2, 32, 64, 6
    w_up = (torch.randn(E, F, H) / H ** 0.5).to(torch.bfloat16)
    w_down = (torch.randn(E, H, F) / F ** 0.5).to(torch.bfloat16)
    layer = MoELayer(E, k, H, T, w_up, w_down)
    x = torch.randn(T, H).to(torch.bfloat16)
    idx = torch.rand(T, E).argsort(1)[:, :k].to(torch.int32)
    w = torch.softmax(torch.randn(T, k), -1)
    y = layer(x, idx, w)
    manual = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(idx[t, j])
            h = torch.nn.functional.silu(x[t].float() @ w_up[e].float().t())
            manual[t] += w[t, j] * (h @ w_down[e].float().t())
    assert torch.allclose(y.float(), manual, rtol=5e-2, atol=5e-2)


def _moe_layer_ranks(rank, world):
    """Forward of the expert-parallel layer on CPU ranks (host-heap dispatch and
    combine around real expert MLPs) against the single-process formulation with all experts."""
    from kernel_b200.models import MoELayer

    E, k, H, F, T = 3 * world, 2, 32, 64, 5 + rank
    El = E // world
    full = torch.Generator().manual_seed(9)
    w_up = (torch.randn(E, F, H, generator=full) / H ** 0.5).to(torch.bfloat16)
    w_down = (torch.randn(E, H, F, generator=full) / F ** 0.5).to(torch.bfloat16)
    layer = MoELayer(E, k, H, 8, w_up[rank * El:(rank + 1) * El], w_down[rank * El:(rank + 1) * El])
    g = torch.Generator().manual_seed(20 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    idx = torch.rand(T, E, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, generator=g), -1)
    y1 = layer(x, idx, w)
    y2 = layer(x, idx, w)
    manual = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(idx[t, j])
            h = torch.nn.functional.silu(x[t].float() @ w_up[e].float().t())
            manual[t] += w[t, j] * (h @ w_down[e].float().t())
    ok = torch.allclose(y1.float(), manual, rtol=5e-2, atol=5e-2) and torch.equal(y1, y2)
    layer.close()
    return bool(ok)


def test_moe_layer_on_cpu_ranks_world3():
    from _mp import run_ranks

    assert all(run_ranks(_moe_layer_ranks, 3))
