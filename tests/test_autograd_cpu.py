"""Backward passes of the fused linear layers against dense fp32 autograd (CPU paths of the ops)."""
import torch

from _mp import run_ranks


def _dense_reference(x_full, w1_full, b1_full, w2_full, b2, act):
    """fp32 leaf copies -> loss = sum(y * g) with the same rounding points as the sharded block."""
    leaves = [t.detach().float().requires_grad_(True) for t in (x_full, w1_full, b1_full, w2_full, b2)]
    x, w1, b1, w2, bb2 = leaves
    h = act(x @ w1.t() + b1)
    y = h @ w2.t() + bb2
    return y, leaves


def _mlp_rank(rank, world):
    import torch.distributed as dist

    from kernel_b200.models import TrainableSequenceParallelMLP

    torch.manual_seed(7)  # same on every rank: full tensors, then slices
    tokens, hidden, ffn = 16 * world, 32, 48 * world
    x_full = torch.randn(tokens, hidden).to(torch.bfloat16)
    w1_full = (torch.randn(ffn, hidden) / hidden ** 0.5).to(torch.bfloat16)
    b1_full = (torch.randn(ffn) * 0.1).to(torch.bfloat16)
    w2_full = (torch.randn(hidden, ffn) / ffn ** 0.5).to(torch.bfloat16)
    b2 = (torch.randn(hidden) * 0.1).to(torch.bfloat16)
    g_full = torch.randn(tokens, hidden).to(torch.bfloat16)
    fl, tl = ffn // world, tokens // world
    mlp = TrainableSequenceParallelMLP(tokens, hidden, fl, activation="silu", device="cpu")
    with torch.no_grad():
        mlp.up.weight.copy_(w1_full[rank * fl:(rank + 1) * fl])
        mlp.up.bias.copy_(b1_full[rank * fl:(rank + 1) * fl])
        mlp.down.weight.copy_(w2_full[:, rank * fl:(rank + 1) * fl])
        mlp.down.bias.copy_(b2)
    x_local = x_full[rank * tl:(rank + 1) * tl].clone().requires_grad_(True)
    y_local = mlp(x_local)
    (y_local.float() * g_full[rank * tl:(rank + 1) * tl].float()).sum().backward()

    y_ref, (x, w1, b1, w2, bb2) = _dense_reference(x_full, w1_full, b1_full, w2_full, b2, torch.nn.functional.silu)
    (y_ref * g_full.float()).sum().backward()
    db2 = mlp.down.bias.grad.float().clone()
    if world > 1:
        dist.all_reduce(db2)  # replicated parameter: partial sums over each rank's rows

    def close(a, b, tol=6e-2):
        scale = b.abs().max().item() + 1e-6
        return (a.float() - b).abs().max().item() / scale < tol

    return {
        "y": close(y_local, y_ref[rank * tl:(rank + 1) * tl].detach()),
        "dx": close(x_local.grad, x.grad[rank * tl:(rank + 1) * tl]),
        "dw1": close(mlp.up.weight.grad, w1.grad[rank * fl:(rank + 1) * fl]),
        "db1": close(mlp.up.bias.grad, b1.grad[rank * fl:(rank + 1) * fl]),
        "dw2": close(mlp.down.weight.grad, w2.grad[:, rank * fl:(rank + 1) * fl]),
        "db2": close(db2, bb2.grad),
        "shapes": (tuple(x_local.grad.shape), tuple(mlp.up.weight.grad.shape), tuple(mlp.down.weight.grad.shape)),
    }


def _check(res, world):
    for r in res:
        bad = [k for k, v in r.items() if k != "shapes" and not v]
        assert not bad, bad
        assert r["shapes"] == ((16, 32), (48, 32), (32, 48))


def test_trainable_mlp_backward_single_process():
    _check([_mlp_rank(0, 1)], 1)


def test_trainable_mlp_backward_gloo_world2():
    _check(run_ranks(_mlp_rank, 2), 2)


def test_no_weight_grad_skips_gather():
    from kernel_b200.ops.autograd import RowParallelLinear

    lin = RowParallelLinear(8, 16, 24, bias=False, device="cpu")
    lin.weight.requires_grad_(False)
    x = torch.randn(8, 16).to(torch.bfloat16).requires_grad_(True)
    lin(x).float().sum().backward()
    assert lin.weight.grad is None and x.grad.shape == (8, 16)
    expect = lin.weight.detach().float().sum(0).expand(8, 16)
    assert torch.allclose(x.grad.float(), expect, rtol=2e-2, atol=2e-2)


def _moe_rank(rank, world):
    import torch.distributed as dist

    from kernel_b200.models import TrainableMoELayer

    E, k, H, F, T = 4 * world, 2, 32, 48, 6 + rank
    El = E // world
    full = torch.Generator().manual_seed(5)  # identical expert weights on every rank
    w_up_full = (torch.randn(E, F, H, generator=full) / H ** 0.5).to(torch.bfloat16)
    w_down_full = (torch.randn(E, H, F, generator=full) / F ** 0.5).to(torch.bfloat16)
    layer = TrainableMoELayer(E, k, H, F, 16, device="cpu")
    with torch.no_grad():
        layer.w_up.copy_(w_up_full[rank * El:(rank + 1) * El])
        layer.w_down.copy_(w_down_full[rank * El:(rank + 1) * El])
    g = torch.Generator().manual_seed(50 + rank)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).requires_grad_(True)
    idx = torch.rand(T, E, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, generator=g), -1).requires_grad_(True)
    gy = torch.randn(T, H, generator=g).to(torch.bfloat16)
    for _ in range(2):  # two steps on the same workspaces
        for t in (x, w, layer.w_up, layer.w_down):
            t.grad = None
        y = layer(x, idx, w)
        (y.float() * gy.float()).sum().backward()

    # dense fp32 autograd over all experts; expert gradients summed over the ranks' losses
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    up = w_up_full.float().requires_grad_(True)
    down = w_down_full.float().requires_grad_(True)
    yr = torch.zeros(T, H)
    for t in range(T):
        for j in range(k):
            e = int(idx[t, j])
            yr[t] = yr[t] + wr[t, j] * (torch.nn.functional.silu(xr[t] @ up[e].t()) @ down[e].t())
    (yr * gy.float()).sum().backward()
    gup, gdown = up.grad.clone(), down.grad.clone()
    if world > 1:
        dist.all_reduce(gup)
        dist.all_reduce(gdown)

    def close(a, b, tol=6e-2):
        return (a.float() - b).abs().max().item() / (b.abs().max().item() + 1e-6) < tol

    res = {
        "y": close(y, yr.detach()),
        "dx": close(x.grad, xr.grad),
        "dw": close(w.grad, wr.grad),
        "dup": close(layer.w_up.grad, gup[rank * El:(rank + 1) * El]),
        "ddown": close(layer.w_down.grad, gdown[rank * El:(rank + 1) * El]),
    }
    layer.close()
    return res


def test_trainable_moe_backward_single_process():
    r = _moe_rank(0, 1)
    assert all(r.values()), r


def test_trainable_moe_backward_host_heap_world3():
    for r in run_ranks(_moe_rank, 3):
        assert all(r.values()), r


def test_expert_major_rows_order():
    from kernel_b200.models.moe import _expert_major_rows

    counts = torch.tensor([[2, 0, 1], [1, 3, 0]], dtype=torch.int32)   # [world 2, El 3], capacity 10 rows per source
    idx, n_e = _expert_major_rows(counts, 10)
    assert n_e == [3, 3, 1]
    # expert 0: src0 rows 0,1 and src1 row 0; expert 1: src1 rows 1..3; expert 2: src0 row 2
    assert idx.tolist() == [0, 1, 10, 11, 12, 13, 2]


def _demo(rank, world, moe):
    from kernel_b200.utils.train_demo import train

    return train(steps=12, tokens=64 * world, hidden=32, ffn=64 * world, moe=moe, lr=0.05, device="cpu")


def test_training_demo_loss_decreases_single_process():
    losses = _demo(0, 1, True)
    assert losses[-1] < 0.9 * losses[0] and all(b <= a * 1.02 for a, b in zip(losses, losses[1:]))


def test_training_demo_loss_decreases_gloo_world2():
    res = run_ranks(_demo, 2, True)
    assert res[0] == res[1]                       # the all-reduced loss is the same number on both ranks
    assert res[0][-1] < 0.9 * res[0][0]
