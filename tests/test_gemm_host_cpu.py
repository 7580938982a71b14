"""The fused GEMM protocols run by CPU ranks over the host-backed symmetric heap:
tile schedule, staging layouts, epoch flags, parity reuse and time-outs."""
import pytest
import torch

from kernel_b200 import _native as N

from _mp import run_ranks


def _rs(rank, world, M, Nn, Kl, with_bias, calls):
    import torch.distributed as dist

    from kernel_b200.ops.gemm import GemmRS

    ctx = GemmRS(M, Nn, device="cpu")
    assert ctx.host_heap and ctx.heap.backend == "host"
    oks = []
    for it in range(calls):  # several epochs on one workspace: both parities get reused
        g = torch.Generator().manual_seed(1000 * it + rank)
        a = torch.randn(M, Kl, generator=g).to(torch.bfloat16)
        w = (torch.randn(Nn, Kl, generator=g) / Kl ** 0.5).to(torch.bfloat16)
        bias = (torch.randn(Nn, generator=torch.Generator().manual_seed(it)) * 0.1).to(torch.bfloat16) if with_bias else None
        out = ctx(a, w, bias, bias_scale=0.5)
        part = a.float() @ w.float().t()
        mag = part.abs()
        dist.all_reduce(part)
        dist.all_reduce(mag)
        rows = M // world
        ref = part[rank * rows:(rank + 1) * rows]
        if with_bias:
            ref = ref + 0.5 * bias.float()
        err = (out.float() - ref).abs()
        tol = 1e-2 + 1e-2 * mag[rank * rows:(rank + 1) * rows]  # bf16 partials: error scales with sum |partial|
        oks.append(bool((err <= tol).all()) and out.shape == (rows, Nn))
    ctx.heap.close()
    return all(oks)


@pytest.mark.parametrize("world,M,Nn,Kl,with_bias", [
    (2, 256, 264, 72, True),     # one row block per rank, N tail
    (3, 192, 512, 40, False),    # rows per rank 64: two owners share a row block, M tail
    (4, 1024, 256, 24, True),    # several row blocks per rank
    (8, 512, 264, 16, True),     # the flagship world size: 64 rows per rank, two owners per row block
])
def test_gemm_rs_over_host_heap(world, M, Nn, Kl, with_bias):
    assert all(run_ranks(_rs, world, M, Nn, Kl, with_bias, 3))


def _ag(rank, world, M, Nl, K, with_bias, calls):
    import torch.distributed as dist

    from kernel_b200.ops.gemm import AGGemm

    ctx = AGGemm(M, K, device="cpu")
    assert ctx.host_heap
    rows = M // world
    oks = []
    for it in range(calls):
        g = torch.Generator().manual_seed(77 * it + rank)
        a_local = torch.randn(rows, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(Nl, K, generator=g) / K ** 0.5).to(torch.bfloat16)
        bias = (torch.randn(Nl, generator=g) * 0.1).to(torch.bfloat16) if with_bias else None
        out = ctx(a_local, w, bias)
        full = torch.empty(M, K, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, a_local)
        ref = full.float() @ w.float().t()
        if with_bias:
            ref = ref + bias.float()
        oks.append(bool(torch.allclose(out.float(), ref, rtol=1e-2, atol=1e-2)) and out.shape == (M, Nl))
    ctx.heap.close()
    return all(oks)


@pytest.mark.parametrize("world,M,Nl,K,with_bias", [
    (2, 256, 264, 72, True),
    (3, 192, 256, 40, False),    # rows per rank 64: a row block waits for two sources
    (4, 1024, 128, 24, True),
    (8, 1024, 72, 16, False),    # the flagship world size: one row block per rank
])
def test_ag_gemm_over_host_heap(world, M, Nl, K, with_bias):
    assert all(run_ranks(_ag, world, M, Nl, K, with_bias, 3))


def _rs_absent(rank, world):
    from kernel_b200.ops.gemm import GemmRS

    ctx = GemmRS(256, 64, device="cpu")
    a = torch.randn(256, 16).to(torch.bfloat16)
    w = torch.randn(64, 16).to(torch.bfloat16)
    ctx(a, w)  # epoch 1: everybody takes part
    if rank == 1:
        return "absent"
    try:
        ctx(a, w)
    except N.SymmTimeoutError as e:
        return str(e)
    return "no error"


def test_gemm_rs_wait_names_the_rank_that_never_arrived():
    res = run_ranks(_rs_absent, 2, env={"KB200_WAIT_LIMIT_MS": "300"})
    assert res[1] == "absent"
    assert "rank 1 never delivered its partial tile of epoch 2" in res[0]


def test_gemm_host_rejects_bad_arguments():
    lib = N.lib()
    args = N.GemmArgs()
    args.mode, args.world, args.rank = N.GEMM_RS, 1, 0
    assert lib.kb_gemm_host(args, 10) == N.KB_ERR_ARG and "world >= 2" in N.last_error()
    args.world, args.mode = 2, N.GEMM_PLAIN
    assert lib.kb_gemm_host(args, 10) == N.KB_ERR_ARG and "not a fused mode" in N.last_error()
    args.mode, args.M, args.N, args.K = N.GEMM_AG, 96 * 2, 8, 8   # 96 rows per rank: neither divides nor is a multiple of 128
    assert lib.kb_gemm_host(args, 10) == N.KB_ERR_ARG and "rows per rank" in N.last_error()


def test_collectives_path_still_selectable(monkeypatch):
    from kernel_b200.ops.gemm import GemmRS

    monkeypatch.setenv("KB200_GEMM_CPU_PATH", "collectives")
    ctx = GemmRS(128, 64, device="cpu")
    assert not ctx.host_heap and ctx.heap is None


def _many_shapes(rank, world, seed):
    """Both fused ops over a handful of random shapes in one set of ranks."""
    import random

    import torch.distributed as dist

    from kernel_b200.ops.gemm import AGGemm, GemmRS

    rnd = random.Random(seed)   # same shapes on every rank
    bad = []
    for case in range(6):
        rpo = rnd.choice([8, 16, 32, 64, 128, 256])
        M = rpo * world
        Nn = rnd.randrange(1, 60) * 8
        K = rnd.randrange(1, 12) * 8
        g = torch.Generator().manual_seed(seed * 100 + case * 10 + rank)
        # reduce-scatter: K is the local share
        a = torch.randn(M, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(Nn, K, generator=g) / (K * world) ** 0.5).to(torch.bfloat16)
        rs = GemmRS(M, Nn, device="cpu")
        out = rs(a, w)
        part = a.float() @ w.float().t()
        mag = part.abs()
        dist.all_reduce(part)
        dist.all_reduce(mag)
        sl = slice(rank * rpo, (rank + 1) * rpo)
        if not bool(((out.float() - part[sl]).abs() <= 1e-2 + 1e-2 * mag[sl]).all()):
            bad.append(("rs", M, Nn, K))
        rs.heap.close()
        # all-gather: N is the local share
        a_local = torch.randn(rpo, K, generator=g).to(torch.bfloat16)
        ag = AGGemm(M, K, device="cpu")
        out = ag(a_local, w)
        full = torch.empty(M, K, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, a_local)
        if not torch.allclose(out.float(), full.float() @ w.float().t(), rtol=1e-2, atol=1e-2):
            bad.append(("ag", M, Nn, K))
        ag.heap.close()
    return bad


@pytest.mark.parametrize("world,seed", [(2, 1), (4, 2), (3, 3)])
def test_random_shapes_over_host_heap(world, seed):
    for bad in run_ranks(_many_shapes, world, seed, timeout=300):
        assert bad == []
