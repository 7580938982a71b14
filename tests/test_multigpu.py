"""The three fused ops across GPUs (one process per GPU, NCCL as control plane
only), checked with the tasks' own oracles.  Needs at least two GPUs."""
import pytest
import torch

from _mp import run_ranks

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]


def _world():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else (4 if n >= 4 else 2)


def _a2a(rank, world, specs):
    import torch

    from kernel_b200.tasks.all2all import reference as R
    from kernel_b200.tasks.all2all import submission as S

    res = []
    for spec in specs:
        data = R.generate_input(**spec, rank=rank, world_size=world)
        out1 = S.custom_kernel(data)
        out2 = S.custom_kernel(data)
        torch.cuda.synchronize()
        ctx = S.get_context(data[0], world, data[1].x.device)
        ctx.heap.check_status()
        ok, msg = R.check_implementation(data, out1)
        closed = torch.allclose(out1.float(), R.ref_closed_form(data).float(), rtol=1e-2, atol=5e-3)
        res.append((ok, msg, bool(closed), bool(torch.equal(out1, out2))))
    S.release_contexts()
    return res


def test_all2all_task_cases():
    world = _world()
    specs = [
        dict(num_experts=8, experts_per_token=2, hidden_dim=6144, max_num_tokens=4, seed=1236),
        dict(num_experts=64, experts_per_token=6, hidden_dim=2048, max_num_tokens=8, seed=542),
        dict(num_experts=128, experts_per_token=4, hidden_dim=2880, max_num_tokens=32, seed=51),
        dict(num_experts=256, experts_per_token=8, hidden_dim=7168, max_num_tokens=128, seed=4),
        dict(num_experts=256, experts_per_token=8, hidden_dim=7168, max_num_tokens=256, seed=11, dtype="bf16",
             fixed_tokens=True, weight_mode="softmax", expert_scale="expert"),
        dict(num_experts=8, experts_per_token=2, hidden_dim=256, max_num_tokens=64, seed=3, dtype="fp32",
             fixed_tokens=True, weight_mode="softmax", expert_scale="identity"),
    ]
    for per_rank in run_ranks(_a2a, world, specs, backend="nccl", timeout=300):
        for ok, msg, closed, repeat in per_rank:
            assert ok, msg
            assert closed and repeat


def _gemm_rs(rank, world, shapes):
    import torch

    from kernel_b200.tasks.gemm_rs import reference as R
    from kernel_b200.tasks.gemm_rs import submission as S

    res = []
    for (m, n, k, bias, dist_mode, bias_mode) in shapes:
        data = R.generate_input(rank, world, m, n, k, bias, seed=7, dist=dist_mode, bias_mode=bias_mode)
        out1 = S.custom_kernel(data)
        out2 = S.custom_kernel(data)
        torch.cuda.synchronize()
        ctx = S.get_context(m, n, data[0].device)
        if ctx.heap is not None:
            ctx.heap.check_status()
        ok, msg = R.check_implementation(data, out1)
        res.append((ok, msg, bool(torch.equal(out1, out2)), tuple(out1.shape) == (m // world, n)))
    S.release_contexts()
    return res


def test_gemm_rs_task_shapes():
    world = _world()
    shapes = [
        (64, 2880, 2880 // 8 * world, True, "uniform", "per_rank"),   # rows per rank < tile: row-granular ownership
        (512, 3584, 14336 // 8 * world, True, "normal", "once"),
        (2048, 4096, 7168 // 8 * world, False, "normal", "once"),
        (4096, 2880, 2880 // 8 * world, True, "normal", "per_rank"),
        (8192, 8192, 29568 // 8 * world, True, "normal", "once"),     # K_local 3696: K tail of 48
    ]
    for per_rank in run_ranks(_gemm_rs, world, shapes, backend="nccl", timeout=300):
        for ok, msg, repeat, shape_ok in per_rank:
            assert ok, msg
            assert repeat and shape_ok


def _ag_gemm(rank, world, shapes):
    import torch

    from kernel_b200.tasks.ag_gemm import reference as R
    from kernel_b200.tasks.ag_gemm import submission as S

    res = []
    for (m, n, k, bias) in shapes:
        data = R.generate_input(rank, world, m, n, k, bias, seed=9)
        out1 = S.custom_kernel(data)
        out2 = S.custom_kernel(data)
        torch.cuda.synchronize()
        ctx = S.get_context(m, k, data[0].device)
        if ctx.heap is not None:
            ctx.heap.check_status()
        ok, msg = R.check_implementation(data, out1)
        res.append((ok, msg, bool(torch.equal(out1, out2))))
    S.release_contexts()
    return res


def test_ag_gemm_shapes():
    world = _world()
    shapes = [
        (64, 2880 * world // 8 * 8, 2880, True),   # rows per rank < tile: several sources per row block
        (1024, 4096, 4096, False),
        (4096, 2880 * world, 2880, True),
        (8192, 3696 * world, 8192, True),           # N_local 3696: N tail of 112
    ]
    for per_rank in run_ranks(_ag_gemm, world, shapes, backend="nccl", timeout=300):
        for ok, msg, repeat in per_rank:
            assert ok, msg
            assert repeat


def _nvls_bring_up(rank, world):
    """Multicast object over a 1 MB buffer: create, add, bind, multimem.st from every
    rank, every rank reads all slices; then a multimem.ld_reduce over all ranks' copies;
    unbind and close in order with all ranks alive."""
    import torch

    from kernel_b200 import _native as N
    from kernel_b200.parallel.symm import SymmHeap

    dev = torch.device("cuda", rank)
    heap = SymmHeap(4 << 20, device=dev, nvls=True)
    if heap.mc_ptr is None:
        heap.close()
        return "no multicast"
    lib = N.lib()
    stream = torch.cuda.current_stream(dev).cuda_stream
    nbytes = 1 << 20
    piece = nbytes // world // 16 * 16
    off = heap.alloc(nbytes)
    src = torch.full((piece // 2,), float(rank + 1), dtype=torch.bfloat16, device=dev)
    N.check(lib.kb_multimem_store(heap.mc_ptr + off + rank * piece, src.data_ptr(), piece, stream))
    heap.barrier()
    torch.cuda.synchronize()
    got = heap.tensor(off, (world, piece // 2), torch.bfloat16)
    stored = all(bool((got[r] == r + 1).all()) for r in range(world))
    off2 = heap.alloc(nbytes)
    heap.tensor(off2, (nbytes // 2,), torch.bfloat16).fill_(float(rank + 1))
    heap.barrier()
    total = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=dev)
    N.check(lib.kb_multimem_reduce_bf16(total.data_ptr(), heap.mc_ptr + off2, nbytes, stream))
    torch.cuda.synchronize()
    reduced = bool((total == world * (world + 1) // 2).all())
    heap.barrier()  # nobody unbinds while a peer's load may still be in the switch
    torch.cuda.synchronize()
    heap.check_status()
    heap.close()
    return stored, reduced


def test_nvls_multicast_bring_up():
    world = _world()
    res = run_ranks(_nvls_bring_up, world, backend="nccl", timeout=180)
    if all(r == "no multicast" for r in res):
        pytest.skip("the devices or the driver offer no multicast objects")
    assert all(r == (True, True) for r in res), res


def _fused_gemms_over_nvls(rank, world):
    """The reduce-scatter pull through multimem.ld_reduce and the all-gather push
    through multimem.st, checked by the tasks' oracles."""
    import torch

    from kernel_b200.tasks.ag_gemm import reference as AR
    from kernel_b200.tasks.ag_gemm import submission as AS
    from kernel_b200.tasks.gemm_rs import reference as RR
    from kernel_b200.tasks.gemm_rs import submission as RS

    res = []
    for (m, n, k, bias) in [(64, 2880, 2880 // 8 * world, True), (2048, 4096, 7168 // 8 * world, True),
                            (8192, 8192, 29568 // 8 * world, True)]:
        data = RR.generate_input(rank, world, m, n, k, bias, seed=7, dist="normal", bias_mode="once")
        out = RS.custom_kernel(data)
        out2 = RS.custom_kernel(data)
        torch.cuda.synchronize()
        ctx = RS.get_context(m, n, data[0].device)
        ctx.heap.check_status()
        ok, msg = RR.check_implementation(data, out)
        res.append(("gemm_rs", ctx.heap.mc_ptr is not None, ok and bool(torch.equal(out, out2)), msg))
    for (m, n, k, bias) in [(64, 2880, 2880, True), (1024, 4096, 4096, False), (8192, 3696 * world, 8192, True)]:
        data = AR.generate_input(rank, world, m, n, k, bias, seed=9)
        out = AS.custom_kernel(data)
        out2 = AS.custom_kernel(data)
        torch.cuda.synchronize()
        ctx = AS.get_context(m, k, data[0].device)
        ctx.heap.check_status()
        ok, msg = AR.check_implementation(data, out)
        res.append(("ag_gemm", ctx.heap.mc_ptr is not None, ok and bool(torch.equal(out, out2)), msg))
    RS.release_contexts()
    AS.release_contexts()
    return res


@pytest.mark.parametrize("nvls", ["1", "0"])
def test_fused_gemms_with_and_without_nvls(nvls):
    world = _world()
    res = run_ranks(_fused_gemms_over_nvls, world, backend="nccl", timeout=300, env={"KB200_NVLS": nvls})
    if nvls == "0":
        for per_rank in res:
            for op, mc, ok, msg in per_rank:
                assert not mc and ok, (op, msg)
        return
    if not any(mc for per_rank in res for _, mc, _, _ in per_rank):
        pytest.skip("the devices or the driver offer no multicast objects")
    for per_rank in res:
        for op, mc, ok, msg in per_rank:
            assert mc and ok, (op, msg)


def _mlp_backward(rank, world):
    """Forward + backward of the trainable sequence-parallel MLP; returns the
    relative errors against dense fp32 autograd on the gathered problem."""
    import torch
    import torch.distributed as dist

    from kernel_b200.models import TrainableSequenceParallelMLP

    dev = torch.device("cuda", rank)
    torch.manual_seed(11)  # identical full tensors on every rank
    tokens, hidden, fl = 128 * world, 512, 256
    ffn, tl = fl * world, 128
    x_full = torch.randn(tokens, hidden, device=dev).to(torch.bfloat16)
    w1_full = (torch.randn(ffn, hidden, device=dev) / hidden ** 0.5).to(torch.bfloat16)
    b1_full = (torch.randn(ffn, device=dev) * 0.05).to(torch.bfloat16)
    w2_full = (torch.randn(hidden, ffn, device=dev) / ffn ** 0.5).to(torch.bfloat16)
    b2 = (torch.randn(hidden, device=dev) * 0.05).to(torch.bfloat16)
    g_full = torch.randn(tokens, hidden, device=dev).to(torch.bfloat16)
    mlp = TrainableSequenceParallelMLP(tokens, hidden, fl, activation="silu", device=dev)
    with torch.no_grad():
        mlp.up.weight.copy_(w1_full[rank * fl:(rank + 1) * fl])
        mlp.up.bias.copy_(b1_full[rank * fl:(rank + 1) * fl])
        mlp.down.weight.copy_(w2_full[:, rank * fl:(rank + 1) * fl])
        mlp.down.bias.copy_(b2)
    x_local = x_full[rank * tl:(rank + 1) * tl].clone().requires_grad_(True)
    y_local = mlp(x_local)
    (y_local.float() * g_full[rank * tl:(rank + 1) * tl].float()).sum().backward()
    torch.cuda.synchronize()
    for lin in (mlp.up, mlp.down):
        for c in (lin.fwd, lin.bwd):
            c.heap.check_status()
    leaves = [t.detach().float().requires_grad_(True) for t in (x_full, w1_full, b1_full, w2_full, b2)]
    x, w1, b1, w2, bb2 = leaves
    y_ref = torch.nn.functional.silu(x @ w1.t() + b1) @ w2.t() + bb2
    (y_ref * g_full.float()).sum().backward()
    db2 = mlp.down.bias.grad.float().clone()
    dist.all_reduce(db2)

    def err(a, b):
        return (a.float() - b).abs().max().item() / (b.abs().max().item() + 1e-6)

    res = {
        "y": err(y_local, y_ref[rank * tl:(rank + 1) * tl].detach()),
        "dx": err(x_local.grad, x.grad[rank * tl:(rank + 1) * tl]),
        "dw1": err(mlp.up.weight.grad, w1.grad[rank * fl:(rank + 1) * fl]),
        "db1": err(mlp.up.bias.grad, b1.grad[rank * fl:(rank + 1) * fl]),
        "dw2": err(mlp.down.weight.grad, w2.grad[:, rank * fl:(rank + 1) * fl]),
        "db2": err(db2, bb2.grad),
    }
    dist.barrier()
    mlp.close()
    return res


def test_trainable_mlp_backward_across_gpus():
    world = _world()
    for errs in run_ranks(_mlp_backward, world, backend="nccl", timeout=300):
        assert max(errs.values()) < 5e-2, errs


def _moe_backward(rank, world):
    """Two training steps of the expert-parallel MoE block; relative errors against
    dense fp32 autograd over all experts (expert gradients summed over the ranks)."""
    import torch
    import torch.distributed as dist

    from kernel_b200.models import TrainableMoELayer

    dev = torch.device("cuda", rank)
    E, k, H, F, T = 4 * world, 2, 256, 384, 24 + rank
    El = E // world
    full = torch.Generator(device=dev).manual_seed(5)
    w_up_full = (torch.randn(E, F, H, device=dev, generator=full) / H ** 0.5).to(torch.bfloat16)
    w_down_full = (torch.randn(E, H, F, device=dev, generator=full) / F ** 0.5).to(torch.bfloat16)
    layer = TrainableMoELayer(E, k, H, F, 64, device=dev)
    with torch.no_grad():
        layer.w_up.copy_(w_up_full[rank * El:(rank + 1) * El])
        layer.w_down.copy_(w_down_full[rank * El:(rank + 1) * El])
    g = torch.Generator(device=dev).manual_seed(50 + rank)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    idx = torch.rand(T, E, device=dev, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, device=dev, generator=g), -1).requires_grad_(True)
    gy = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    for _ in range(2):
        for t in (x, w, layer.w_up, layer.w_down):
            t.grad = None
        y = layer(x, idx, w)
        (y.float() * gy.float()).sum().backward()
    torch.cuda.synchronize()
    layer.a2a.heap.check_status()
    layer.meta.heap.check_status()

    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    up = w_up_full.float().requires_grad_(True)
    down = w_down_full.float().requires_grad_(True)
    hid = torch.nn.functional.silu(torch.einsum("th,tkfh->tkf", xr, up[idx.long()]))
    yr = (torch.einsum("tkf,tkhf->tkh", hid, down[idx.long()]) * wr.unsqueeze(-1)).sum(1)
    (yr * gy.float()).sum().backward()
    gup, gdown = up.grad.clone(), down.grad.clone()
    dist.all_reduce(gup)
    dist.all_reduce(gdown)

    def err(a, b):
        return (a.float() - b).abs().max().item() / (b.abs().max().item() + 1e-6)

    res = {"y": err(y, yr.detach()), "dx": err(x.grad, xr.grad), "dw": err(w.grad, wr.grad),
           "dup": err(layer.w_up.grad, gup[rank * El:(rank + 1) * El]),
           "ddown": err(layer.w_down.grad, gdown[rank * El:(rank + 1) * El])}
    dist.barrier()
    layer.close()
    return res


def test_trainable_moe_backward_across_gpus():
    world = _world()
    for errs in run_ranks(_moe_backward, world, backend="nccl", timeout=300):
        assert max(errs.values()) < 5e-2, errs


def _rank_leaves(rank, world):
    """A rank leaves between steps (nothing in flight); the others learn of it
    from the host-side store before their next launch."""
    import torch
    import torch.distributed as dist

    from kernel_b200.ops.gemm import GemmRS

    dev = torch.device("cuda", rank)
    ctx = GemmRS(256, 512, device=dev)
    a = torch.randn(256, 64, device=dev).to(torch.bfloat16)
    w = torch.randn(512, 64, device=dev).to(torch.bfloat16)
    ctx(a, w)
    torch.cuda.synchronize()
    ctx.heap.check_status()
    store = dist.distributed_c10d._get_default_store()
    store.set(f"alive/{rank}", "1")
    dist.barrier()
    if rank == world - 1:
        store.set(f"alive/{rank}", "0")  # announces its departure, then stops taking part
        left = True
    else:
        left = False
    dist.barrier()
    gone = [r for r in range(world) if store.get(f"alive/{r}") == b"0"]
    if not left and not gone:
        ctx(a, w)  # would only run if everybody were still there
    dist.barrier()
    ctx.heap.close()
    return gone


def test_departed_rank_is_seen_on_the_host_before_the_next_launch(monkeypatch):
    world = 2
    # no multicast anywhere in a test where a rank stops taking part: neither in NCCL nor in the heap
    res = run_ranks(_rank_leaves, world, backend="nccl", timeout=120, env={"NCCL_NVLS_ENABLE": "0", "KB200_NVLS": "0"})
    assert all(gone == [world - 1] for gone in res)


def _two_devices_one_process(rank, world):
    """The same process runs the one-launch MoE kernel (more than 48 KB of dynamic
    shared memory: a per-device function attribute) and a GEMM first on one device,
    then on another, as an evaluator's pool worker does when it serves rank 0 in
    one case and rank 1 in the next."""
    import torch

    from kernel_b200.ops.dispatch_combine import MoEAllToAll
    from kernel_b200.ops.gemm import gemm

    res = []
    for index in (0, 1):
        dev = torch.device("cuda", index)
        torch.cuda.set_device(dev)
        g = torch.Generator(device=dev).manual_seed(3)
        E, k, H, T = 64, 4, 4096, 100          # above the low-latency limit: the regular one-launch kernel
        x = torch.randn(T, H, device=dev, generator=g).to(torch.float16)
        idx = torch.rand(T, E, device=dev, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
        w = torch.rand(T, k, device=dev, generator=g)
        ctx = MoEAllToAll(E, k, H, 128, dtype=torch.float16, device=dev)
        out = ctx.dispatch_scale_combine(x, idx, w, 0)
        torch.cuda.synchronize(dev)
        ctx.heap.check_status()
        want = x.float() * w.sum(-1, keepdim=True)
        ok_a2a = bool(torch.allclose(out.float(), want, rtol=1e-2, atol=5e-3))
        ctx.heap.close()
        a = torch.randn(512, 1024, device=dev, generator=g).to(torch.bfloat16)
        b = (torch.randn(768, 1024, device=dev, generator=g) / 32).to(torch.bfloat16)
        c = gemm(a, b)
        torch.cuda.synchronize(dev)
        ok_gemm = bool(torch.allclose(c.float(), a.float() @ b.float().t(), rtol=2e-2, atol=2e-2))
        res.append((ok_a2a, ok_gemm))
    return res


def test_one_process_uses_the_kernels_on_two_devices_in_turn():
    (res,) = run_ranks(_two_devices_one_process, 1, backend="nccl", timeout=300)
    assert res == [(True, True), (True, True)]
