"""MoE dispatch/combine kernels on one GPU (world 1: every expert is local, the
rows still travel through the symmetric workspace with the same code path)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = [
    # E, k, H, T, dtype, scale_mode
    (8, 2, 256, 64, torch.float32, 0),
    (64, 6, 2048, 7, torch.float16, 1),
    (128, 4, 2880, 33, torch.float16, 1),
    (256, 8, 7168, 256, torch.bfloat16, 2),
    (256, 8, 7168, 1, torch.bfloat16, 2),
    (32, 8, 1024, 700, torch.bfloat16, 2),  # several tokens per CTA
]


def _inputs(E, k, H, T, dtype, dev, seed=0):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(T, H, device=dev, generator=g).to(dtype)
    idx = torch.rand(T, E, device=dev, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, device=dev, generator=g), -1)
    return x, idx, w


def _expected(x, idx, w, E, mode):
    from kernel_b200.ops.dispatch_combine import expert_scale_vector

    sc = expert_scale_vector(E, 1, mode, x.device)[idx.long()]
    y = (x.float().unsqueeze(1) * sc.unsqueeze(-1)).to(x.dtype).float()
    return (y * w.unsqueeze(-1)).sum(1)


@pytest.mark.parametrize("fused", ["1", "0"])
@pytest.mark.parametrize("E,k,H,T,dtype,mode", CASES)
def test_round_trip_matches_fp32_reference(E, k, H, T, dtype, mode, fused, monkeypatch):
    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    monkeypatch.setenv("KB200_A2A_FUSED", fused)
    dev = torch.device("cuda")
    ctx = MoEAllToAll(E, k, H, max(T, 2), dtype=dtype, device=dev)
    x, idx, w = _inputs(E, k, H, T, dtype, dev)
    out1 = ctx.dispatch_scale_combine(x, idx, w, mode)
    out2 = ctx.dispatch_scale_combine(x, idx, w, mode)  # second epoch on the same workspace
    torch.cuda.synchronize()
    ctx.heap.check_status()
    ref = _expected(x, idx, w, E, mode)
    tol = dict(rtol=1e-2, atol=5e-3) if dtype != torch.float32 else dict(rtol=1e-5, atol=1e-6)
    assert torch.allclose(out1.float(), ref, **tol)
    assert torch.equal(out1, out2)  # fixed k order: bit-reproducible


def test_split_dispatch_expert_combine_api():
    """dispatch -> user expert kernel on the received rows -> combine."""
    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    E, k, H, T = 16, 4, 512, 40
    dev = torch.device("cuda")
    ctx = MoEAllToAll(E, k, H, T, dtype=torch.bfloat16, device=dev)
    x, idx, w = _inputs(E, k, H, T, torch.bfloat16, dev, seed=3)
    counts, recv = ctx.dispatch(x, idx)
    torch.cuda.synchronize()
    assert int(counts.sum()) == T * k
    assert torch.equal(counts[0].long(), torch.bincount(idx.reshape(-1).long(), minlength=E))
    # rows of expert e are contiguous, in expert order; every received row equals a token of that expert
    off = 0
    for e in range(E):
        c = int(counts[0, e])
        toks = (idx == e).any(1).nonzero().flatten()
        got = recv[0, off:off + c]
        assert c == toks.numel()
        assert torch.equal(got.float().sum(0), x[toks].float().sum(0)) or torch.allclose(got.float().sort(0).values, x[toks].float().sort(0).values)
        off += c
    num, ex = ctx.expert_view(counts, recv)  # reference-style expert-major padded view
    assert ex.shape == (E, T, H) and torch.equal(num.cpu().long(), counts[0].cpu().long())
    y = ctx.expert_output_buffer()
    y.copy_(recv * 2)  # the "expert": doubles its input
    out = ctx.combine(x, idx, w)
    torch.cuda.synchronize()
    ctx.heap.check_status()
    ref = (x.float() * 2).to(torch.bfloat16).float() * w.sum(-1, keepdim=True)
    assert torch.allclose(out.float(), ref, rtol=1e-2, atol=5e-3)


@pytest.mark.parametrize("T", [0, 1, 16, 32])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_low_latency_path_equals_regular_path(T, dtype, monkeypatch):
    """Contexts of at most 32 tokens per rank take the flag-in-data kernel; its
    rounding points are those of the regular one-launch kernel, so the outputs are
    equal bit for bit, call after call (the count lines alternate with the epoch)."""
    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    dev = torch.device("cuda")
    E, k, H = 64, 8, 7168
    x, idx, w = _inputs(E, k, H, T, dtype, dev, seed=T)
    ll = MoEAllToAll(E, k, H, 32, dtype=dtype, device=dev)
    assert ll.low_latency
    monkeypatch.setenv("KB200_A2A_LL", "0")
    regular = MoEAllToAll(E, k, H, 32, dtype=dtype, device=dev)
    assert not regular.low_latency
    want = regular.dispatch_scale_combine(x, idx, w, 2)
    for _ in range(3):
        got = ll.dispatch_scale_combine(x, idx, w, 2)
        assert torch.equal(got, want)
    torch.cuda.synchronize()
    ll.heap.check_status()
    ref = _expected(x, idx, w, E, 2)
    tol = dict(rtol=1e-2, atol=5e-3) if dtype != torch.float32 else dict(rtol=1e-5, atol=1e-6)
    assert torch.allclose(got.float(), ref, **tol)


def test_out_of_range_expert_is_reported_not_written():
    from kernel_b200 import _native as N
    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    dev = torch.device("cuda")
    ctx = MoEAllToAll(8, 2, 128, 4, dtype=torch.bfloat16, device=dev)
    x, idx, w = _inputs(8, 2, 128, 4, torch.bfloat16, dev)
    idx[1, 0] = 99  # not an expert
    out = ctx.dispatch_scale_combine(x, idx, w, 0)
    torch.cuda.synchronize()
    with pytest.raises(N.NativeError, match="index out of bounds"):
        ctx.heap.check_status()
    assert torch.isfinite(out.float()).all()


def test_argument_validation():
    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    dev = torch.device("cuda")
    ctx = MoEAllToAll(8, 2, 128, 4, dtype=torch.bfloat16, device=dev)
    x, idx, w = _inputs(8, 2, 128, 4, torch.bfloat16, dev)
    with pytest.raises(ValueError):
        ctx.dispatch_scale_combine(x.float(), idx, w)
    with pytest.raises(ValueError):
        ctx.dispatch_scale_combine(x, idx.long(), w)
    x5, idx5, w5 = _inputs(8, 2, 128, 5, torch.bfloat16, dev)
    with pytest.raises(ValueError):
        ctx.dispatch_scale_combine(x5, idx5, w5)


def test_sentinel_and_guard_rows_after_dispatch(monkeypatch):
    """Poisoned workspace: every row the counts declare valid was written, nothing
    else was touched (the role a memory checker would play).  Runs the three-launch
    path, whose receive layout (rows grouped by expert) the check understands."""
    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    monkeypatch.setenv("KB200_A2A_FUSED", "0")

    E, k, H, T = 32, 4, 1024, 50
    dev = torch.device("cuda")
    ctx = MoEAllToAll(E, k, H, 64, dtype=torch.bfloat16, device=dev)  # capacity 256 rows, 200 used
    x, idx, w = _inputs(E, k, H, T, torch.bfloat16, dev, seed=9)
    ctx.poison_workspace()
    out = ctx.dispatch_scale_combine(x, idx, w, 2)
    torch.cuda.synchronize()
    ctx.heap.check_status()
    inside, outside = ctx.verify_workspace()
    assert inside == 0 and outside == 0
    assert torch.isfinite(out.float()).all()


@pytest.mark.parametrize("fused", ["1", "0"])
@pytest.mark.parametrize("E,k,T", [(2, 1, 3), (2, 2, 3), (4, 2, 2), (3, 3, 1)])
def test_every_routing_of_tiny_cases(E, k, T, fused, monkeypatch):
    """All ordered picks of k distinct experts for every token, one call each on the
    same workspace (an epoch per call): no slot combination is left untested at
    these sizes.  fp32, closed-form expectation."""
    import itertools

    from kernel_b200.ops.dispatch_combine import SCALE_EXPERT, MoEAllToAll, expert_scale_vector

    monkeypatch.setenv("KB200_A2A_FUSED", fused)
    dev = torch.device("cuda")
    H = 64
    ctx = MoEAllToAll(E, k, H, 4, dtype=torch.float32, device=dev)
    per_token = list(itertools.permutations(range(E), k))
    combos = list(itertools.product(per_token, repeat=T))
    g = torch.Generator(device=dev).manual_seed(E * 100 + k * 10 + T)
    x = torch.randn(T, H, device=dev, generator=g)
    w = torch.rand(T, k, device=dev, generator=g)
    scale = expert_scale_vector(E, 1, SCALE_EXPERT, dev)
    all_idx = torch.tensor(combos, dtype=torch.int32, device=dev)       # [combos, T, k]
    outs = [ctx.dispatch_scale_combine(x, all_idx[c].contiguous(), w, SCALE_EXPERT) for c in range(len(combos))]
    torch.cuda.synchronize()
    ctx.heap.check_status()
    got = torch.stack(outs)
    ref = x.unsqueeze(0) * (w.unsqueeze(0) * scale[all_idx.long()]).sum(-1, keepdim=True)
    assert torch.allclose(got, ref, rtol=1e-5, atol=1e-6)
    ctx.heap.close()
