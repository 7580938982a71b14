"""Model-level blocks on one GPU against fp32 references."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_sequence_parallel_mlp_world1():
    from kernel_b200.models import SequenceParallelMLP

    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    tokens, hidden, ffn = 256, 512, 1024
    x = torch.randn(tokens, hidden, device=dev).to(torch.bfloat16)
    w1 = (torch.randn(ffn, hidden, device=dev) / hidden ** 0.5).to(torch.bfloat16)
    w2 = (torch.randn(hidden, ffn, device=dev) / ffn ** 0.5).to(torch.bfloat16)
    b1 = (torch.randn(ffn, device=dev) * 0.02).to(torch.bfloat16)
    b2 = (torch.randn(hidden, device=dev) * 0.02).to(torch.bfloat16)
    mlp = SequenceParallelMLP(tokens, hidden, w1, w2, b1, b2)
    y = mlp(x)
    torch.cuda.synchronize()
    ref = mlp.reference(x, w1, w2, b1, b2)
    assert y.shape == (tokens, hidden)
    assert torch.allclose(y.float(), ref, rtol=2e-2, atol=2e-2)


def test_moe_layer_world1():
    from kernel_b200.models import MoELayer

    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    E, k, H, F, T = 8, 2, 256, 512, 24
    w_up = (torch.randn(E, F, H, device=dev) / H ** 0.5).to(torch.bfloat16)
    w_down = (torch.randn(E, H, F, device=dev) / F ** 0.5).to(torch.bfloat16)
    layer = MoELayer(E, k, H, T, w_up, w_down)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    idx = torch.rand(T, E, device=dev).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, device=dev), -1)
    y = layer(x, idx, w)
    torch.cuda.synchronize()
    layer.a2a.heap.check_status()
    ref = layer._dense(x.cpu(), idx.cpu(), w.cpu())
    cpu_layer_ok = torch.allclose(y.float().cpu(), ref.float(), rtol=3e-2, atol=3e-2)
    assert cpu_layer_ok, (y.float().cpu() - ref.float()).abs().max()
    layer.close()


def _dense_grads(x_full, w1_full, b1_full, w2_full, b2, g_full):
    leaves = [t.detach().float().requires_grad_(True) for t in (x_full, w1_full, b1_full, w2_full, b2)]
    x, w1, b1, w2, bb2 = leaves
    y = torch.nn.functional.silu(x @ w1.t() + b1) @ w2.t() + bb2
    (y * g_full.float()).sum().backward()
    return y.detach(), [t.grad for t in leaves]


def _rel_err(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-6)


def test_trainable_mlp_forward_backward_world1():
    """Forward and backward of the sequence-parallel MLP on one GPU: every GEMM of
    both passes is the tcgen05 kernel (fused front-ends at world 1, plain GEMM for
    the weight gradients); compared with dense fp32 autograd."""
    from kernel_b200.models import TrainableSequenceParallelMLP
    from kernel_b200.ops import gemm as G

    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    tokens, hidden, ffn = 256, 512, 768
    mlp = TrainableSequenceParallelMLP(tokens, hidden, ffn, activation="silu", device=dev)
    with torch.no_grad():
        mlp.up.bias.normal_(std=0.05)
        mlp.down.bias.normal_(std=0.05)
    x = torch.randn(tokens, hidden, device=dev).to(torch.bfloat16).requires_grad_(True)
    g = torch.randn(tokens, hidden, device=dev).to(torch.bfloat16)
    before = G.launch_count
    y = mlp(x)
    (y.float() * g.float()).sum().backward()
    torch.cuda.synchronize()
    assert G.launch_count - before >= 6  # 2 forward, 2 input-gradient, 2 weight-gradient GEMMs (+ one-off tuning launches)
    y_ref, (dx, dw1, db1, dw2, db2) = _dense_grads(x, mlp.up.weight, mlp.up.bias, mlp.down.weight, mlp.down.bias, g)
    assert _rel_err(y, y_ref) < 3e-2
    assert _rel_err(x.grad, dx) < 4e-2
    assert _rel_err(mlp.up.weight.grad, dw1) < 4e-2
    assert _rel_err(mlp.up.bias.grad, db1) < 4e-2
    assert _rel_err(mlp.down.weight.grad, dw2) < 4e-2
    assert _rel_err(mlp.down.bias.grad, db2) < 4e-2
    mlp.close()


def test_trainable_moe_forward_backward_world1():
    """MoE block with backward on one GPU against dense fp32 autograd: the exchanges
    are the dispatch/combine kernels (also for the gradients), the GEMMs the tcgen05 kernel."""
    from kernel_b200.models import TrainableMoELayer

    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    E, k, H, F, T = 8, 2, 256, 384, 40
    layer = TrainableMoELayer(E, k, H, F, 64, device=dev)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16).requires_grad_(True)
    idx = torch.rand(T, E, device=dev).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, device=dev), -1).requires_grad_(True)
    gy = torch.randn(T, H, device=dev).to(torch.bfloat16)
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
    up = layer.w_up.detach().float().requires_grad_(True)
    down = layer.w_down.detach().float().requires_grad_(True)
    hid = torch.nn.functional.silu(torch.einsum("th,tkfh->tkf", xr, up[idx.long()]))
    yr = (torch.einsum("tkf,tkhf->tkh", hid, down[idx.long()]) * wr.unsqueeze(-1)).sum(1)
    (yr * gy.float()).sum().backward()
    assert _rel_err(y, yr.detach()) < 3e-2
    assert _rel_err(x.grad, xr.grad) < 5e-2
    assert _rel_err(w.grad, wr.grad) < 5e-2
    assert _rel_err(layer.w_up.grad, up.grad) < 5e-2
    assert _rel_err(layer.w_down.grad, down.grad) < 5e-2
    layer.close()
