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
