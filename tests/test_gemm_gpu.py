"""tcgen05 GEMM core against a plain fp32 torch reference (single GPU)."""
import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [
    (128, 256, 64),      # one tile, one k-block
    (256, 256, 64),      # one pair tile
    (384, 512, 192),     # odd number of 128-row blocks: the partner CTA of the last pair is all padding
    (128, 256, 256),     # one tile, ring wraps once
    (256, 512, 512),     # 2x2 tiles
    (128, 256, 48),      # K tail inside the first block
    (384, 768, 3696),    # flagship K_local, K tail 48
    (64, 2880, 360),     # M tail, N tail (2880 = 11*256 + 64)
    (1000, 1000, 1000),  # ragged everywhere (multiples of 8)
    (2048, 3696, 1024),  # N tail 112
    (4096, 4096, 4096),
]


def _ref(a, b, bias, scale):
    out = a.float() @ b.float().t()
    if bias is not None:
        out = out + scale * bias.float()
    return out


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("has_bias", [False, True])
@pytest.mark.parametrize("pair", [True, False])
def test_gemm_matches_fp32_reference(M, N, K, has_bias, pair):
    from kernel_b200.ops.gemm import gemm

    torch.manual_seed(M * 7 + N * 3 + K)
    dev = torch.device("cuda")
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
    bias = (torch.randn(N, device=dev) * 0.02).to(torch.bfloat16) if has_bias else None
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    out = gemm(a, b, bias, bias_scale=2.0 if has_bias else 1.0, status=status, pair=pair)
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0, f"device status {status.cpu().tolist()}"
    ref = _ref(a, b, bias, 2.0)
    err = (out.float() - ref).abs()
    tol = 1e-2 + 1e-2 * ref.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g}, bad {(err > tol).sum().item()} of {err.numel()}"


def test_gemm_rejects_bad_shapes():
    from kernel_b200 import _native as N
    from kernel_b200.ops.gemm import gemm

    dev = torch.device("cuda")
    a = torch.zeros(128, 60, device=dev, dtype=torch.bfloat16)
    b = torch.zeros(256, 60, device=dev, dtype=torch.bfloat16)
    with pytest.raises(N.NativeError):
        gemm(a, b)


def test_gemm_few_ctas_exercises_persistent_loop():
    from kernel_b200.ops.gemm import gemm

    torch.manual_seed(5)
    dev = torch.device("cuda")
    a = torch.randn(1024, 512, device=dev).to(torch.bfloat16)
    b = (torch.randn(1024, 512, device=dev) / 512 ** 0.5).to(torch.bfloat16)
    ref = _ref(a, b, None, 1.0)
    for pair, ctas in ((False, 3), (True, 2), (True, 6)):  # few CTAs: both accumulators, many ring wraps
        out = gemm(a, b, num_ctas=ctas, pair=pair)
        torch.cuda.synchronize()
        assert torch.allclose(out.float(), ref, rtol=1e-2, atol=1e-2), (pair, ctas)
