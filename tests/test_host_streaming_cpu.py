"""``run_from_host`` of the two fused GEMM front-ends on CPU ranks: the chunked
row bookkeeping (which rows of the host tensors form which sub-problem) against
the un-chunked call.  The overlap of copies and kernels needs a GPU and is
covered by the GPU tests; the arithmetic of the split does not."""
import pytest
import torch

from _mp import run_ranks


def _rs(rank, world, M, Nn, Kl, chunks):
    from kernel_b200.ops.gemm import GemmRS

    ctx = GemmRS(M, Nn, device="cpu")
    g = torch.Generator().manual_seed(5 + rank)
    a = torch.randn(M, Kl, generator=g).to(torch.bfloat16)
    w = (torch.randn(Nn, Kl, generator=g) / Kl ** 0.5).to(torch.bfloat16)
    bias = (torch.randn(Nn, generator=torch.Generator().manual_seed(1)) * 0.1).to(torch.bfloat16)
    whole = ctx(a, w, bias, bias_scale=2.0)
    streamed = ctx.run_from_host(a, w, bias, bias_scale=2.0, chunks=chunks)
    again = ctx.run_from_host(a, w, bias, bias_scale=2.0, out_host=torch.empty_like(streamed), chunks=chunks)
    ctx.close()
    return bool(torch.equal(whole, streamed)), bool(torch.equal(streamed, again)), tuple(streamed.shape)


def _ag(rank, world, M, Nl, K, chunks):
    from kernel_b200.ops.gemm import AGGemm

    ctx = AGGemm(M, K, device="cpu")
    g = torch.Generator().manual_seed(9 + rank)
    a = torch.randn(M // world, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(Nl, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    bias = (torch.randn(Nl, generator=g) * 0.1).to(torch.bfloat16)
    whole = ctx(a, w, bias)
    streamed = ctx.run_from_host(a, w, bias, chunks=chunks)
    ctx.close()
    return bool(torch.equal(whole, streamed)), True, tuple(streamed.shape)


@pytest.mark.parametrize("world,M,chunks", [(1, 512, 4), (2, 1024, 4), (2, 512, 3), (4, 1024, 2)])
def test_gemm_rs_streamed_equals_whole(world, M, chunks):
    for same, repeat, shape in run_ranks(_rs, world, M, 264, 40, chunks):
        assert same and repeat and shape == (M // world, 264)


@pytest.mark.parametrize("world,M,chunks", [(1, 512, 4), (2, 1024, 4), (4, 1024, 2)])
def test_ag_gemm_streamed_equals_whole(world, M, chunks):
    for same, _, shape in run_ranks(_ag, world, M, 136, 72, chunks):
        assert same and shape == (M, 136)
