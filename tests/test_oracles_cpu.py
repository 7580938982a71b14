"""Task oracles and the CPU paths of the ops on gloo ranks (no GPU)."""
import pytest
import torch

from _mp import run_ranks


def _a2a_config1(rank, world):
    """8 experts (4 per rank), top-2, hidden 256, 64 tokens per rank, fp32: after
    the round trip the output equals the local tokens times the weight sum."""
    from kernel_b200.baseline import all2all as base
    from kernel_b200.tasks.all2all import reference as R
    from kernel_b200.tasks.all2all import submission as S

    data = R.generate_input(8, 2, 256, 64, 11, rank, world, dtype="fp32", fixed_tokens=True, weight_mode="softmax",
                            expert_scale="identity", device="cpu")
    cfg, rd = data[0], data[1]
    assert rd.num_tokens == 64 and rd.indices.shape == (64, 2) and rd.x.dtype == torch.float32
    assert all(len(set(row)) == 2 for row in rd.indices.tolist())          # distinct experts per token
    assert torch.allclose(rd.weights.sum(-1), torch.ones(64), atol=1e-6)   # softmax weights
    expect = rd.x * rd.weights.sum(-1, keepdim=True)
    outs = {
        "fused_cpu_path": S.custom_kernel(data),
        "oracle": R.ref_kernel(data),
        "oracle_loop": R.ref_kernel_loop(data),
        "oracle_closed_form": R.ref_closed_form(data),
        "baseline": base.custom_kernel(data),
        "baseline_packed": base.custom_kernel_packed(data),
    }
    ok = {k: bool(torch.allclose(v, expect, rtol=1e-5, atol=1e-6)) for k, v in outs.items()}
    check = R.check_implementation(data, outs["fused_cpu_path"])
    bad = R.check_implementation(data, outs["fused_cpu_path"] + 0.1)
    return ok, check, bad[0]


def test_all2all_config1_round_trip_gloo_world2():
    for ok, check, bad in run_ranks(_a2a_config1, 2):
        assert all(ok.values()), ok
        assert check == (True, "")
        assert bad is False


def _a2a_compat(rank, world):
    """Reference-compatible mode: fp16, random token count, uniform weights,
    expert = x * (1 + owner rank)."""
    from kernel_b200.baseline import all2all as base
    from kernel_b200.tasks.all2all import reference as R
    from kernel_b200.tasks.all2all import submission as S

    data = R.generate_input(16, 4, 64, 9, 1234, rank, world, device="cpu")
    cfg, rd = data[0], data[1]
    assert cfg.in_dtype == torch.float16 and 1 <= rd.num_tokens < 9
    owner = (rd.indices.long() // (16 // world)).float()
    expect = rd.x.float() * (rd.weights * (1 + owner)).sum(-1, keepdim=True)
    res = {}
    for name, fn in [("oracle", R.ref_kernel), ("two_step", R.ref_kernel_two_step), ("loop", R.ref_kernel_loop), ("closed", R.ref_closed_form),
                     ("fused_cpu_path", S.custom_kernel), ("baseline", base.custom_kernel),
                     ("packed", base.custom_kernel_packed)]:
        out = fn(data)
        res[name] = (tuple(out.shape) == (rd.num_tokens, 64)) and bool(torch.allclose(out.float(), expect, rtol=1e-2, atol=5e-3))
    return res, rd.num_tokens


def test_all2all_reference_compatible_mode_gloo_world4():
    results = run_ranks(_a2a_compat, 4)
    assert len({n for _, n in results}) > 1  # token counts differ between ranks
    for res, _ in results:
        assert all(res.values()), res


def _gemm_rs(rank, world, bias_mode):
    import torch.distributed as dist

    from kernel_b200.baseline import gemm_rs as base
    from kernel_b200.tasks.gemm_rs import reference as R
    from kernel_b200.tasks.gemm_rs import submission as S
    from kernel_b200.tasks.gemm_rs import task

    data = R.generate_input(rank, world, 64, 48, 256, True, 21, dist="normal", bias_mode=bias_mode, device="cpu")
    a, w, bias = data
    assert a.shape == (64, 256 // world) and w.shape == (48, 256 // world) and bias.shape == (48,)
    assert task.bias_mode_of(data) == bias_mode and task.bias_mode_of((a, w, bias)) == "per_rank"  # plain tuple: default
    shards_a, shards_w = [None] * world, [None] * world
    dist.all_gather_object(shards_a, a)
    dist.all_gather_object(shards_w, w)
    truth = R.ref_fp32(shards_a, shards_w, bias, rank, bias_mode)
    out = S.custom_kernel(data)
    lib = base.custom_kernel(data)
    return (
        bool(torch.allclose(out.float(), truth, rtol=1e-2, atol=1e-2)),
        bool(torch.allclose(lib.float(), truth, rtol=2e-2, atol=2e-2)),
        R.check_implementation(data, out),
        tuple(out.shape),
        bool(torch.equal(shards_a[0], shards_a[1])),
    )


@pytest.mark.parametrize("bias_mode", ["once", "per_rank"])
def test_gemm_rs_bias_modes_gloo_world2(bias_mode):
    for ok, lib_ok, check, shape, same_inputs in run_ranks(_gemm_rs, 2, bias_mode):
        assert ok and lib_ok and check == (True, "")
        assert shape == (32, 48)
        assert not same_inputs  # per-rank seeds differ


def _gemm_rs_uniform_generator(rank, world):
    from kernel_b200.tasks.gemm_rs import reference as R

    a, w, bias = R.generate_input(rank, world, 16, 8, 64, True, 5, device="cpu")
    return float(a.abs().max()), float(w.abs().max()), bias.tolist()


def test_gemm_rs_uniform_inputs_and_shared_bias():
    res = run_ranks(_gemm_rs_uniform_generator, 2)
    for amax, wmax, _ in res:
        assert amax <= 0.01 + 1e-4 and wmax <= 0.01 + 1e-4  # +-0.01 as in the reference's generator
    assert res[0][2] == res[1][2]  # bias identical on every rank


def _ag_gemm(rank, world):
    import torch.distributed as dist

    from kernel_b200.tasks.ag_gemm import reference as R
    from kernel_b200.tasks.ag_gemm import submission as S

    data = R.generate_input(rank, world, 64, 96, 128, True, 9, device="cpu")
    a, w, bias = data
    assert a.shape == (64 // world, 128) and w.shape == (96 // world, 128)
    parts = [None] * world
    dist.all_gather_object(parts, a)
    truth = torch.cat(parts).float() @ w.float().t() + bias.float()
    out = S.custom_kernel(data)
    return bool(torch.allclose(out.float(), truth, rtol=1e-2, atol=1e-2)), R.check_implementation(data, out), tuple(out.shape)


def test_ag_gemm_gloo_world2():
    for ok, check, shape in run_ranks(_ag_gemm, 2):
        assert ok and check == (True, "") and shape == (64, 48)


def _two_step_buffers(rank, world):
    """dispatch returns expert-major padded buffers with consistent metadata."""
    from kernel_b200.tasks.all2all import reference as R

    data = R.generate_input(8, 2, 16, 6, 77, rank, world, dtype="fp32", fixed_tokens=True, device="cpu")
    cfg, rd = data[0], data[1]
    ata = R.PyTorchAllToAll(cfg, rank, world)
    num, ex, meta = ata.dispatch(rd.x, rd.indices)
    El = cfg.num_experts // world
    ok = num.shape == (El,) and ex.shape == (El, cfg.max_num_tokens * world, 16) and meta.shape[-1] == R.PyTorchAllToAll.META_DIM
    for le in range(El):
        m = meta[le, : int(num[le])]
        ok = ok and bool((m[:, 0] == rank * El + le).all())          # every row sits in its expert's buffer
        ok = ok and bool(((m[:, 1] >= 0) & (m[:, 1] < world)).all())
    import torch.distributed as dist
    total = num.sum().long().clone()
    dist.all_reduce(total)
    return bool(ok), int(total)


def test_two_step_dispatch_buffers_gloo_world2():
    res = run_ranks(_two_step_buffers, 2)
    assert all(ok for ok, _ in res)
    assert res[0][1] == 2 * 6 * 2  # every (token, k) copy landed exactly once


def _gemm_rs_one_rank_wrong(rank, world):
    """Rank 0 hands the checker a wrong shard, rank 1 a right one: both get their
    own verdict and both leave the checker (its collectives do not depend on the
    verdict), so the barrier behind it is reached."""
    import torch.distributed as dist

    from kernel_b200.tasks.gemm_rs import reference as R

    data = R.generate_input(rank, world, 64, 128, 256, True, seed=5)
    out = R.ref_kernel(data)
    if rank == 0:
        out = out + 1.0
    verdict = R.check_implementation(data, out)
    dist.barrier()
    return verdict[0]


def test_gemm_rs_checker_verdicts_may_differ_between_ranks():
    assert run_ranks(_gemm_rs_one_rank_wrong, 2, timeout=120) == [False, True]
