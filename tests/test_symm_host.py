"""Host side of the symmetric-memory layer, without a GPU: descriptor exchange,
peer mapping, barriers and the failure paths (a rank that never joins, a rank
that dies, an exhausted heap).  Failures are made on the host only."""
import ctypes as C
import os
import time

import pytest
import torch

from _mp import run_ranks
from kernel_b200 import _native as N


def _exchange(rank, world, session):
    lib = N.lib()
    mine = os.memfd_create(f"kb200-test-{rank}")
    os.write(mine, f"hello from {rank}".encode())
    fds = (C.c_int * world)()
    N.check(lib.kb_fd_allgather(session.encode(), b"t", rank, world, mine, fds, 20000))
    got = [os.pread(fds[p], 64, 0).decode() if p != rank else None for p in range(world)]
    for fd in list(fds) + [mine]:
        if fd >= 0:
            os.close(fd)
    return got


def test_fd_allgather_passes_descriptors():
    world = 3
    res = run_ranks(_exchange, world, f"s{os.getpid()}")
    for rank, got in enumerate(res):
        for p in range(world):
            if p != rank:
                assert got[p] == f"hello from {p}"


def _heap(rank, world):
    from kernel_b200.parallel.symm import SymmHeap

    heap = SymmHeap(1 << 20, backend="host")
    assert heap.nbytes >= (1 << 20) and heap.world == world
    off = heap.alloc(4096)
    assert off % 256 == 0 and off >= 4096
    mine = heap.tensor(off, (1024,), torch.int32)
    mine.fill_(100 + rank)
    heap.barrier()
    seen = [int(heap.tensor(off, (1024,), torch.int32, peer=p)[17]) for p in range(world)]
    heap.barrier()
    # a store into a peer's segment is visible to the peer
    heap.tensor(off, (1024,), torch.int32, peer=(rank + 1) % world)[0] = 7000 + rank
    heap.barrier()
    from_left = int(mine[0])
    with pytest.raises(MemoryError):
        heap.alloc(1 << 30)
    heap.close()
    return seen, from_left


def test_host_heap_peer_views_and_barrier():
    world = 2
    res = run_ranks(_heap, world)
    for rank, (seen, from_left) in enumerate(res):
        assert seen == [100, 101]
        assert from_left == 7000 + (rank - 1) % world


def test_fd_allgather_times_out_when_a_peer_never_joins():
    lib = N.lib()
    fds = (C.c_int * 2)()
    t0 = time.time()
    code = lib.kb_fd_allgather(f"lonely{os.getpid()}".encode(), b"t", 0, 2, -1, fds, 300)
    assert code == N.KB_ERR_TIMEOUT and time.time() - t0 < 5
    with pytest.raises(N.SymmTimeoutError):
        N.check(code)
    assert "timed out" in N.last_error()


def _barrier_with_dead_peer(rank, world):
    from kernel_b200.parallel.symm import SymmHeap

    heap = SymmHeap(1 << 16, backend="host", timeout_s=0.5)
    heap.barrier()
    if rank == 1:
        return "left"  # leaves between steps, nothing in flight
    try:
        heap.barrier()
    except N.SymmTimeoutError as e:
        return f"timeout: {e}"
    return "no error"


def test_host_barrier_reports_a_rank_that_left():
    res = run_ranks(_barrier_with_dead_peer, 2)
    assert res[1] == "left" and res[0].startswith("timeout") and "rank 1" in res[0]


def test_bad_arguments_are_rejected_with_a_message():
    lib = N.lib()
    h = C.c_void_p()
    assert lib.kb_symm_create(N.BACKEND_HOST, 3, 2, 4096, 0, C.byref(h)) == N.KB_ERR_ARG
    assert "bad arguments" in N.last_error()
    assert lib.kb_symm_create(99, 0, 1, 4096, 0, C.byref(h)) == N.KB_ERR_ARG


def _moe_over_host_heap(rank, world, dtype_name):
    """The MoE round trip of CPU ranks runs the kernels' protocol (slots, peer
    stores, epoch flags, pull combine) over the memfd-backed heap."""
    import torch

    from kernel_b200.ops.dispatch_combine import SCALE_EXPERT, MoEAllToAll, expert_scale_vector

    dtype = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}[dtype_name]
    E = 18 if 18 % world == 0 else 3 * world
    k, H, T = 4, 64, 5 + rank  # token counts differ between ranks
    ctx = MoEAllToAll(E, k, H, 16, dtype=dtype, device="cpu")
    assert ctx.host_heap and ctx.heap.backend == "host"
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(T, H, generator=g).to(dtype)
    idx = torch.rand(T, E, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, generator=g), -1)
    outs = [ctx.dispatch_scale_combine(x, idx, w, SCALE_EXPERT) for _ in range(3)]  # three epochs on one workspace
    sc = expert_scale_vector(E, world, SCALE_EXPERT)[idx.long()]
    y = (x.float().unsqueeze(1) * sc.unsqueeze(-1)).to(dtype).float()
    ref = (y * w.unsqueeze(-1)).sum(1)
    tol = dict(rtol=1e-5, atol=1e-6) if dtype == torch.float32 else dict(rtol=1e-2, atol=5e-3)
    ok = all(torch.allclose(o.float(), ref, **tol) for o in outs) and torch.equal(outs[0], outs[2])
    ctx.heap.close()
    return bool(ok)


@pytest.mark.parametrize("dtype_name", ["fp32", "bf16", "fp16"])
def test_moe_round_trip_over_host_heap(dtype_name):
    assert all(run_ranks(_moe_over_host_heap, 3, dtype_name))


def test_moe_round_trip_over_host_heap_world8():
    assert all(run_ranks(_moe_over_host_heap, 8, "bf16", timeout=300))


def _moe_with_absent_rank(rank, world):
    import torch

    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    ctx = MoEAllToAll(8, 2, 32, 4, dtype=torch.float32, device="cpu")
    x = torch.randn(4, 32)
    idx = torch.tensor([[0, 5], [1, 4], [2, 7], [3, 6]], dtype=torch.int32)
    w = torch.full((4, 2), 0.5)
    ctx.dispatch_scale_combine(x, idx, w)  # epoch 1: everybody takes part
    if rank == 1:
        return "absent"  # epoch 2: this rank never calls
    try:
        ctx.dispatch_scale_combine(x, idx, w)
    except N.SymmTimeoutError as e:
        return str(e)
    return "no error"


@pytest.mark.parametrize("low_latency,message", [("0", "rank 1 never finished its dispatch of epoch 2"),
                                                 ("1", "rank 1 never sent its counts of epoch 2")])
def test_moe_wait_names_the_rank_that_never_arrived(low_latency, message):
    """Both host protocols (flag hand-offs; flags inside the data, the default for so
    small a context) end the wait for a missing rank with its number."""
    res = run_ranks(_moe_with_absent_rank, 2, env={"KB200_WAIT_LIMIT_MS": "300", "KB200_A2A_LL": low_latency})
    assert res[1] == "absent"
    assert message in res[0]


def _moe_recovers_after_a_late_rank(rank, world):
    """Rank 1 sits out one call, so rank 0's wait runs out; both then call
    ``recover()`` (rank 1 is one call behind: the ranks agree on the largest call
    number) and the next round trip is right on both."""
    import time

    import torch
    import torch.distributed as dist

    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    ctx = MoEAllToAll(8, 2, 32, 4, dtype=torch.float32, device="cpu")
    g = torch.Generator().manual_seed(rank)
    x = torch.randn(4, 32, generator=g)
    idx = torch.tensor([[0, 5], [1, 4], [2, 7], [3, 6]], dtype=torch.int32)
    w = torch.full((4, 2), 0.5)
    first = ctx.dispatch_scale_combine(x, idx, w)
    timed_out = False
    if rank == 0:
        try:
            ctx.dispatch_scale_combine(x, idx, w)
        except N.SymmTimeoutError:
            timed_out = True
    else:
        time.sleep(0.8)  # longer than the wait limit: rank 0 gives up meanwhile
    dist.barrier()
    ctx.recover()
    again = ctx.dispatch_scale_combine(x, idx, w)
    ok = bool(torch.allclose(again, first)) and bool(torch.allclose(again, x))  # weights sum to one, identity expert
    ctx.heap.close()
    return timed_out, ok


def test_moe_context_recovers_after_a_wait_ran_out():
    res = run_ranks(_moe_recovers_after_a_late_rank, 2, env={"KB200_WAIT_LIMIT_MS": "300"})
    assert res[0] == (True, True) and res[1] == (False, True)


def test_multicast_probe_and_entry_points_fail_cleanly_without_a_device():
    """No driver, no multicast: the probe says no and the set-up entry points refuse
    a heap that is not a VMM heap, instead of touching the driver."""
    lib = N.lib()
    assert lib.kb_symm_mc_supported(0) == 0
    h = C.c_void_p()
    assert lib.kb_symm_create(N.BACKEND_HOST, 0, 1, 4096, 0, C.byref(h)) == N.KB_OK
    fd = C.c_int(-1)
    assert lib.kb_symm_mc_create(h, C.byref(fd)) == N.KB_ERR_ARG and fd.value == -1
    assert not lib.kb_symm_mc_ptr(h)
    lib.kb_symm_destroy(h)


def _host_heap_with_nvls_requested(rank, world):
    from kernel_b200.parallel.symm import SymmHeap

    heap = SymmHeap(1 << 16, backend="host", nvls=True)   # asked for, not available on a host heap
    ok = heap.mc_ptr is None and heap.backend == "host"
    heap.close()
    return ok


def test_nvls_request_on_host_heap_is_ignored():
    assert all(run_ranks(_host_heap_with_nvls_requested, 2))
