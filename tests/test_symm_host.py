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
