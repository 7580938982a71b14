"""Bounded device-side waits: a flag that nothing sets makes the kernel give up
after its limit and report a status; the context stays usable."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_on_unset_flag_times_out_and_context_survives():
    from kernel_b200 import _native as N

    dev = torch.device("cuda")
    flags = torch.zeros(4, dtype=torch.int32, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.time()
    N.check(N.lib().kb_wait_flags(flags.data_ptr(), 4, 1, 5_000_000, status.data_ptr(), stream))  # 5 ms limit
    torch.cuda.synchronize()
    assert time.time() - t0 < 2.0
    st = status.cpu().tolist()
    assert st[0] == 2 and st[3] == 1  # flag timeout, epoch 1
    # the GPU still answers
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    # a set flag passes immediately and leaves the status clean
    status.zero_()
    flags.fill_(3)
    N.check(N.lib().kb_wait_flags(flags.data_ptr(), 4, 3, 5_000_000, status.data_ptr(), stream))
    torch.cuda.synchronize()
    assert status.cpu().tolist()[0] == 0


def test_heap_barrier_and_status_on_one_rank():
    from kernel_b200.parallel.symm import SymmHeap

    heap = SymmHeap(1 << 20)
    assert heap.backend in ("vmm", "ipc") and heap.world == 1
    off = heap.alloc(4096)
    t = heap.tensor(off, (1024,), torch.float32)
    assert float(t.abs().sum()) == 0.0  # segments start zeroed
    t.fill_(1.5)
    heap.barrier()
    torch.cuda.synchronize()
    heap.check_status()
    assert float(heap.tensor(off, (1024,), torch.float32, peer=0).sum()) == 1536.0
    heap.close()


def test_ipc_backend_single_rank():
    from kernel_b200.parallel.symm import SymmHeap

    heap = SymmHeap(1 << 20, backend="ipc")
    assert heap.backend == "ipc"
    t = heap.tensor(heap.alloc(64), (16,), torch.int32)
    t.fill_(7)
    torch.cuda.synchronize()
    assert int(t.sum()) == 112
    heap.close()
