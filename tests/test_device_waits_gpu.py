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
    N.check(N.lib().kb_wait_flags(flags.data_ptr(), 4, 1, 1, 5_000_000, status.data_ptr(), stream))  # 5 ms limit
    torch.cuda.synchronize()
    assert time.time() - t0 < 2.0
    st = status.cpu().tolist()
    assert st[0] == 2 and st[3] == 1  # flag timeout, epoch 1
    # the GPU still answers
    assert float((torch.ones(8, device=dev) * 2).sum()) == 16.0
    # a set flag passes immediately and leaves the status clean
    status.zero_()
    flags.fill_(3)
    N.check(N.lib().kb_wait_flags(flags.data_ptr(), 4, 1, 3, 5_000_000, status.data_ptr(), stream))
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


def test_context_works_again_after_a_wait_ran_out(monkeypatch):
    """A combine whose expert-output flag nothing sets gives up after 5 ms and
    reports it; ``recover()`` brings the context back and the next round trip is
    right."""
    import ctypes as C

    from kernel_b200 import _native as N
    from kernel_b200.ops import dispatch_combine as dc

    monkeypatch.setattr(dc, "_WAIT_LIMIT_NS", 5_000_000)
    dev = torch.device("cuda")
    E, k, H, T = 16, 2, 256, 24
    ctx = dc.MoEAllToAll(E, k, H, T, dtype=torch.bfloat16, device=dev)
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    idx = torch.rand(T, E, device=dev, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, device=dev, generator=g), -1)
    good = ctx.dispatch_scale_combine(x, idx, w, dc.SCALE_EXPERT)
    torch.cuda.synchronize()
    ctx.heap.check_status()
    # a combine of a call whose expert pass never ran: its flag keeps the old epoch
    ctx.epoch += 1
    out = torch.empty_like(x)
    a = ctx._args(x, idx, w, out, dc.SCALE_EXPERT)
    t0 = time.time()
    N.check(N.lib().kb_a2a_combine(C.byref(a), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert time.time() - t0 < 2.0
    with pytest.raises(N.SymmTimeoutError):
        ctx.heap.check_status()
    ctx.recover()
    again = ctx.dispatch_scale_combine(x, idx, w, dc.SCALE_EXPERT)
    torch.cuda.synchronize()
    ctx.heap.check_status()
    assert torch.equal(again, good)
    ctx.heap.close()
