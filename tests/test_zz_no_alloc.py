"""The allocation-free MoE round trip (`kb_a2a_round_trip_static`).

Some callers may not allocate device memory when they want to run the op: a
plug-in whose host application fixed its memory budget up front, a serving loop
that must stay out of the allocator, a process whose pool already owns all free
memory.  For them the library carries a built-in workspace.  This test calls the
entry point through its exported C symbol, twice in a row on the same workspace,
and compares both results with the regular entry point (which uses an allocated
symmetric workspace) and with the closed form of the round trip.  The kernels
check their inputs on the GPU after the call has returned, so a bad expert id
cannot come back as a return code: the second test reads it from the workspace's
status words through ``kb_a2a_static_status``, which allocates nothing either.
The file is collected last on purpose, and also passes when it is the only test
of a fresh process.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbol():
    from kernel_b200 import _native as N

    fn = N.lib().kb_a2a_round_trip_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                   C.c_void_p]
    return fn, N


def _status_symbol(N):
    fn = N.lib().kb_a2a_static_status
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
    return fn


def _closed_form(x, idx, w, E, mode):
    """out[t] = sum_k w[t,k] * bf16(scale(expert) * x[t]) in fp32."""
    from kernel_b200.ops.dispatch_combine import expert_scale_vector

    sc = expert_scale_vector(E, 1, mode, x.device)[idx.long()]
    y = (x.float().unsqueeze(1) * sc.unsqueeze(-1)).to(x.dtype).float()
    return (y * w.unsqueeze(-1)).sum(1)


def _inputs(E, k, H, T, dtype, dev, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(T, H, device=dev, generator=g).to(dtype)
    idx = torch.rand(T, E, device=dev, generator=g).argsort(1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, device=dev, generator=g), -1)
    return x, idx, w


@pytest.mark.parametrize("E,k,H,T,dtype,code,mode", [(64, 4, 1024, 100, torch.bfloat16, 0, 2), (16, 2, 512, 33, torch.float32, 2, 1)])
def test_static_workspace_matches_regular_entry_point_twice(E, k, H, T, dtype, code, mode):
    from kernel_b200.ops.dispatch_combine import MoEAllToAll

    fn, N = _symbol()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    regular = MoEAllToAll(E, k, H, T, dtype=dtype, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    tol = dict(rtol=1e-2, atol=5e-3) if dtype != torch.float32 else dict(rtol=1e-5, atol=1e-6)
    for call, seed in enumerate((5, 6)):  # two calls in a row, different data, same built-in workspace
        x, idx, w = _inputs(E, k, H, T, dtype, dev, seed)
        out = torch.empty_like(x)
        rc = fn(x.data_ptr(), idx.data_ptr(), w.data_ptr(), out.data_ptr(), T, E, k, H, code, mode, stream)
        assert rc == 0, N.last_error()
        expect = regular.dispatch_scale_combine(x, idx, w, mode)
        torch.cuda.synchronize()
        regular.heap.check_status()
        assert torch.allclose(out.float(), expect.float(), **tol), f"call {call}: max diff {(out.float() - expect.float()).abs().max()}"
        assert torch.allclose(out.float(), _closed_form(x, idx, w, E, mode), **tol), f"call {call}: differs from the closed form"
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    assert _status_symbol(N)(st.data_ptr(), 0, stream) == 0, N.last_error()
    torch.cuda.synchronize()
    assert st.cpu().tolist()[0] == 0  # healthy after valid calls
    regular.heap.close()


def test_static_workspace_reports_a_bad_expert_id_through_its_status_words():
    fn, N = _symbol()
    status_fn = _status_symbol(N)
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    E, k, H, T = 8, 2, 128, 4
    x, idx, w = _inputs(E, k, H, T, torch.bfloat16, dev, 7)
    idx[2, 1] = 99  # not an expert: the kernel must skip the copy and say so
    out = torch.empty_like(x)
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    assert status_fn(st.data_ptr(), 1, stream) == 0  # start from clean words
    assert fn(x.data_ptr(), idx.data_ptr(), w.data_ptr(), out.data_ptr(), T, E, k, H, 0, 0, stream) == 0
    assert status_fn(st.data_ptr(), 1, stream) == 0  # read, then clear
    torch.cuda.synchronize()
    words = st.cpu().tolist()
    assert words[0] == 3 and words[2] == 2 * k + 1  # KB_DEV_BAD_INDEX, entry (token 2, pick 1)
    assert torch.isfinite(out.float()).all()
    good = torch.ones(T, dtype=torch.bool)
    good[2] = False  # the other tokens are untouched by the bad entry
    x2, idx2 = x.clone(), idx.clone()
    idx2[2, 1] = 0
    assert torch.allclose(out.float()[good], _closed_form(x2, idx2, w, E, 0)[good], rtol=1e-2, atol=5e-3)
    assert status_fn(st.data_ptr(), 0, stream) == 0
    torch.cuda.synchronize()
    assert st.cpu().tolist()[0] == 0  # cleared by the previous read
    assert status_fn(None, 0, stream) == N.KB_ERR_ARG


def test_static_workspace_rejects_oversized_requests():
    fn, N = _symbol()
    dev = torch.device("cuda", 0)
    x = torch.zeros(8, 64, device=dev, dtype=torch.bfloat16)
    idx = torch.zeros(8, 2, device=dev, dtype=torch.int32)
    w = torch.zeros(8, 2, device=dev)
    out = torch.empty_like(x)
    # 4096 tokens * 8 * 7168 * 2 bytes is far beyond the 4 MiB per region
    rc = fn(x.data_ptr(), idx.data_ptr(), w.data_ptr(), out.data_ptr(), 4096, 256, 8, 7168, 0, 0, None)
    assert rc == N.KB_ERR_ARG and "exceeds the built-in workspace" in N.last_error()
    rc = fn(x.data_ptr(), idx.data_ptr(), w.data_ptr(), out.data_ptr(), 8, 4096, 2, 64, 0, 0, None)
    assert rc == N.KB_ERR_ARG
    rc = fn(None, idx.data_ptr(), w.data_ptr(), out.data_ptr(), 8, 8, 2, 64, 0, 0, None)
    assert rc == N.KB_ERR_ARG
