"""Argument checks of the device entry points that run before any CUDA call: a bad
problem is refused with a message, on a machine without a GPU too."""
import ctypes as C

import pytest

from kernel_b200 import _native as N


def _args(**kw):
    a = N.GemmArgs()
    buf = C.create_string_buffer(4096 + 16)
    base = (C.addressof(buf) + 15) & ~15
    a.mode, a.M, a.N, a.K = N.GEMM_PLAIN, 128, 256, 64
    a.A = a.B = a.out = base
    a.rank, a.world, a.epoch = 0, 1, 1
    for k, v in kw.items():
        setattr(a, k, v)
    a._keepalive = buf
    return a, base


@pytest.mark.parametrize("kw,needle", [
    (dict(M=0), "need M,N,K > 0"),
    (dict(K=60), "multiples of 8"),
    (dict(N=100), "multiples of 8"),
    (dict(world=0), "bad rank/world"),
    (dict(world=2, rank=2), "bad rank/world"),
    (dict(world=N.KB_MAX_WORLD + 1), "bad rank/world"),
])
def test_gemm_refuses_bad_problem(kw, needle):
    a, _ = _args(**kw)
    assert N.lib().kb_gemm(C.byref(a), None) == N.KB_ERR_ARG
    assert needle in N.last_error()


def test_gemm_refuses_misaligned_operands():
    a, base = _args()
    a.B = base + 8
    assert N.lib().kb_gemm(C.byref(a), None) == N.KB_ERR_ARG
    assert "16-byte aligned" in N.last_error()
    a, base = _args()
    a.bias = base + 2
    assert N.lib().kb_gemm(C.byref(a), None) == N.KB_ERR_ARG


@pytest.mark.parametrize("mode", [N.GEMM_RS, N.GEMM_AG])
def test_fused_gemm_refuses_bad_sharding(mode):
    lib = N.lib()
    a, _ = _args(mode=mode, world=3, rank=0, M=128)
    assert lib.kb_gemm(C.byref(a), None) == N.KB_ERR_ARG and "divisible by world" in N.last_error()
    a, _ = _args(mode=mode, world=2, rank=0, M=192)      # 96 rows per rank
    assert lib.kb_gemm(C.byref(a), None) == N.KB_ERR_ARG and "rows per rank" in N.last_error()
    a, _ = _args(mode=mode, world=2, rank=1, M=256)      # no peer segments given
    assert lib.kb_gemm(C.byref(a), None) == N.KB_ERR_ARG and "peer_base[0] is null" in N.last_error()


def test_null_argument_block():
    assert N.lib().kb_gemm(None, None) == N.KB_ERR_ARG
    assert N.lib().kb_gemm_host(None, 1) == N.KB_ERR_ARG
    assert N.lib().kb_a2a_round_trip_host(None, 1) == N.KB_ERR_ARG
    assert N.lib().kb_a2a_dispatch_host(None, 1) == N.KB_ERR_ARG
    assert N.lib().kb_a2a_combine_host(None, 1) == N.KB_ERR_ARG


def test_schedule_refuses_bad_problem():
    lib = N.lib()
    blk, nb = C.c_int(), C.c_int()
    assert lib.kb_gemm_schedule(N.GEMM_RS, 100, 256, 0, 3, 0, 0, C.byref(blk), C.byref(nb)) == -1    # M % world
    assert lib.kb_gemm_schedule(N.GEMM_RS, 256, 256, 2, 2, 0, 0, C.byref(blk), C.byref(nb)) == -1    # rank out of range
    assert lib.kb_gemm_schedule(N.GEMM_AG, 256, 256, 0, 2, 1, 0, C.byref(blk), C.byref(nb)) == -1    # pairs need 256-row shards
