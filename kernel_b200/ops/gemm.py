"""Front-ends of the tcgen05 GEMM family: plain GEMM, GEMM + reduce-scatter and
all-gather + GEMM.

On CUDA tensors these always launch the hand-written sm_100a kernel
(``csrc/kernels/gemm_sm100.cu``); there is no library fallback on a GPU.  CPU
tensors take a torch reference path (``torch.matmul`` plus gloo collectives) so
that host-side logic can be tested without a GPU; with more than one CPU rank the
fused ops run the kernels' protocol over a host-backed symmetric heap.

Counterparts in the reference: ``gemm_rs/submission.py:5-29`` (matmul, bias add,
``reduce_scatter_tensor``).  The all-gather variant has no counterpart there.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch
import torch.distributed as dist

from .. import _native as N
from ..parallel.symm import SymmHeap, _dist_info

_WAIT_LIMIT_NS = int(float(os.environ.get("KB200_WAIT_LIMIT_MS", "2000")) * 1e6)

launch_count = 0  # kernels launched by this module (bench accounting)


def _check_bf16_2d(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.bfloat16 or t.dim() != 2 or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous 2-D bf16 tensor")


def _launch(args: N.GemmArgs, device: torch.device) -> None:
    global launch_count
    stream = torch.cuda.current_stream(device).cuda_stream
    code = N.lib().kb_gemm(C.byref(args), stream)
    if code:
        N.check(code)
    launch_count += 1


def _cpu_heap_path() -> bool:
    """CPU ranks run the kernels' protocol over a memfd-backed symmetric heap
    (``csrc/symm/gemm_host.cpp``) unless ``KB200_GEMM_CPU_PATH=collectives`` selects
    torch matmul + gloo collectives."""
    return os.environ.get("KB200_GEMM_CPU_PATH", "heap") == "heap"


def _new_heap(nbytes: int, group, device, native: bool) -> SymmHeap:
    if native:
        return SymmHeap(nbytes, group=group, device=device)
    return SymmHeap(nbytes, group=group, backend="host", timeout_s=_WAIT_LIMIT_NS / 1e9 + 5)


def _host_args(ctx, mode: int, M: int, Nn: int, K: int, a, w, bias, bias_scale: float, out) -> N.GemmArgs:
    args = N.GemmArgs()
    args.mode = mode
    args.M, args.N, args.K = M, Nn, K
    args.A, args.B, args.out = a.data_ptr(), w.data_ptr(), out.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    args.bias_scale = bias_scale
    args.rank, args.world, args.epoch = ctx.rank, ctx.world, ctx.epoch
    args.peer_base = ctx.heap.peer_array()
    args.data_off, args.flag_off = ctx.data_off, ctx.flag_off
    args.wait_limit_ns = _WAIT_LIMIT_NS
    return args


def _rows_bad(rpo: int) -> bool:
    """The tile schedule needs the rows per rank to divide, or be a multiple of, the 128-row block."""
    return rpo <= 0 or (rpo % 128 != 0 and 128 % rpo != 0)


_NO_PAIR_BIT = 1 << 30
_pair_choice: dict = {}  # (M, N, K) -> True if the CTA-pair kernel is the faster one on this device


def _tuned_pair(args: N.GemmArgs, device: torch.device) -> bool:
    """Single-rank calls pick between the two tile configurations by timing both
    once per shape (three alternating launches each, CUDA events); which one wins depends on
    the shape (pairs win at K around 4096, the single-CTA kernel at very large K)."""
    key = (args.M, args.N, args.K)
    hit = _pair_choice.get(key)
    if hit is not None:
        return hit
    if args.M < 256 or os.environ.get("KB200_GEMM_NO_PAIR") == "1":
        _pair_choice[key] = False
        return False
    base = args.num_ctas & ~_NO_PAIR_BIT
    times = {True: 0.0, False: 0.0}

    def run(use_pair: bool) -> None:
        args.num_ctas = base | (0 if use_pair else _NO_PAIR_BIT)
        _launch(args, device)

    for use_pair in (True, False, True, False):  # warm up both; the clocks settle under load
        run(use_pair)
    # Alternate the two so that neither is measured on a cooler, faster-clocked GPU.
    for _ in range(3):
        for use_pair in (True, False):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            run(use_pair)
            e1.record()
            e1.synchronize()
            times[use_pair] += e0.elapsed_time(e1)
    args.num_ctas = base
    _pair_choice[key] = times[True] <= times[False]
    return _pair_choice[key]


def gemm(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
         bias_scale: float = 1.0, status: Optional[torch.Tensor] = None, num_ctas: int = 0,
         pair: Optional[bool] = None) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ b[N,K]^T (+ bias_scale * bias)`` in bf16 with fp32 accumulation.

    ``pair=True`` uses clusters of two CTAs sharing 256x256 tiles (``cta_group::2``,
    M >= 256), ``pair=False`` the single-CTA 128x256 kernel, ``None`` times both
    once per shape and keeps the faster."""
    _check_bf16_2d(a, "a")
    _check_bf16_2d(b, "b")
    M, K = a.shape
    Nn = b.shape[0]
    if b.shape[1] != K:
        raise ValueError("inner dimensions differ")
    if not a.is_cuda:
        res = a.float() @ b.float().t()
        if bias is not None:
            res = res + bias_scale * bias.float()
        res = res.to(torch.bfloat16)
        if out is not None:
            out.copy_(res)
            return out
        return res
    if out is None:
        out = torch.empty((M, Nn), dtype=torch.bfloat16, device=a.device)
    args = N.GemmArgs()
    args.mode = N.GEMM_PLAIN
    args.M, args.N, args.K = M, Nn, K
    args.A, args.B, args.out = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    args.bias_scale = bias_scale
    args.rank, args.world, args.epoch = 0, 1, 1
    args.status = status.data_ptr() if status is not None else None
    args.wait_limit_ns = _WAIT_LIMIT_NS
    args.num_ctas = num_ctas
    if pair is None:
        pair = _tuned_pair(args, a.device)
    args.num_ctas = num_ctas | (0 if pair else _NO_PAIR_BIT)
    _launch(args, a.device)
    return out


class GemmRS:
    """GEMM fused with reduce-scatter for one problem shape.

    Each rank holds ``a[M, K_local]`` and ``w[N, K_local]``; the result
    ``sum_r a_r @ w_r^T (+ bias_scale * bias)`` is row-scattered so that this
    rank returns rows ``[rank*M/world, (rank+1)*M/world)``.  Construction is
    collective (it allocates symmetric staging memory); calls are collective in
    the sense that every rank must make the same sequence of calls.
    """

    def __init__(self, M: int, Nn: int, group=None, device: Optional[torch.device] = None, heap: Optional[SymmHeap] = None):
        self.M, self.N = M, Nn
        self.group = group
        self.rank, self.world = _dist_info(group)
        if M % self.world:
            raise ValueError("M must be divisible by the world size")
        self.native = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.epoch = 0
        self.heap = None
        self._hot = None
        self.host_heap = not self.native and self.world > 1 and _cpu_heap_path() and not _rows_bad(M // self.world)
        if (self.native and self.world > 1) or self.host_heap:
            lib = N.lib()
            data = int(lib.kb_gemm_rs_data_bytes(M, Nn, self.world))
            flags = int(lib.kb_gemm_rs_flag_bytes(M, Nn, self.world))
            self.heap = heap or _new_heap(data + flags + 1024, group, device, self.native)
            self.data_off = self.heap.alloc(data)
            self.flag_off = self.heap.alloc(flags)
            self.status = self.heap.status
        elif self.native:
            self.status = torch.zeros(8, dtype=torch.int32, device=device or torch.device("cuda", torch.cuda.current_device()))

    def __call__(self, a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, bias_scale: float = 1.0,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _check_bf16_2d(a, "a")
        _check_bf16_2d(w, "w")
        M, K = a.shape
        if M != self.M or w.shape[0] != self.N or w.shape[1] != K:
            raise ValueError("shape does not match this GemmRS context")
        rows = M // self.world
        if not a.is_cuda and self.host_heap:
            if out is None:
                out = torch.empty((rows, self.N), dtype=torch.bfloat16)
            self.epoch += 1
            args = _host_args(self, N.GEMM_RS, M, self.N, K, a, w, bias, bias_scale, out)
            N.check(N.lib().kb_gemm_host(C.byref(args), max(1, _WAIT_LIMIT_NS // 1_000_000)))
            return out
        if not a.is_cuda:
            full = a.float() @ w.float().t()
            full = full.to(torch.bfloat16)
            res = torch.empty((rows, self.N), dtype=torch.bfloat16)
            if self.world > 1:
                dist.reduce_scatter_tensor(res, full, group=self.group)
            else:
                res.copy_(full)
            if bias is not None:
                res = (res.float() + bias_scale * bias.float()).to(torch.bfloat16)
            if out is not None:
                out.copy_(res)
                return out
            return res
        if out is None:
            out = torch.empty((rows, self.N), dtype=torch.bfloat16, device=a.device)
        self.epoch += 1
        args = self._hot
        if args is None:  # built once; calls only refresh pointers, K and the epoch
            args = self._hot = N.GemmArgs()
            args.mode = N.GEMM_RS
            args.M, args.N = M, self.N
            args.rank, args.world = self.rank, self.world
            if self.heap is not None:
                args.peer_base = self.heap.peer_array()
                args.data_off, args.flag_off = self.data_off, self.flag_off
            args.status = self.status.data_ptr()
            args.wait_limit_ns = _WAIT_LIMIT_NS
        args.K = K
        args.A, args.B, args.out = a.data_ptr(), w.data_ptr(), out.data_ptr()
        args.bias = bias.data_ptr() if bias is not None else None
        args.bias_scale = bias_scale
        args.epoch = self.epoch
        if self.world == 1:
            args.num_ctas = 0
            args.num_ctas = 0 if _tuned_pair(args, a.device) else _NO_PAIR_BIT
        _launch(args, a.device)
        return out


class AGGemm:
    """All-gather fused with GEMM for one problem shape.

    Each rank holds ``a_local[M/world, K]`` and a column shard ``w[N_local, K]``;
    returns ``all_gather(a_local) @ w^T (+ bias)`` of shape ``[M, N_local]``.
    """

    def __init__(self, M: int, K: int, group=None, device: Optional[torch.device] = None, heap: Optional[SymmHeap] = None):
        self.M, self.K = M, K
        self.group = group
        self.rank, self.world = _dist_info(group)
        if M % self.world:
            raise ValueError("M must be divisible by the world size")
        self.native = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.epoch = 0
        self.heap = None
        self._hot = None
        self.host_heap = not self.native and self.world > 1 and _cpu_heap_path() and not _rows_bad(M // self.world)
        if (self.native and self.world > 1) or self.host_heap:
            lib = N.lib()
            data = int(lib.kb_gemm_ag_data_bytes(M, K))
            flags = int(lib.kb_gemm_ag_flag_bytes(M, self.world))
            ctr = int(lib.kb_gemm_ag_counter_bytes(M, self.world))
            self.heap = heap or _new_heap(data + flags + ctr + 2048, group, device, self.native)
            self.data_off = self.heap.alloc(data)
            self.flag_off = self.heap.alloc(flags)
            self.counter_off = self.heap.alloc(ctr)
            self.status = self.heap.status
        elif self.native:
            self.status = torch.zeros(8, dtype=torch.int32, device=device or torch.device("cuda", torch.cuda.current_device()))

    def __call__(self, a_local: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                 out: Optional[torch.Tensor] = None) -> torch.Tensor:
        _check_bf16_2d(a_local, "a_local")
        _check_bf16_2d(w, "w")
        rows, K = a_local.shape
        if rows * self.world != self.M or K != self.K or w.shape[1] != K:
            raise ValueError("shape does not match this AGGemm context")
        Nl = w.shape[0]
        if not a_local.is_cuda and self.host_heap:
            if out is None:
                out = torch.empty((self.M, Nl), dtype=torch.bfloat16)
            self.epoch += 1
            args = _host_args(self, N.GEMM_AG, self.M, Nl, K, a_local, w, bias, 1.0, out)
            N.check(N.lib().kb_gemm_host(C.byref(args), max(1, _WAIT_LIMIT_NS // 1_000_000)))
            return out
        if not a_local.is_cuda:
            full = torch.empty((self.M, K), dtype=a_local.dtype)
            if self.world > 1:
                dist.all_gather_into_tensor(full, a_local, group=self.group)
            else:
                full.copy_(a_local)
            res = full.float() @ w.float().t()
            if bias is not None:
                res = res + bias.float()
            res = res.to(torch.bfloat16)
            if out is not None:
                out.copy_(res)
                return out
            return res
        if out is None:
            out = torch.empty((self.M, Nl), dtype=torch.bfloat16, device=a_local.device)
        self.epoch += 1
        args = self._hot
        if args is None:
            args = self._hot = N.GemmArgs()
            args.mode = N.GEMM_AG
            args.M, args.K = self.M, K
            args.bias_scale = 1.0
            args.rank, args.world = self.rank, self.world
            if self.heap is not None:
                args.peer_base = self.heap.peer_array()
                args.data_off, args.flag_off, args.counter_off = self.data_off, self.flag_off, self.counter_off
            args.status = self.status.data_ptr()
            args.wait_limit_ns = _WAIT_LIMIT_NS
        args.N = Nl
        args.A, args.B, args.out = a_local.data_ptr(), w.data_ptr(), out.data_ptr()
        args.bias = bias.data_ptr() if bias is not None else None
        args.epoch = self.epoch
        if self.world == 1:
            args.num_ctas = 0
            args.num_ctas = 0 if _tuned_pair(args, a_local.device) else _NO_PAIR_BIT
        _launch(args, a_local.device)
        return out
