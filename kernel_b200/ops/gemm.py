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
        return SymmHeap(nbytes, group=group, device=device)  # with an NVLS multicast mapping when KB200_NVLS=1
    return SymmHeap(nbytes, group=group, backend="host", timeout_s=_WAIT_LIMIT_NS / 1e9 + 5)


def _mc_base(heap: Optional[SymmHeap]):
    """Multicast mapping of the heap for the kernels, or None (peer loads and stores)."""
    return heap.mc_ptr if heap is not None and getattr(heap, "mc_ptr", None) else None


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


class _HostPipeline:
    """Streams, events and device buffers of a ``run_from_host`` call: chunk i+1 is
    copied in on one stream while chunk i runs on the caller's stream and chunk
    i-1's result is copied out on a third.  Two input and two output buffers.  For
    CPU ranks the three steps simply run one after the other."""

    def __init__(self, device: torch.device, in_shape, out_shape):
        self.cuda = device.type == "cuda"
        self.device = device
        if self.cuda:
            self.h2d, self.d2h = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.inp = [torch.empty(in_shape, dtype=torch.bfloat16, device=device) for _ in range(2)]
        self.out = [torch.empty(out_shape, dtype=torch.bfloat16, device=device) for _ in range(2)]

    def begin(self, chunks: int) -> None:
        if self.cuda:
            self.cur = torch.cuda.current_stream(self.device)
            self.in_ready, self.computed, self.out_done = ([torch.cuda.Event() for _ in range(chunks)] for _ in range(3))
            self.h2d.wait_stream(self.cur)

    def copy_in(self, i: int, fn) -> None:
        if not self.cuda:
            return fn()
        with torch.cuda.stream(self.h2d):
            if i >= 2:
                self.h2d.wait_event(self.computed[i - 2])  # the kernel that read this buffer has finished
            fn()
            self.in_ready[i].record(self.h2d)

    def compute(self, i: int, fn) -> None:
        if not self.cuda:
            return fn()
        self.cur.wait_event(self.in_ready[i])
        if i >= 2:
            self.cur.wait_event(self.out_done[i - 2])  # its previous result has left the output buffer
        fn()
        self.computed[i].record(self.cur)

    def copy_out(self, i: int, fn) -> None:
        if not self.cuda:
            return fn()
        with torch.cuda.stream(self.d2h):
            self.d2h.wait_event(self.computed[i])
            fn()
            self.out_done[i].record(self.d2h)

    def end(self) -> None:
        if self.cuda:
            self.cur.wait_stream(self.d2h)


def _host_buffer(shape) -> torch.Tensor:
    t = torch.empty(shape, dtype=torch.bfloat16)
    return t.pin_memory() if torch.cuda.is_available() else t


def _check_pinned(t: torch.Tensor, name: str, shape) -> None:
    if t.is_cuda or t.dtype != torch.bfloat16 or tuple(t.shape) != tuple(shape) or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous bf16 host tensor of shape {tuple(shape)}")
    if torch.cuda.is_available() and not t.is_pinned() and not os.environ.get("KB200_ALLOW_PAGEABLE"):
        raise ValueError(f"{name} must be in pinned host memory (tensor.pin_memory()), or the copies cannot overlap the kernel")


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
                args.mc_base = _mc_base(self.heap)
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

    def recover(self) -> None:
        """Collective.  After ``heap.check_status()`` reported a failed wait: waits
        for this rank's kernels, clears the status words and moves every rank to the
        same call number, past every flag value already written."""
        if self.heap is None:
            return
        if self.native:
            torch.cuda.synchronize(self.heap.device)
        self.heap.status.zero_()
        self.epoch = self.heap.agree_epoch(self.epoch) + 1
        self.heap._control_barrier()

    def run_from_host(self, a_host: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                      bias_scale: float = 1.0, out_host: Optional[torch.Tensor] = None, chunks: int = 4) -> torch.Tensor:
        """The op with its activations in pinned host memory and its result wanted
        there: ``a_host [M, K_local]`` -> ``out_host [M/world, N]`` (``w``, ``bias`` on
        the device).  The rows every rank owns are cut into ``chunks`` pieces; piece i
        of all owners forms a problem of ``M/chunks`` rows that runs through the
        same fused kernel, while piece i+1 is on its way in and the result of
        piece i-1 on its way out (one ``cudaMemcpyAsync`` per contiguous block), so
        the PCIe transfers overlap the kernel instead of bracketing it.  Returns
        ``out_host``; the caller's stream is done when everything has arrived.
        Collective like ``__call__``.  The reference has no counterpart (its
        evaluator clones the inputs on the device inside its timed region,
        ``eval.py:358``)."""
        world, M, Nn = self.world, self.M, self.N
        rows_rank = M // world
        while chunks > 1 and (rows_rank % chunks or _rows_bad(rows_rank // chunks)):
            chunks -= 1
        rows = rows_rank // chunks
        K = a_host.shape[1]
        _check_pinned(a_host, "a_host", (M, K))
        if out_host is None:
            out_host = _host_buffer((rows_rank, Nn))
        _check_pinned(out_host, "out_host", (rows_rank, Nn))
        dev = w.device
        key = (chunks, K)
        st = self._stream_state.get(key) if hasattr(self, "_stream_state") else None
        if st is None:
            if not hasattr(self, "_stream_state"):
                self._stream_state = {}
            sub = self if chunks == 1 else GemmRS(M // chunks, Nn, group=self.group, device=dev)
            st = self._stream_state[key] = (sub, _HostPipeline(dev, (world, rows, K), (rows, Nn)))
        sub, pipe = st
        src = a_host.view(world, chunks, rows, K)
        dst = out_host.view(chunks, rows, Nn)
        pipe.begin(chunks)
        for i in range(chunks):
            buf, res = pipe.inp[i % 2], pipe.out[i % 2]

            def copy_in():
                for r in range(world):
                    buf[r].copy_(src[r, i], non_blocking=True)

            pipe.copy_in(i, copy_in)
            pipe.compute(i, lambda: sub(buf.view(world * rows, K), w, bias, bias_scale=bias_scale, out=res))
            pipe.copy_out(i, lambda: dst[i].copy_(res, non_blocking=True))
        pipe.end()
        return out_host

    def close(self) -> None:
        """Frees this context's workspaces (collective)."""
        for sub, _ in getattr(self, "_stream_state", {}).values():
            if sub is not self and sub.heap is not None:
                sub.heap.close()
        self._stream_state = {}
        if self.heap is not None:
            self.heap.close()


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
                args.mc_base = _mc_base(self.heap)
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

    def recover(self) -> None:
        """Collective.  After ``heap.check_status()`` reported a failed wait: waits
        for this rank's kernels, clears the status words, zeroes the push counters
        and moves every rank to the same call number, past every flag value already
        written."""
        if self.heap is None:
            return
        if self.native:
            torch.cuda.synchronize(self.heap.device)
        self.heap.status.zero_()
        self.heap.tensor(self.counter_off, (256,), torch.int32).zero_()
        self.epoch = self.heap.agree_epoch(self.epoch) + 1
        if self.native:
            torch.cuda.synchronize(self.heap.device)
        self.heap._control_barrier()

    def run_from_host(self, a_host: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
                      out_host: Optional[torch.Tensor] = None, chunks: int = 4) -> torch.Tensor:
        """The op with its activations in pinned host memory and its result wanted
        there: ``a_host [M/world, K]`` -> ``out_host [M, N_local]``.  This rank's rows
        are cut into ``chunks`` pieces; piece i of every rank forms a gathered problem
        of ``M/chunks`` rows for the same fused kernel, overlapped with the copy of
        piece i+1 coming in and of piece i-1's result going out (see
        ``GemmRS.run_from_host``).  Collective like ``__call__``."""
        world, M, K = self.world, self.M, self.K
        rows_rank = M // world
        while chunks > 1 and (rows_rank % chunks or _rows_bad(rows_rank // chunks)):
            chunks -= 1
        rows = rows_rank // chunks
        Nl = w.shape[0]
        _check_pinned(a_host, "a_host", (rows_rank, K))
        if out_host is None:
            out_host = _host_buffer((M, Nl))
        _check_pinned(out_host, "out_host", (M, Nl))
        dev = w.device
        key = (chunks, Nl)
        st = self._stream_state.get(key) if hasattr(self, "_stream_state") else None
        if st is None:
            if not hasattr(self, "_stream_state"):
                self._stream_state = {}
            sub = self if chunks == 1 else AGGemm(M // chunks, K, group=self.group, device=dev)
            st = self._stream_state[key] = (sub, _HostPipeline(dev, (rows, K), (world, rows, Nl)))
        sub, pipe = st
        src = a_host.view(chunks, rows, K)
        dst = out_host.view(world, chunks, rows, Nl)
        pipe.begin(chunks)
        for i in range(chunks):
            buf, res = pipe.inp[i % 2], pipe.out[i % 2]

            def copy_out():
                for r in range(world):
                    dst[r, i].copy_(res[r], non_blocking=True)

            pipe.copy_in(i, lambda: buf.copy_(src[i], non_blocking=True))
            pipe.compute(i, lambda: sub(buf, w, bias, out=res.view(world * rows, Nl)))
            pipe.copy_out(i, copy_out)
        pipe.end()
        return out_host

    def close(self) -> None:
        """Frees this context's workspaces (collective)."""
        for sub, _ in getattr(self, "_stream_state", {}).values():
            if sub is not self and sub.heap is not None:
                sub.heap.close()
        self._stream_state = {}
        if self.heap is not None:
            self.heap.close()
