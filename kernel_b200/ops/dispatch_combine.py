"""MoE expert-parallel dispatch / combine.

``MoEAllToAll`` owns the symmetric workspace of one configuration and exposes
``dispatch`` -> (expert compute) -> ``combine`` plus the fused
``dispatch_scale_combine`` round trip the all2all task measures.  On CUDA it
launches the hand-written kernels in ``csrc/kernels/a2a.cu`` (no NCCL call, no
host synchronisation, no allocation after construction apart from the output
tensor).  CPU ranks run the kernels' protocol (sender-computed slots, stores into
the owner's segment, epoch flags, pull combine) over a memfd-backed symmetric heap
(``csrc/symm/a2a_host.cpp``), round trip or split; ``KB200_A2A_CPU_PATH=collectives``
selects a vectorised torch implementation over ``torch.distributed`` instead.

Reference counterparts: ``reference.py:54-234`` (``PyTorchAllToAll``) and
``submission.py:5-219`` (``OptimizedAllToAll`` / ``custom_kernel``).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native as N
from ..parallel.symm import SymmHeap, _dist_info

_WAIT_LIMIT_NS = int(float(os.environ.get("KB200_WAIT_LIMIT_MS", "2000")) * 1e6)
_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
SCALE_IDENTITY, SCALE_RANK, SCALE_EXPERT = 0, 1, 2

launch_count = 0  # kernels launched by this module (bench accounting)


def expert_scale_vector(num_experts: int, world: int, mode: int, device=None) -> torch.Tensor:
    """Per-expert multiplier of the simulated expert, as a float32 vector [E]."""
    e = torch.arange(num_experts, device=device)
    if mode == SCALE_IDENTITY:
        return torch.ones(num_experts, device=device)
    if mode == SCALE_RANK:
        return (1 + e // (num_experts // world)).float()
    if mode == SCALE_EXPERT:
        return (e + 1).float() / num_experts
    raise ValueError(f"unknown scale mode {mode}")


class MoEAllToAll:
    def __init__(self, num_experts: int, experts_per_token: int, hidden_dim: int, max_num_tokens: int,
                 dtype: torch.dtype = torch.bfloat16, group=None, device: Optional[torch.device] = None,
                 heap: Optional[SymmHeap] = None):
        self.E, self.k, self.H, self.max_tokens = num_experts, experts_per_token, hidden_dim, max_num_tokens
        self.dtype = dtype
        self.group = group
        self.rank, self.world = _dist_info(group)
        if num_experts % self.world:
            raise ValueError("num_experts must be divisible by the world size")
        self.El = num_experts // self.world
        self.cap = max_num_tokens * experts_per_token
        self.native = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.epoch = 0
        self.low_latency = False
        self.ll_off = 0
        self.heap = None
        self._trace = None
        # CPU ranks: the same protocol over a memfd-backed symmetric heap (bf16, fp16,
        # fp32), or torch.distributed collectives (any dtype; KB200_A2A_CPU_PATH=collectives).
        self.host_heap = (not self.native and dtype in _DTYPES
                          and os.environ.get("KB200_A2A_CPU_PATH", "heap") == "heap")
        if self.native or self.host_heap:
            if dtype not in _DTYPES:
                raise ValueError(f"unsupported dtype {dtype}")
            lib = N.lib()
            eb = torch.empty((), dtype=dtype).element_size()
            rows = int(lib.kb_a2a_rows_bytes(self.world, max_num_tokens, experts_per_token, hidden_dim, eb))
            counts = (self.world * self.El * 4 + 255) // 256 * 256
            flag_bytes, sync_bytes = int(lib.kb_a2a_flag_bytes()), int(lib.kb_a2a_sync_bytes())
            meta_bytes = int(lib.kb_a2a_meta_bytes(self.world, max_num_tokens, experts_per_token))
            # small contexts get the landing areas of the low-latency round trip (flags inside the data)
            ll_bytes = 0
            if os.environ.get("KB200_A2A_LL", "1") == "1":  # CPU ranks run the same protocol (a2a_ll_host.cpp)
                ll_bytes = int(lib.kb_a2a_ll_bytes(self.world, max_num_tokens, experts_per_token, hidden_dim, eb))
            need = 2 * rows + counts + flag_bytes + sync_bytes + meta_bytes + ll_bytes + 8192
            # no multicast mapping here: these kernels use peer loads and stores only
            self.heap = heap or (SymmHeap(need, group=group, device=device, nvls=False) if self.native
                                 else SymmHeap(need, group=group, backend="host", timeout_s=_WAIT_LIMIT_NS / 1e9 + 5))
            self.recv_off = self.heap.alloc(rows)
            self.y_off = self.heap.alloc(rows)
            self.count_off = self.heap.alloc(counts)
            self.flag_off = self.heap.alloc(flag_bytes)
            self.sync_off = self.heap.alloc(sync_bytes)
            self.meta_off = self.heap.alloc(meta_bytes)  # expert lists and weights of the one-launch round trip's rows
            self.ll_off = self.heap.alloc(ll_bytes) if ll_bytes else 0
            self.low_latency = bool(self.ll_off)  # round trips of this context poll the data, not flags
            self._flag_stride = int(lib.kb_a2a_flag_stride_words())
            self.rank_slots = torch.empty(max_num_tokens * self.world, dtype=torch.int32, device=self.heap.device)
            self.slots = torch.empty(self.cap, dtype=torch.int32, device=self.heap.device)
            self.status = self.heap.status
            self._eb = eb
            self._fused = os.environ.get("KB200_A2A_FUSED", "1") == "1"
            self._trace = None
            self._hot_args = None
            self._lib = lib
            if os.environ.get("KB200_TRACE", "0") == "1":
                self.enable_trace()

    # ------------------------------------------------------------- native ----
    def _args(self, x, indices, weights, out, scale_mode) -> N.A2aArgs:
        a = N.A2aArgs()
        a.rank, a.world = self.rank, self.world
        a.num_experts, a.topk, a.hidden, a.max_tokens = self.E, self.k, self.H, self.max_tokens
        a.num_tokens = x.shape[0]
        a.elem_bytes, a.dtype = self._eb, _DTYPES[self.dtype]
        a.x, a.indices = x.data_ptr(), indices.data_ptr()
        a.weights = weights.data_ptr() if weights is not None else None
        a.out = out.data_ptr() if out is not None else None
        a.slots = self.slots.data_ptr()
        a.epoch = self.epoch
        a.peer_base = self.heap.peer_array()
        a.recv_off, a.y_off, a.count_off = self.recv_off, self.y_off, self.count_off
        a.flag_off, a.sync_off = self.flag_off, self.sync_off
        a.scale_mode = scale_mode
        a.status = self.status.data_ptr()
        a.wait_limit_ns = _WAIT_LIMIT_NS
        a.trace = self._trace.data_ptr() if self._trace is not None else None
        a.meta_off = self.meta_off
        a.rank_slots = self.rank_slots.data_ptr()
        a.ll_off, a.ll_max_tokens = self.ll_off, (self.max_tokens if self.ll_off else 0)
        return a

    # -------------------------------------------------------------- tracing ----
    TRACE_PHASES = ("slots", "push", "dispatch_flag", "wait_first_source", "expert_pass", "expert_flag",
                    "wait_expert", "combine")

    def enable_trace(self, on: bool = True) -> None:
        """Phase stamps: CTA 0 records the global timer at every phase boundary of
        the next calls (the role of the reference's per-phase ``TimingContext``,
        ``all2all/submission_timed.py:9-33``, without host synchronisation)."""
        self._trace = torch.zeros(16, dtype=torch.int64, device=self.heap.device) if on else None

    def read_trace(self) -> dict:
        """Durations in microseconds between consecutive stamps of the last call
        (synchronises).  ``expert_pass`` runs source by source and contains the waits
        for the later sources; ``waited_in_expert_pass`` is their sum,
        ``waited_for_combine`` the wait for every rank's expert outputs.  ``total`` is
        entry to end as seen by CTA 0."""
        t = self._trace.cpu().tolist()
        out = {name: (t[i + 1] - t[i]) / 1e3 for i, name in enumerate(self.TRACE_PHASES)}
        out["waited_in_expert_pass"] = t[10] / 1e3
        out["waited_for_combine"] = t[11] / 1e3
        # the CTA that finishes a phase last: when it arrived and when its flags were out, after the kernel's entry
        for name, i in (("dispatch_last_cta", 12), ("dispatch_flags_out", 13), ("expert_last_cta", 14), ("expert_flags_out", 15)):
            out[name] = (t[i] - t[0]) / 1e3
        out["total"] = (t[8] - t[0]) / 1e3
        return out

    def _validate(self, x, indices, weights) -> None:
        T = x.shape[0]
        if x.dtype != self.dtype or x.shape[1] != self.H or not x.is_contiguous():
            raise ValueError("x must be contiguous [T, hidden] in the context dtype")
        if indices.dtype != torch.int32 or tuple(indices.shape) != (T, self.k) or not indices.is_contiguous():
            raise ValueError("indices must be contiguous int32 [T, k]")
        if weights is not None and (weights.dtype != torch.float32 or tuple(weights.shape) != (T, self.k) or not weights.is_contiguous()):
            raise ValueError("weights must be contiguous float32 [T, k]")
        if T > self.max_tokens:
            raise ValueError("more tokens than max_num_tokens")

    def dispatch_scale_combine(self, x: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor,
                               scale_mode: int = SCALE_IDENTITY) -> torch.Tensor:
        """Full round trip with the simulated expert ``y = scale(expert) * x``."""
        self._validate(x, indices, weights)
        if not x.is_cuda:
            if self.host_heap:
                out = torch.empty_like(x)
                self.epoch += 1
                a = self._args(x, indices, weights, out, scale_mode)
                fn = self._lib.kb_a2a_round_trip_host_ll if self.ll_off else self._lib.kb_a2a_round_trip_host
                N.check(fn(C.byref(a), max(1, _WAIT_LIMIT_NS // 1_000_000)))
                return out
            return self._cpu_round_trip(x, indices, weights, scale_mode)
        global launch_count
        out = torch.empty_like(x)
        self.epoch += 1
        # The argument block is built once; a call only refreshes what changes.
        # Host time matters here: a rank whose launch is late keeps all its peers
        # waiting inside their kernels.
        a = self._hot_args
        if a is None:
            a = self._hot_args = self._args(x, indices, weights, out, scale_mode)
            self._hot_ref = C.byref(a)
            self._dev_index = x.device.index if x.device.index is not None else torch.cuda.current_device()
        else:
            a.num_tokens = x.shape[0]
            a.x, a.indices, a.weights, a.out = x.data_ptr(), indices.data_ptr(), weights.data_ptr(), out.data_ptr()
            a.epoch, a.scale_mode = self.epoch, scale_mode
            a.trace = self._trace.data_ptr() if self._trace is not None else None
        st = torch._C._cuda_getCurrentRawStream(self._dev_index)  # the raw handle, without building a Stream object
        lib = self._lib
        if self._fused:
            code = lib.kb_a2a_round_trip(self._hot_ref, st)
            if code == N.KB_OK:
                launch_count += 1
                return out
            if code != N.KB_ERR_UNSUPPORTED:
                N.check(code)
            self._fused = False  # too many CTAs for one cooperative launch: three launches
        N.check(lib.kb_a2a_dispatch(self._hot_ref, st))
        N.check(lib.kb_a2a_expert_scale(self._hot_ref, st))
        N.check(lib.kb_a2a_combine(self._hot_ref, st))
        launch_count += 3
        return out

    def dispatch(self, x: torch.Tensor, indices: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Pushes token rows to their experts' ranks.

        Returns ``(counts, recv)``: ``counts[src, local_expert]`` (int32) and the
        receive region ``recv[src, row, H]`` of this rank; the rows of one
        source are grouped by local expert in expert order.  Both alias the
        symmetric workspace and are valid once the stream has passed the wait
        that ``expert_rows`` / ``combine`` enqueue.
        """
        self._validate(x, indices, None)
        if not x.is_cuda:
            if not self.host_heap:
                raise RuntimeError("split dispatch/combine on CPU needs the host-heap path (KB200_A2A_CPU_PATH=heap)")
            self.epoch += 1
            a = self._args(x, indices, None, None, SCALE_IDENTITY)
            N.check(self._lib.kb_a2a_dispatch_host(C.byref(a), max(1, _WAIT_LIMIT_NS // 1_000_000)))
            counts = self.heap.tensor(self.count_off, (self.world, self.El), torch.int32)
            recv = self.heap.tensor(self.recv_off, (self.world, self.cap, self.H), self.dtype)
            return counts, recv
        global launch_count
        self.epoch += 1
        a = self._args(x, indices, None, None, SCALE_IDENTITY)
        lib = N.lib()
        st = torch.cuda.current_stream(x.device).cuda_stream
        N.check(lib.kb_a2a_dispatch(C.byref(a), st))
        flags = self.heap.peer_ptr(self.rank) + self.flag_off
        N.check(lib.kb_wait_flags(flags, self.world, self._flag_stride, self.epoch, _WAIT_LIMIT_NS,
                                  self.status.data_ptr(), st))
        launch_count += 2
        counts = self.heap.tensor(self.count_off, (self.world, self.El), torch.int32)
        recv = self.heap.tensor(self.recv_off, (self.world, self.cap, self.H), self.dtype)
        return counts, recv

    def expert_output_buffer(self) -> torch.Tensor:
        """``y[src, row, H]``: where expert outputs must be written, row for row."""
        return self.heap.tensor(self.y_off, (self.world, self.cap, self.H), self.dtype)

    def combine(self, x_like: torch.Tensor, indices: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
        """Publishes this rank's expert outputs and gathers the weighted sum
        ``out[t] = sum_k w[t,k] * y(t,k)`` for the local tokens."""
        self._validate(x_like, indices, weights)
        global launch_count
        out = torch.empty_like(x_like)
        a = self._args(x_like, indices, weights, out, SCALE_IDENTITY)
        if not x_like.is_cuda:
            if not self.host_heap:
                raise RuntimeError("split dispatch/combine on CPU needs the host-heap path (KB200_A2A_CPU_PATH=heap)")
            N.check(self._lib.kb_a2a_combine_host(C.byref(a), max(1, _WAIT_LIMIT_NS // 1_000_000)))
            return out
        lib = N.lib()
        st = torch.cuda.current_stream(x_like.device).cuda_stream
        # y-ready flags of this epoch go out first; the combine kernel waits for every rank's.
        N.check(lib.kb_a2a_post_ready(C.byref(a), st))
        N.check(lib.kb_a2a_combine(C.byref(a), st))
        launch_count += 2
        return out

    def recover(self) -> None:
        """Collective.  Brings the context back into a usable state after
        ``heap.check_status()`` reported a failed wait (a peer that was late or
        absent): waits for this rank's kernels, clears the status words, zeroes the
        block counters and arrival words, and moves every rank to the same call
        number, past every flag value already written."""
        if self.heap is None:
            return
        if self.native:
            torch.cuda.synchronize(self.heap.device)
        self.heap.status.zero_()
        words = int(self._lib.kb_a2a_sync_bytes()) // 4
        self.heap.tensor(self.sync_off, (words,), torch.int32).zero_()
        self.epoch = self.heap.agree_epoch(self.epoch) + 1
        if self.native:
            torch.cuda.synchronize(self.heap.device)
        self.heap._control_barrier()

    # ------------------------------------------------------- debug checks ----
    _POISON = 0x7FC1  # a bf16/fp16 NaN bit pattern that no kernel produces

    def poison_workspace(self) -> None:
        """Fills both row regions of this rank with a sentinel.  Together with
        ``verify_workspace`` this is the stand-in for a memory checker: after a
        call no sentinel may survive inside the rows the counts declare valid,
        and nothing may have been written outside them."""
        nbytes = self.world * self.cap * self.H * self._eb
        for off in (self.recv_off, self.y_off):
            self.heap.tensor(off, (nbytes // 2,), torch.int16).fill_(self._POISON)

    def verify_workspace(self) -> Tuple[int, int]:
        """Returns ``(sentinel words inside valid rows, written words outside valid
        rows)`` for this rank's receive region; both must be zero.  Synchronises."""
        counts = self.heap.tensor(self.count_off, (self.world, self.El), torch.int32).clone()
        words_per_row = self.H * self._eb // 2
        recv = self.heap.tensor(self.recv_off, (self.world, self.cap, words_per_row), torch.int16)
        is_poison = recv == (self._POISON)
        totals = counts.sum(1)
        valid = torch.arange(self.cap, device=recv.device).unsqueeze(0) < totals.unsqueeze(1)  # [world, cap]
        inside = int((is_poison & valid.unsqueeze(-1)).sum())
        outside = int((~is_poison & ~valid.unsqueeze(-1)).sum())
        return inside, outside

    def expert_view(self, counts: torch.Tensor, recv: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Expert-major padded view ``(expert_num_tokens [El], expert_x [El, max_recv, H])``
        like ``PyTorchAllToAll.dispatch`` returns (reference.py:123-148).  Copies."""
        counts_h = counts.cpu()
        max_recv = self.max_tokens * self.world
        ex = torch.zeros((self.El, max_recv, self.H), dtype=self.dtype, device=recv.device)
        num = counts_h.sum(0).to(torch.int32)
        fill = [0] * self.El
        for s in range(self.world):
            off = 0
            for le in range(self.El):
                c = int(counts_h[s, le])
                if c:
                    ex[le, fill[le]:fill[le] + c] = recv[s, off:off + c]
                    fill[le] += c
                off += c
        return num.to(recv.device), ex

    # ---------------------------------------------------------------- CPU ----
    def _cpu_round_trip(self, x, indices, weights, scale_mode) -> torch.Tensor:
        T = x.shape[0]
        flat_e = indices.reshape(-1).long()
        dst = flat_e // self.El
        order = torch.argsort(dst, stable=True)
        send_counts = torch.bincount(dst, minlength=self.world)
        tok = torch.arange(T).repeat_interleave(self.k)
        send_x = x[tok][order]
        send_e = flat_e[order]
        if self.world > 1:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts, group=self.group)
            rc, sc = recv_counts.tolist(), send_counts.tolist()
            recv_x = torch.empty((sum(rc), self.H), dtype=x.dtype)
            recv_e = torch.empty(sum(rc), dtype=torch.long)
            dist.all_to_all_single(recv_x, send_x, rc, sc, group=self.group)
            dist.all_to_all_single(recv_e, send_e, rc, sc, group=self.group)
        else:
            rc = sc = send_counts.tolist()
            recv_x, recv_e = send_x, send_e
        scale = expert_scale_vector(self.E, self.world, scale_mode)[recv_e].unsqueeze(1)
        y = (recv_x.float() * scale).to(x.dtype)
        if self.world > 1:
            back = torch.empty_like(send_x)
            dist.all_to_all_single(back, y, sc, rc, group=self.group)
        else:
            back = y
        contrib = torch.empty_like(back)
        contrib[order] = back
        w = weights.reshape(-1, 1)
        out = (contrib.float() * w).view(T, self.k, self.H).sum(1)
        return out.to(x.dtype)
