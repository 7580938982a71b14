"""Symmetric heap: one equally sized segment per rank, all mapped everywhere.

``SymmHeap`` is the Python face of the C++ layer in ``csrc/symm``.  It replaces
the role NCCL plays as data plane in the reference (``eval.py:176``,
``reference.py:91-119``, ``gemm_rs/reference.py:59``): kernels address "offset
X on rank r" directly.  ``torch.distributed`` is used only as control plane
(session id, IPC handle exchange, one barrier at construction).

Backends: ``vmm`` (cuMem + POSIX fd passing, optional NVLS multicast), ``ipc``
(cudaMalloc + cudaIpc handles), ``host`` (memfd + mmap; CPU-only ranks).
"""
from __future__ import annotations

import ctypes as C
import os
import uuid
from typing import Optional, Sequence

import torch
import torch.distributed as dist

from .. import _native as N

_BACKENDS = {"host": N.BACKEND_HOST, "vmm": N.BACKEND_VMM, "ipc": N.BACKEND_IPC}
_RESERVED = 4096  # heap-level barrier pad and bookkeeping at offset 0


class _CudaView:
    """Minimal ``__cuda_array_interface__`` carrier for a raw device pointer."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {
            "shape": (nbytes,),
            "typestr": "|u1",
            "data": (ptr, False),
            "version": 3,
            "strides": None,
        }
        self._owner = owner


def _dist_info(group) -> tuple[int, int]:
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(group), dist.get_world_size(group)
    return 0, 1


class SymmHeap:
    """A symmetric allocation of ``nbytes`` per rank with a bump allocator.

    Construction is collective over ``group``.  ``peer_ptr(r)`` is the address
    of rank r's segment in this process; ``tensor(off, shape, dtype, peer)``
    views a range of any segment as a torch tensor.
    """

    def __init__(
        self,
        nbytes: int,
        group=None,
        backend: str = "auto",
        device: Optional[torch.device] = None,
        timeout_s: float = 60.0,
        nvls: Optional[bool] = None,
    ):
        self.group = group
        self.rank, self.world = _dist_info(group)
        if self.world > N.KB_MAX_WORLD:
            raise ValueError(f"world size {self.world} exceeds {N.KB_MAX_WORLD}")
        if backend == "auto":
            backend = os.environ.get("KB200_SYMM_BACKEND", "vmm" if torch.cuda.is_available() else "host")
        if backend not in _BACKENDS:
            raise ValueError(f"unknown symmetric-memory backend {backend!r}")
        if backend != "host":
            device = torch.device("cuda") if device is None else torch.device(device)
            if device.index is None:
                device = torch.device("cuda", torch.cuda.current_device())
            torch.cuda.set_device(device)
        self.device = torch.device("cpu") if backend == "host" else torch.device(device)
        self.timeout_ms = int(timeout_s * 1000)
        self._lib = N.lib()
        self._h = C.c_void_p()
        self._bump = _RESERVED
        self._barrier_epoch = 0
        self._views = {}  # host backend: (address, bytes) -> ctypes buffer kept alive for the tensors that alias it
        self.mc_ptr: Optional[int] = None

        session = self._broadcast_session()
        backend = self._create(backend, nbytes + _RESERVED)
        self.backend = backend
        self.nbytes = int(self._lib.kb_symm_segment_bytes(self._h))
        self._map(session)
        if nvls is None:  # KB200_NVLS=0 keeps every kernel on plain peer loads and stores
            nvls = os.environ.get("KB200_NVLS", "1") == "1"
        if nvls and backend == "vmm" and self.world > 1:
            self._setup_multicast(session)
        self._control_barrier()
        self.peer_ptrs = [int(self._lib.kb_symm_peer_ptr(self._h, r) or 0) for r in range(self.world)]
        self.status = torch.zeros(8, dtype=torch.int32, device=self.device)

    # ------------------------------------------------------------- set-up ----
    def _broadcast_session(self) -> str:
        obj = [uuid.uuid4().hex[:16] if self.rank == 0 else None]
        if self.world > 1:
            dist.broadcast_object_list(obj, src=dist.get_global_rank(self.group, 0) if self.group else 0, group=self.group)
        return obj[0]

    def _control_barrier(self) -> None:
        if self.world > 1:
            dist.barrier(group=self.group)

    def _all_agree(self, ok: bool) -> bool:
        if self.world == 1:
            return ok
        flags = [None] * self.world
        dist.all_gather_object(flags, bool(ok), group=self.group)
        return all(flags)

    def _agree_or_raise(self, code: int, what: str) -> None:
        """All ranks learn whether a set-up step worked everywhere: a rank whose
        step failed raises its own error, the others raise instead of waiting for
        it in the next barrier until the collective library's time-out."""
        err = N.last_error() if code != N.KB_OK else ""
        if not self._all_agree(code == N.KB_OK):
            if code != N.KB_OK:
                N.check(code)
            raise N.NativeError(N.KB_ERR_IO, err or f"a peer failed to {what}")

    def _create(self, backend: str, nbytes: int) -> str:
        dev_index = self.device.index if self.device.type == "cuda" else 0
        code = self._lib.kb_symm_create(_BACKENDS[backend], self.rank, self.world, nbytes, dev_index, C.byref(self._h))
        err = N.last_error() if code != N.KB_OK else ""
        if not self._all_agree(code == N.KB_OK):
            if self._h:
                self._lib.kb_symm_destroy(self._h)
                self._h = C.c_void_p()
            if backend == "vmm":
                # cuMem export refused somewhere: every rank falls back together.
                return self._create("ipc", nbytes)
            raise N.NativeError(code, err or "a peer failed to allocate its symmetric segment")
        return backend

    def _map(self, session: str) -> None:
        lib = self._lib
        if self.backend == "ipc":
            mine = C.create_string_buffer(64)
            N.check(lib.kb_symm_ipc_handle(self._h, mine))
            handles = [None] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, mine.raw, group=self.group)
            else:
                handles[0] = mine.raw
            blob = C.create_string_buffer(b"".join(handles), 64 * self.world)
            self._agree_or_raise(lib.kb_symm_map_peers(self._h, None, blob), "map the peers' segments")
            return
        fds = (C.c_int * self.world)()
        N.check(
            lib.kb_fd_allgather(session.encode(), b"seg", self.rank, self.world, lib.kb_symm_local_fd(self._h), fds, self.timeout_ms)
        )
        try:
            code = lib.kb_symm_map_peers(self._h, fds, None)
        finally:
            for fd in fds:
                if fd >= 0:
                    os.close(fd)
        self._agree_or_raise(code, "map the peers' segments")

    def _setup_multicast(self, session: str) -> None:
        lib = self._lib
        dev_index = self.device.index or 0
        ok = bool(lib.kb_symm_mc_supported(dev_index))
        if not self._all_agree(ok):
            return
        fd0 = C.c_int(-1)
        code = lib.kb_symm_mc_create(self._h, C.byref(fd0)) if self.rank == 0 else N.KB_OK
        if not self._all_agree(code == N.KB_OK):
            return
        fds = (C.c_int * self.world)()
        N.check(lib.kb_fd_allgather(session.encode(), b"mc", self.rank, self.world, fd0.value if self.rank == 0 else -1, fds, self.timeout_ms))
        code = lib.kb_symm_mc_join(self._h, fds[0])
        for fd in fds:
            if fd >= 0:
                os.close(fd)
        if fd0.value >= 0:
            os.close(fd0.value)
        if not self._all_agree(code == N.KB_OK):
            return
        self._control_barrier()  # every device added before anyone binds
        code = lib.kb_symm_mc_bind(self._h)
        if self._all_agree(code == N.KB_OK):
            self.mc_ptr = int(lib.kb_symm_mc_ptr(self._h) or 0) or None

    # ---------------------------------------------------------- allocation ----
    def alloc(self, nbytes: int, align: int = 256) -> int:
        """Reserves ``nbytes`` at the same offset on every rank; returns the offset."""
        off = (self._bump + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {off + nbytes} of {self.nbytes} bytes")
        self._bump = off + nbytes
        return off

    def peer_ptr(self, peer: int) -> int:
        return self.peer_ptrs[peer]

    def peer_array(self):
        arr = (C.c_void_p * N.KB_MAX_WORLD)()
        for r in range(self.world):
            arr[r] = self.peer_ptrs[r]
        return arr

    def tensor(self, offset: int, shape: Sequence[int], dtype: torch.dtype, peer: Optional[int] = None) -> torch.Tensor:
        """A tensor aliasing ``[offset, offset + numel*itemsize)`` of a segment."""
        peer = self.rank if peer is None else peer
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if offset < 0 or offset + nbytes > self.nbytes:
            raise ValueError("range outside the symmetric segment")
        ptr = self.peer_ptrs[peer] + offset
        if self.backend == "host":
            buf = self._views.get((ptr, nbytes))
            if buf is None:  # one buffer object per range however often it is viewed
                buf = self._views[(ptr, nbytes)] = (C.c_char * nbytes).from_address(ptr)
            flat = torch.frombuffer(buf, dtype=torch.uint8)
        else:
            flat = torch.as_tensor(_CudaView(ptr, nbytes, self), device=self.device)
        return flat.view(dtype).view(*shape)

    # ------------------------------------------------------------- barrier ----
    def barrier(self, stream: Optional[torch.cuda.Stream] = None, limit_ns: int = 2_000_000_000) -> None:
        """Cross-rank barrier executed on the device (or by CPU atomics)."""
        self._barrier_epoch += 1
        if self.backend == "host":
            N.check(self._lib.kb_symm_host_barrier(self._h, 0, self._barrier_epoch, self.timeout_ms))
            return
        st = stream or torch.cuda.current_stream(self.device)
        N.check(
            self._lib.kb_device_barrier(
                self.peer_array(), 0, self.rank, self.world, self._barrier_epoch, limit_ns, self.status.data_ptr(), st.cuda_stream
            )
        )

    def check_status(self) -> None:
        """Raises if a kernel recorded a failed wait or index check (synchronises)."""
        st = self.status.cpu().tolist()
        if st[0] != 0:
            self.status.zero_()
            msg = f"{N.DEV_CODES.get(st[0], st[0])}: site {st[1]}, waiting on {st[2]}, epoch {st[3]}, block {st[4]}"
            if st[0] in (1, 2):
                raise N.SymmTimeoutError(N.KB_ERR_TIMEOUT, msg)
            raise N.NativeError(N.KB_ERR_ARG, msg)

    def agree_epoch(self, epoch: int) -> int:
        """Collective: the largest ``epoch`` any rank holds.  After a failed call the
        ranks of a context may have counted different numbers of calls; flags only
        grow, so everybody continues from the maximum."""
        if self.world == 1:
            return epoch
        vals = [None] * self.world
        dist.all_gather_object(vals, int(epoch), group=self.group)
        return max(vals)

    def close(self, collective: bool = True) -> None:
        """Unmaps and frees the segments.  Collective by default (a control-plane
        barrier first: nobody unmaps while a peer may still touch the memory);
        ``collective=False`` is for a heap whose process group is gone, when no
        peer can be using it any more."""
        if self._h:
            if self.backend != "host" and torch.cuda.is_available():
                torch.cuda.synchronize(self.device)
            if collective:
                self._control_barrier()
            self._lib.kb_symm_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            if self._h and self.world == 1:
                self._lib.kb_symm_destroy(self._h)
        except Exception:
            pass
