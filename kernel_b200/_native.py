"""ctypes binding of libkb200.so (C ABI in csrc/include/kb200.h).

The library is built in-tree by ``kernel_b200.csrc.build``.  Loading never
falls back silently: on a machine with a GPU a missing library is an error,
because every fused op must run its hand-written kernel there.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

KB_MAX_WORLD = 16

KB_OK, KB_ERR_CUDA, KB_ERR_ARG, KB_ERR_TIMEOUT, KB_ERR_IO, KB_ERR_UNSUPPORTED = range(6)
BACKEND_HOST, BACKEND_VMM, BACKEND_IPC = 0, 1, 2
GEMM_PLAIN, GEMM_RS, GEMM_AG = 0, 1, 2

DEV_CODES = {0: "ok", 1: "pipeline barrier timeout", 2: "peer flag timeout", 3: "index out of bounds"}

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libkb200.so"


class NativeError(RuntimeError):
    """A call into libkb200 returned a non-zero status."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libkb200 status {code}: {message}")
        self.code = code
        self.message = message

    def __reduce__(self):
        # Exceptions cross process boundaries (a pool worker's error travels to the
        # evaluator pickled); the default reduction would call __init__ with the one
        # formatted string and fail on the receiving side.
        return (type(self), (self.code, self.message))


class SymmTimeoutError(NativeError):
    """A rendezvous step or a device-side wait ran out of time."""


class GemmArgs(C.Structure):
    _fields_ = [
        ("mode", C.c_int),
        ("M", C.c_int),
        ("N", C.c_int),
        ("K", C.c_int),
        ("A", C.c_void_p),
        ("B", C.c_void_p),
        ("bias", C.c_void_p),
        ("bias_scale", C.c_float),
        ("out", C.c_void_p),
        ("rank", C.c_int),
        ("world", C.c_int),
        ("epoch", C.c_uint32),
        ("peer_base", C.c_void_p * KB_MAX_WORLD),
        ("data_off", C.c_uint64),
        ("flag_off", C.c_uint64),
        ("counter_off", C.c_uint64),
        ("status", C.c_void_p),
        ("wait_limit_ns", C.c_uint64),
        ("num_ctas", C.c_int),
        ("mc_base", C.c_void_p),
    ]


class A2aArgs(C.Structure):
    _fields_ = [
        ("rank", C.c_int),
        ("world", C.c_int),
        ("num_experts", C.c_int),
        ("topk", C.c_int),
        ("hidden", C.c_int),
        ("max_tokens", C.c_int),
        ("num_tokens", C.c_int),
        ("elem_bytes", C.c_int),
        ("dtype", C.c_int),
        ("x", C.c_void_p),
        ("indices", C.c_void_p),
        ("weights", C.c_void_p),
        ("out", C.c_void_p),
        ("slots", C.c_void_p),
        ("epoch", C.c_uint32),
        ("peer_base", C.c_void_p * KB_MAX_WORLD),
        ("recv_off", C.c_uint64),
        ("y_off", C.c_uint64),
        ("count_off", C.c_uint64),
        ("flag_off", C.c_uint64),
        ("sync_off", C.c_uint64),
        ("scale_mode", C.c_int),
        ("status", C.c_void_p),
        ("wait_limit_ns", C.c_uint64),
        ("num_ctas", C.c_int),
        ("trace", C.c_void_p),
        ("meta_off", C.c_uint64),
        ("rank_slots", C.c_void_p),
        ("ll_off", C.c_uint64),
        ("ll_max_tokens", C.c_int),
    ]


_lib = None


def _declare(lib: C.CDLL) -> None:
    vp, i, u32, u64 = C.c_void_p, C.c_int, C.c_uint32, C.c_uint64
    sig = {
        "kb_last_error": (C.c_char_p, []),
        "kb_fd_allgather": (i, [C.c_char_p, C.c_char_p, i, i, i, C.POINTER(i), i]),
        "kb_symm_create": (i, [i, i, i, u64, i, C.POINTER(vp)]),
        "kb_symm_segment_bytes": (u64, [vp]),
        "kb_symm_local_fd": (i, [vp]),
        "kb_symm_ipc_handle": (i, [vp, vp]),
        "kb_symm_map_peers": (i, [vp, C.POINTER(i), vp]),
        "kb_symm_peer_ptr": (vp, [vp, i]),
        "kb_symm_local_ptr": (vp, [vp]),
        "kb_symm_mc_supported": (i, [i]),
        "kb_symm_mc_create": (i, [vp, C.POINTER(i)]),
        "kb_symm_mc_join": (i, [vp, i]),
        "kb_symm_mc_bind": (i, [vp]),
        "kb_symm_mc_ptr": (vp, [vp]),
        "kb_symm_destroy": (i, [vp]),
        "kb_symm_host_barrier": (i, [vp, u64, u32, i]),
        "kb_multimem_store": (i, [vp, vp, u64, vp]),
        "kb_multimem_reduce_bf16": (i, [vp, vp, u64, vp]),
        "kb_wait_flags": (i, [vp, i, i, u32, u64, vp, vp]),
        "kb_device_barrier": (i, [C.POINTER(vp), u64, i, i, u32, u64, vp, vp]),
        "kb_gemm": (i, [C.POINTER(GemmArgs), vp]),
        "kb_gemm_schedule": (i, [i, i, i, i, i, i, i, C.POINTER(i), C.POINTER(i)]),
        "kb_gemm_rs_data_bytes": (u64, [i, i, i]),
        "kb_gemm_rs_flag_bytes": (u64, [i, i, i]),
        "kb_gemm_ag_data_bytes": (u64, [i, i]),
        "kb_gemm_ag_flag_bytes": (u64, [i, i]),
        "kb_gemm_ag_counter_bytes": (u64, [i, i]),
        "kb_a2a_rows_bytes": (u64, [i, i, i, i, i]),
        "kb_a2a_meta_bytes": (u64, [i, i, i]),
        "kb_a2a_ll_max_tokens": (i, []),
        "kb_a2a_ll_bytes": (u64, [i, i, i, i, i]),
        "kb_a2a_flag_bytes": (u64, []),
        "kb_a2a_sync_bytes": (u64, []),
        "kb_a2a_flag_stride_words": (i, []),
        "kb_a2a_post_ready": (i, [C.POINTER(A2aArgs), vp]),
        "kb_a2a_round_trip_static": (i, [vp, vp, vp, vp, i, i, i, i, i, i, vp]),
        "kb_a2a_static_status": (i, [vp, i, vp]),
        "kb_a2a_dispatch": (i, [C.POINTER(A2aArgs), vp]),
        "kb_a2a_expert_scale": (i, [C.POINTER(A2aArgs), vp]),
        "kb_a2a_combine": (i, [C.POINTER(A2aArgs), vp]),
        "kb_a2a_round_trip": (i, [C.POINTER(A2aArgs), vp]),
        "kb_a2a_round_trip_host": (i, [C.POINTER(A2aArgs), i]),
        "kb_a2a_round_trip_host_ll": (i, [C.POINTER(A2aArgs), i]),
        "kb_a2a_dispatch_host": (i, [C.POINTER(A2aArgs), i]),
        "kb_a2a_combine_host": (i, [C.POINTER(A2aArgs), i]),
        "kb_gemm_host": (i, [C.POINTER(GemmArgs), i]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> C.CDLL:
    """Returns the loaded library, building it first if the file is missing or older
    than its sources (a digest check; a no-op when it is current).  A stale file is
    still used, with a warning, on a machine that cannot rebuild it."""
    global _lib
    if _lib is None:
        from .csrc.build import build

        try:
            build()
        except Exception as e:  # no compiler here
            if not LIB_PATH.exists():
                raise
            import warnings

            warnings.warn(f"libkb200.so could not be checked against its sources ({e}); using the existing file")
        _lib = C.CDLL(str(LIB_PATH))
        _declare(_lib)
    return _lib


def last_error() -> str:
    return (lib().kb_last_error() or b"").decode(errors="replace")


def check(code: int) -> None:
    if code == KB_OK:
        return
    msg = last_error()
    if code == KB_ERR_TIMEOUT:
        raise SymmTimeoutError(code, msg)
    raise NativeError(code, msg)
