"""Build libkb200.so in-tree with nvcc for sm_100a.

The library has a plain C ABI (see include/kb200.h) and depends on nothing but
the statically linked CUDA runtime, so it builds on a machine without a GPU and
loads on a machine without a driver.

    python -m kernel_b200.csrc.build [--force] [--verbose]
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_DIR = CSRC.parent / "lib"
LIB_PATH = LIB_DIR / "libkb200.so"
OBJ_DIR = CSRC / "build"

SOURCES = [
    "common/host_util.cpp",
    "symm/fd_exchange.cpp",
    "symm/symm_heap.cpp",
    "symm/a2a_host.cpp",
    "symm/a2a_ll_host.cpp",
    "symm/gemm_host.cpp",
    "kernels/a2a.cu",
    "kernels/gemm_sm100.cu",
    "kernels/nvls_util.cu",
]

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall", "-x", "cu"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def _sources() -> list[str]:
    srcs = list(SOURCES)
    for extra in sorted((CSRC / "kernels").glob("*.cu")):
        rel = str(extra.relative_to(CSRC))
        if rel not in srcs:
            srcs.append(rel)
    return srcs


def _digest() -> str:
    h = hashlib.sha256()
    files = sorted(p for p in CSRC.rglob("*") if p.suffix in {".cu", ".cuh", ".cpp", ".h", ".py"} and "build/" not in str(p))
    for p in files:
        h.update(str(p.relative_to(CSRC)).encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every source for sm_100a and link libkb200.so; returns its path."""
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    stamp = OBJ_DIR / "digest.txt"
    digest = _digest()

    def current() -> bool:
        return LIB_PATH.exists() and stamp.exists() and stamp.read_text() == digest

    if not force and current():
        return LIB_PATH
    # One builder at a time: the ranks of a job may all find the library stale at once.
    with open(OBJ_DIR / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and current():  # another process built it while this one waited
            return LIB_PATH
        return _build_locked(digest, stamp, verbose)


def _build_locked(digest: str, stamp: Path, verbose: bool) -> Path:
    nvcc = _nvcc()

    def compile_one(rel: str) -> Path:
        src = CSRC / rel
        obj = OBJ_DIR / (rel.replace("/", "_") + ".o")
        cmd = [nvcc, *ARCH_FLAGS, *COMMON, "-I", str(CSRC / "include"), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(f"$ {' '.join(cmd)}\n{res.stdout}{res.stderr}\n")
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {rel}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, _sources()))
    tmp = LIB_PATH.with_suffix(f".so.tmp{os.getpid()}")
    link = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs), "-cudart", "static", "-lpthread", "-ldl", "-lrt"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        sys.stderr.write(f"$ {' '.join(link)}\n{res.stdout}{res.stderr}\n")
        raise RuntimeError("link failed")
    os.replace(tmp, LIB_PATH)  # a process that has the old file mapped keeps it; nobody sees a half-written one
    stamp.write_text(digest)
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
