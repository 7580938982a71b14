"""Multi-process evaluator: correctness first, then device-timed benchmarks.

Command line and protocol follow the reference's ``eval.py`` (``main``
``:527-574``): ``POPCORN_FD=<fd> [POPCORN_SEED=<n>] [POPCORN_GPUS=<n>] python -m
kernel_b200.harness.eval <mode> <tests-file>`` with modes ``test``,
``benchmark``, ``leaderboard`` and ``profile``; ``key: value`` lines go to the
inherited descriptor (``PopcornOutput`` ``:25-40``); exit codes 0 / 2 / 111 /
112 / 113 keep their meaning.

What differs from the reference, on purpose:

* times are device times: a CUDA event pair around ``custom_kernel`` alone on
  every rank, MAX over ranks (the reference times rank 0's wall clock around the
  input clone too, ``eval.py:354-367``); on GPUs a one-element all-reduce queued
  right before the start event lets the devices begin together, so the hosts'
  skew after the barrier is not timed as waiting inside the early ranks' kernels;
* rank r of every case runs in worker process r (one process per GPU for the
  whole run; the reference hands ranks to whichever pool workers are free,
  ``eval.py:201``), a worker's error comes back as text, a failed rank shortens
  the wait for its peers, and workers that are replaced or stopped free their
  workspaces locally before they exit (``_worker_stop``);
* the any-rank-failed flag is an all-reduce, so no rank is left behind in a
  broadcast when another rank fails (``eval.py:376-400``);
* the rendezvous port is a free port unless ``MASTER_PORT`` is set, the
  world size is validated against the pool size up front, ``leaderboard`` and
  ``profile`` return a proper exit status, and ``profile`` works for
  distributed tasks (per-rank table, rank 0 reported);
* the task is a package (``--task all2all|gemm_rs|ag_gemm``; guessed from the
  case keys otherwise), the implementation is selectable (``--impl
  fused|baseline`` or ``--submission some.module | path/to/file.py``) and the backend/device are parameters (``--backend
  nccl|gloo``), so the same flow runs on CPU ranks;
* a tests file may be replaced by ``--yaml <task.yml> --section tests|benchmarks``;
* benchmark modes log, besides the reference's six keys, ``max_rank_us``,
  ``roofline_us`` / ``roofline_frac`` and with ``--with-baseline`` also
  ``baseline_us`` / ``speedup``; ``--json FILE`` dumps the rows.
"""
from __future__ import annotations

import argparse
import base64
import dataclasses
import importlib
import importlib.util
import json
import math
import multiprocessing
import functools
import os
import signal
import socket
import sys
import time
from pathlib import Path
from typing import Any, List, Optional, Tuple

import torch

from ..utils.common import clear_l2_cache, set_seed
from .stats import Stats, calculate_stats, should_stop
from .testcases import SpecError, TestCase, cases_from_yaml, parse_tests

EXIT_OK, EXIT_USAGE, EXIT_NO_FD, EXIT_FAIL, EXIT_BAD_TESTS = 0, 2, 111, 112, 113
TEST_TIMEOUT_S = float(os.environ.get("KB200_EVAL_TEST_TIMEOUT_S", "120"))
BENCH_TIMEOUT_S = float(os.environ.get("KB200_EVAL_BENCH_TIMEOUT_S", "240"))


class PopcornOutput:
    """``key: value`` line writer on an inherited file descriptor."""

    def __init__(self, fd: int):
        self.file = os.fdopen(fd, "w")
        os.set_inheritable(fd, False)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.file.close()

    def print(self, *args, **kwargs):
        print(*args, **kwargs, file=self.file, flush=True)

    def log(self, key: str, value: Any) -> None:
        self.print(f"{key}: {value}")


@dataclasses.dataclass
class RunConfig:
    task: str
    impl: str
    backend: str
    port: int

    def modules(self):
        ref = importlib.import_module(f"kernel_b200.tasks.{self.task}.reference")
        if self.impl == "fused":
            sub = importlib.import_module(f"kernel_b200.tasks.{self.task}.submission")
        elif self.impl == "baseline":
            sub = importlib.import_module(f"kernel_b200.baseline.{self.task}")
        else:
            # any importable module, or a .py file, with a custom_kernel(data): the role of
            # the @SUBMISSION@ placeholder in the reference's task.yml (task.yml:2)
            sub = load_submission(self.impl)
            if not hasattr(sub, "custom_kernel"):
                raise ValueError(f"module {self.impl!r} has no custom_kernel")
        return ref, sub


def load_submission(spec: str):
    """``pkg.module`` is imported; ``path/to/file.py`` is loaded from the file (the
    reference's evaluator imports a ``submission.py`` that sits next to it, eval.py:18)."""
    if spec.endswith(".py") or os.sep in spec:
        path = Path(spec).resolve()
        if not path.is_file():
            raise ValueError(f"submission file {spec!r} not found")
        name = f"kb200_submission_{abs(hash(str(path))) & 0xFFFFFF:x}"
        mod_spec = importlib.util.spec_from_file_location(name, path)
        module = importlib.util.module_from_spec(mod_spec)
        sys.modules[name] = module
        mod_spec.loader.exec_module(module)
        return module
    return importlib.import_module(spec)


def guess_task(args: dict) -> str:
    if "num_experts" in args:
        return "all2all"
    if args.get("op") == "ag_gemm":
        return "ag_gemm"
    return "gemm_rs"


def free_port() -> int:
    env = os.environ.get("MASTER_PORT")
    if env:
        return int(env)
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _device_for(rank: int, backend: str) -> torch.device:
    if backend == "nccl":
        return torch.device("cuda", rank)
    return torch.device("cpu")


def clone_data(data, device: torch.device):
    """Deep copy of every tensor reachable through tuples, lists, dicts and plain
    objects' attributes, placed on ``device`` (the reference's ``_clone_data``
    stops at objects, ``eval.py:127-141``, and hands the originals to the kernel)."""
    if isinstance(data, torch.Tensor):
        return data.detach().clone().to(device)
    if isinstance(data, tuple):
        items = tuple(clone_data(x, device) for x in data)
        if type(data) is tuple:
            return items
        if hasattr(data, "rebuilt"):  # a task's tuple type that carries case attributes
            return data.rebuilt(items)
        if hasattr(data, "_fields"):  # namedtuple
            return type(data)(*items)
        return items
    if isinstance(data, list):
        return [clone_data(x, device) for x in data]
    if isinstance(data, dict):
        return {k: clone_data(v, device) for k, v in data.items()}
    if dataclasses.is_dataclass(data) and not isinstance(data, type):
        return data
    if hasattr(data, "__dict__") and any(isinstance(v, torch.Tensor) for v in vars(data).values()):
        twin = object.__new__(type(data))
        for k, v in vars(data).items():
            setattr(twin, k, clone_data(v, device))
        return twin
    return data


def wrap_check(ref_mod, data, output) -> Tuple[bool, str]:
    res = ref_mod.check_implementation(data, output)
    if isinstance(res, tuple):
        return bool(res[0]), str(res[1])
    return (not bool(res)), str(res)


def _case_args(test: TestCase, rank: Optional[int], device: torch.device) -> dict:
    args = {k: v for k, v in test.args.items() if k != "op"}
    if rank is not None:
        args["rank"] = rank
    args["device"] = device
    return args


def _sync(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)


FAIL_GRACE_S = float(os.environ.get("KB200_EVAL_FAIL_GRACE_S", "10"))


class WorkerFailure(str):
    """What a worker returns instead of raising: the error as text.  An exception
    object may not survive the trip back to the evaluator (one whose constructor
    takes other arguments than ``args`` breaks the pool's result thread, and the
    evaluator then waits for a result that never comes)."""


def _reports_errors(fn):
    @functools.wraps(fn)
    def guarded(*args, **kwargs):
        try:
            return fn(*args, **kwargs)
        except (SystemExit, KeyboardInterrupt):
            raise  # the worker has been told to stop
        except BaseException as e:  # noqa: BLE001 - the text goes back to the evaluator
            return WorkerFailure(f"{type(e).__name__}: {e}")

    return guarded


KILL_GRACE_S = float(os.environ.get("KB200_EVAL_KILL_GRACE_S", "20"))
_SUBMISSION_MODULES = ("all2all", "gemm_rs", "ag_gemm")


def _release_workspaces_locally(settle_s: float) -> int:
    """Frees every cached workspace of this process without waiting for any peer:
    waits for this rank's own kernels (their waits are time-bounded), gives the
    peers' kernels ``settle_s`` to finish with this rank's memory, then unbinds
    and unmaps.  Returns the number of workspaces freed."""
    mods = [sys.modules.get(f"kernel_b200.tasks.{t}.submission") for t in _SUBMISSION_MODULES]
    held = [m for m in mods if m is not None and getattr(m, "_contexts", None)]
    n = sum(len(m._contexts) for m in held)
    if n == 0:
        return 0
    try:
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        time.sleep(settle_s)
    except Exception:
        pass
    for m in held:
        try:
            m.release_contexts(collective=False)
        except Exception:
            pass
    return n


def _worker_stop(signum, frame):
    """SIGTERM in a worker: the evaluator is replacing its pool (a case ran out of
    time) or leaving.  A process that dies while its memory is bound to a multicast
    object, or mapped by a peer that is still inside a kernel, can fault the peers'
    GPUs; so the worker leaves in order: own kernels done, a pause for the peers'
    (all workers get the signal together and all kernel waits are bounded), then
    unbind and unmap.  A worker stuck inside a library call never gets here; the
    evaluator kills it after ``KB200_EVAL_KILL_GRACE_S``, by which time its peers have
    left the shared memory alone."""
    signal.signal(signal.SIGTERM, signal.SIG_DFL)
    freed = _release_workspaces_locally(settle_s=float(os.environ.get("KB200_EVAL_SETTLE_S", "3")))
    trace = os.environ.get("KB200_EVAL_LIFECYCLE_LOG")
    if trace:
        with open(trace, "a") as f:
            f.write(f"{os.getpid()} stopped in order, {freed} workspace(s) freed\n")
    raise SystemExit(128 + signum)


def _worker_init() -> None:
    signal.signal(signal.SIGTERM, _worker_stop)


def _raise_fd_limit() -> None:
    """A pool worker lives through one process group per case, and a communicator
    over eight GPUs holds descriptors per peer; the soft limit of 1024 that
    containers start with is lifted to the hard limit once per worker."""
    try:
        import resource

        soft, hard = resource.getrlimit(resource.RLIMIT_NOFILE)
        want = hard if hard != resource.RLIM_INFINITY else 1 << 20
        if soft != resource.RLIM_INFINITY and soft < want:
            resource.setrlimit(resource.RLIMIT_NOFILE, (want, hard))
    except (ImportError, ValueError, OSError):
        pass


class _Group:
    """Process-group lifetime of one test, as in ``eval.py:167-184`` of the reference."""

    def __init__(self, cfg: RunConfig, rank: int, world: int):
        self.cfg, self.rank, self.world = cfg, rank, world
        self.device = _device_for(rank, cfg.backend)
        self.sub = None

    def __enter__(self):
        import torch.distributed as dist

        _raise_fd_limit()
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(self.cfg.port)
        kwargs = {}
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            kwargs["device_id"] = self.device
        dist.init_process_group(self.cfg.backend, init_method="env://", rank=self.rank, world_size=self.world, **kwargs)
        return self

    def __exit__(self, exc_type, exc, tb):
        import torch.distributed as dist

        if exc_type is not None and issubclass(exc_type, (SystemExit, KeyboardInterrupt)):
            return False  # the process is leaving: no collective of any kind
        try:
            if exc_type is None:
                # the evaluated module, then the built-in submissions a user module may wrap
                mods = [self.sub] + [sys.modules.get(f"kernel_b200.tasks.{t}.submission") for t in ("all2all", "gemm_rs", "ag_gemm")]
                seen = set()
                for m in mods:
                    if m is not None and id(m) not in seen and hasattr(m, "release_contexts"):
                        seen.add(id(m))
                        m.release_contexts()
        finally:
            dist.destroy_process_group()
        return False


def _any_failed(failed: bool, device: torch.device) -> bool:
    import torch.distributed as dist

    flag = torch.tensor([1 if failed else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    return bool(flag.item())


# --------------------------------------------------------------------- test ----
@_reports_errors
def run_distributed_test(cfg: RunConfig, test: TestCase, rank: int) -> Tuple[bool, str]:
    world = test.args["world_size"]
    with _Group(cfg, rank, world) as g:
        ref, sub = cfg.modules()
        g.sub = sub
        data = ref.generate_input(**_case_args(test, rank, g.device))
        _sync(g.device)
        out = sub.custom_kernel(clone_data(data, g.device))
        _sync(g.device)
        return wrap_check(ref, data, out)


@_reports_errors
def run_local_test(cfg: RunConfig, test: TestCase) -> Tuple[bool, str]:
    device = torch.device("cuda", 0) if cfg.backend == "nccl" else torch.device("cpu")
    ref, sub = cfg.modules()
    args = _case_args(test, None, device)
    args.setdefault("rank", 0)
    args.setdefault("world_size", 1)
    data = ref.generate_input(**args)
    _sync(device)
    out = sub.custom_kernel(clone_data(data, device))
    _sync(device)
    return wrap_check(ref, data, out)


# ---------------------------------------------------------------- benchmark ----
def _timed_call(fn, device: torch.device) -> Tuple[Any, float]:
    """Runs ``fn`` once; returns (result, elapsed ns) measured on the device when
    there is one (CUDA events on the launching stream)."""
    if device.type == "cuda":
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        out = fn()
        end.record()
        torch.cuda.synchronize(device)
        return out, start.elapsed_time(end) * 1e6
    t0 = time.perf_counter_ns()
    out = fn()
    return out, float(time.perf_counter_ns() - t0)


@_reports_errors
def run_distributed_benchmark(cfg: RunConfig, test: TestCase, rank: int, recheck: bool, max_repeats: int,
                              max_time_ns: float):
    import torch.distributed as dist

    world = test.args["world_size"]
    with _Group(cfg, rank, world) as g:
        ref, sub = cfg.modules()
        g.sub = sub
        dev = g.device
        args = dict(test.args)
        data = ref.generate_input(**_case_args(TestCase(args, test.spec), rank, dev))
        out = sub.custom_kernel(clone_data(data, dev))
        good, message = wrap_check(ref, data, out)
        if _any_failed(not good, dev):
            return message or "a peer rank failed the correctness check"
        durations: List[float] = []
        align = torch.zeros(1, device=dev)
        t_begin = time.perf_counter_ns()
        for i in range(max_repeats):
            if recheck:
                if "seed" in args:
                    args["seed"] += 13
                data = ref.generate_input(**_case_args(TestCase(args, test.spec), rank, dev))
            work = clone_data(data, dev)  # outside the timed region
            clear_l2_cache(dev if dev.type == "cuda" else None)
            _sync(dev)
            dist.barrier()
            if dev.type == "cuda":
                # The hosts leave the barrier tens of microseconds apart.  A small all-reduce queued on the
                # stream right before the start event makes the GPUs begin together: every rank's kernel is
                # in its queue by the time the slowest host has joined, so the skew of the hosts does not
                # end up inside the early ranks' kernels as waiting time.
                dist.all_reduce(align)
            out, ns = _timed_call(lambda: sub.custom_kernel(work), dev)
            t = torch.tensor([ns], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            durations.append(float(t.item()))
            message = None
            if recheck:
                good, msg = wrap_check(ref, data, out)
                message = None if good else msg
            del out
            if _any_failed(message is not None, dev):
                return message or "a peer rank failed the re-check"
            stop = False
            if rank == 0 and i > 1:
                stop = should_stop(calculate_stats(durations), max_time_ns, time.perf_counter_ns() - t_begin)
            flag = torch.tensor([1 if stop else 0], dtype=torch.int32, device=dev)
            dist.broadcast(flag, 0)
            if flag.item():
                break
        return calculate_stats(durations)


@_reports_errors
def run_local_benchmark(cfg: RunConfig, test: TestCase, recheck: bool, max_repeats: int, max_time_ns: float):
    dev = torch.device("cuda", 0) if cfg.backend == "nccl" else torch.device("cpu")
    ref, sub = cfg.modules()
    args = dict(test.args)
    args.setdefault("rank", 0)
    args.setdefault("world_size", 1)
    data = ref.generate_input(**_case_args(TestCase(args, test.spec), None, dev))
    out = sub.custom_kernel(clone_data(data, dev))
    good, message = wrap_check(ref, data, out)
    if not good:
        return message
    durations: List[float] = []
    t_begin = time.perf_counter_ns()
    for i in range(max_repeats):
        if recheck:
            if "seed" in args:
                args["seed"] += 13
            data = ref.generate_input(**_case_args(TestCase(args, test.spec), None, dev))
        work = clone_data(data, dev)
        clear_l2_cache(dev if dev.type == "cuda" else None)
        _sync(dev)
        out, ns = _timed_call(lambda: sub.custom_kernel(work), dev)
        if recheck:
            good, message = wrap_check(ref, data, out)
            if not good:
                return message
        del out
        durations.append(ns)
        if i > 1 and should_stop(calculate_stats(durations), max_time_ns, time.perf_counter_ns() - t_begin):
            break
    return calculate_stats(durations)


# ------------------------------------------------------------------ profile ----
@_reports_errors
def run_profile(cfg: RunConfig, test: TestCase, rank: int) -> str:
    from torch.profiler import ProfilerActivity, profile

    world = test.args.get("world_size")

    def body(device, rank_arg):
        ref, sub = cfg.modules()
        args = _case_args(test, rank_arg, device)
        args.setdefault("rank", 0)
        args.setdefault("world_size", 1)
        data = ref.generate_input(**args)
        work = clone_data(data, device)
        sub.custom_kernel(work)  # warm-up: workspace creation is not the kernel
        _sync(device)
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if device.type == "cuda" else [])
        with profile(activities=acts) as prof:
            sub.custom_kernel(work)
            _sync(device)
        key = "self_cuda_time_total" if device.type == "cuda" else "self_cpu_time_total"
        return sub, prof.key_averages().table(sort_by=key, row_limit=20)

    if world is None:
        return body(torch.device("cuda", 0) if cfg.backend == "nccl" else torch.device("cpu"), None)[1]
    with _Group(cfg, rank, world) as g:
        g.sub, table = body(g.device, rank)
        return table


# --------------------------------------------------------------- pool front ----
class WorkerPool:
    """One spawned worker process per rank slot, replaceable after a time-out.

    Rank r of every case runs in worker r, hence on GPU r for the whole run: one
    process per GPU, one CUDA context per process.  (The reference's evaluator
    gives a case's ranks to whichever workers of one shared pool are free,
    ``eval.py:201``, so a worker changes GPU between cases and ends up with a
    context, an allocator pool and per-device kernel attributes on several.)

    A case that ran into its time limit leaves its workers running: they hold the
    rendezvous, their GPUs and possibly a device-side wait, and the next case would
    be queued behind them (the reference's evaluator has the same weakness).
    ``rebuild`` terminates those processes and starts fresh ones."""

    def __init__(self, n_workers: int):
        self.n_workers = n_workers
        self._ctx = multiprocessing.get_context("spawn")
        self.pools = [self._ctx.Pool(1, initializer=_worker_init) for _ in range(n_workers)]
        self.rebuilds = 0

    def _stop(self) -> None:
        """SIGTERM to every worker at once (they leave in order, see ``_worker_stop``),
        SIGKILL for those that have not left after ``KB200_EVAL_KILL_GRACE_S``."""
        procs = [w for p in self.pools for w in list(getattr(p, "_pool", []))]
        for w in procs:
            if w.is_alive():
                w.terminate()
        t_end = time.monotonic() + KILL_GRACE_S
        while any(w.is_alive() for w in procs) and time.monotonic() < t_end:
            time.sleep(0.05)
        for w in procs:
            if w.is_alive():
                w.kill()
        for p in self.pools:
            p.terminate()
        for p in self.pools:
            p.join()

    def rebuild(self) -> None:
        self._stop()
        self.pools = [self._ctx.Pool(1, initializer=_worker_init) for _ in range(self.n_workers)]
        self.rebuilds += 1

    def apply(self, fn, args, slot: int = 0):
        return self.pools[slot % self.n_workers].apply(fn, args)

    def apply_async(self, fn, args, slot: int = 0):
        return self.pools[slot % self.n_workers].apply_async(fn, args)

    def close(self) -> None:
        self._stop()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class Runner:
    """Dispatches the per-rank workers of every case onto the worker pool."""

    def __init__(self, pool, n_gpus: int, task: Optional[str], impl: str, backend: str):
        self.pool, self.n_gpus, self.task, self.impl, self.backend = pool, n_gpus, task, impl, backend

    def _timed_out(self) -> None:
        if hasattr(self.pool, "rebuild"):
            self.pool.rebuild()

    def _cfg(self, test: TestCase) -> RunConfig:
        return RunConfig(task=self.task or guess_task(test.args), impl=self.impl, backend=self.backend, port=free_port())

    def _world(self, test: TestCase) -> Optional[int]:
        world = test.args.get("world_size")
        if world is not None and world > self.n_gpus:
            raise SpecError(f"world_size {world} exceeds the {self.n_gpus} worker processes (POPCORN_GPUS)")
        return world

    def _collect(self, pending, limit_s: float):
        """Results of the per-rank workers in rank order.  Waits ``limit_s`` for all
        of them, but once one rank has failed only ``FAIL_GRACE_S`` longer: its peers
        sit in a collective or a device-side wait that nobody will complete.  A rank
        without a result gets a ``WorkerFailure`` and the pool is rebuilt."""
        t_end = time.monotonic() + limit_s
        results: List[Any] = [None] * len(pending)
        have = [False] * len(pending)
        failed_at = None
        while not all(have):
            for i, p in enumerate(pending):
                if have[i] or not p.ready():
                    continue
                try:
                    results[i] = p.get(0)
                except Exception as e:  # the result could not be delivered as sent
                    results[i] = WorkerFailure(f"{type(e).__name__}: {e}")
                have[i] = True
                if isinstance(results[i], WorkerFailure) and failed_at is None:
                    failed_at = time.monotonic()
            now = time.monotonic()
            if all(have) or now > t_end or (failed_at is not None and now > failed_at + FAIL_GRACE_S):
                break
            time.sleep(0.02)
        if not all(have):
            why = f"timed out after {limit_s:g} s" if failed_at is None else "no result: a peer rank failed"
            for i in range(len(pending)):
                if not have[i]:
                    results[i] = WorkerFailure(why)
            self._timed_out()
        return results

    def test(self, test: TestCase) -> Tuple[bool, str]:
        try:
            world = self._world(test)
        except SpecError as e:
            return False, str(e)
        cfg = self._cfg(test)
        if world is None:
            res = self.pool.apply(run_local_test, (cfg, test))
            return (False, str(res)) if isinstance(res, WorkerFailure) else res
        pending = [self.pool.apply_async(run_distributed_test, (cfg, test, r), r) for r in range(world)]
        results = [(False, str(r)) if isinstance(r, WorkerFailure) else r for r in self._collect(pending, TEST_TIMEOUT_S)]
        ok = all(r[0] for r in results)
        errors = "\n".join(f"rank {i} - {r[1]}" for i, r in enumerate(results) if not r[0])
        return ok, errors

    def benchmark(self, test: TestCase, recheck: bool, max_repeats: int, max_time_ns: float):
        try:
            world = self._world(test)
        except SpecError as e:
            return str(e)
        cfg = self._cfg(test)
        if world is None:
            res = self.pool.apply(run_local_benchmark, (cfg, test, recheck, max_repeats, max_time_ns))
            return str(res) if isinstance(res, WorkerFailure) else res
        pending = [self.pool.apply_async(run_distributed_benchmark, (cfg, test, r, recheck, max_repeats, max_time_ns), r)
                   for r in range(world)]
        results = self._collect(pending, BENCH_TIMEOUT_S)
        failed = [(i, r) for i, r in enumerate(results) if not isinstance(r, Stats)]
        if failed:
            return "\n".join(f"rank {i} - {msg}" for i, msg in failed)
        return results[0]  # every rank holds the same MAX-reduced samples

    def profile(self, test: TestCase) -> str:
        world = self._world(test)
        cfg = self._cfg(test)
        if world is None:
            return str(self.pool.apply(run_profile, (cfg, test, 0)))
        pending = [self.pool.apply_async(run_profile, (cfg, test, r), r) for r in range(world)]
        return str(self._collect(pending, BENCH_TIMEOUT_S)[0])


def case_roofline_us(task: str, args: dict) -> Optional[float]:
    """Roofline of a case in microseconds (slower of FLOPs at the nominal bf16 peak
    and NVLink bytes at 900 GB/s per direction), or None if the keys are missing."""
    from ..utils import roofline as rf

    try:
        world = int(args.get("world_size", 1))
        if task == "all2all":
            eb = 4 if str(args.get("dtype", "fp16")) in ("fp32", "float32") else 2
            return rf.a2a_roofline_us(args["max_num_tokens"], args["experts_per_token"], args["hidden_dim"], eb, world)["roofline_us"]
        if task == "gemm_rs":
            return rf.gemm_rs_roofline_us(args["m"], args["n"], args["k"], world)["roofline_us"]
        if task == "ag_gemm":
            return rf.ag_gemm_roofline_us(args["m"], args["n"], args["k"], world)["roofline_us"]
    except (KeyError, ZeroDivisionError):
        pass
    return None


def _log_stats(logger: PopcornOutput, idx: int, stats: Stats, task: Optional[str] = None, args: Optional[dict] = None,
               baseline: Optional[Stats] = None) -> dict:
    """Logs the reference's six keys (ns) plus, in microseconds, ``max_rank_us``,
    ``roofline_us`` / ``roofline_frac`` and, when a baseline was timed,
    ``baseline_us`` / ``speedup``.  Returns the row for the JSON dump."""
    row = {}
    for field in dataclasses.fields(Stats):
        logger.log(f"benchmark.{idx}.{field.name}", getattr(stats, field.name))
        row[field.name] = getattr(stats, field.name)
    row["max_rank_us"] = stats.mean / 1e3
    logger.log(f"benchmark.{idx}.max_rank_us", row["max_rank_us"])
    roof = case_roofline_us(task, args) if task and args else None
    if roof is not None and stats.mean > 0:
        row["roofline_us"], row["roofline_frac"] = roof, roof / row["max_rank_us"]
        logger.log(f"benchmark.{idx}.roofline_us", roof)
        logger.log(f"benchmark.{idx}.roofline_frac", row["roofline_frac"])
    if baseline is not None:
        row["baseline_us"], row["speedup"] = baseline.mean / 1e3, baseline.mean / stats.mean
        logger.log(f"benchmark.{idx}.baseline_us", row["baseline_us"])
        logger.log(f"benchmark.{idx}.speedup", row["speedup"])
    return row


def run_testing(logger: PopcornOutput, runner: Runner, tests: List[TestCase]) -> int:
    passed = True
    logger.log("test-count", len(tests))
    for idx, test in enumerate(tests):
        logger.log(f"test.{idx}.spec", test.spec)
        good, message = runner.test(test)
        if good:
            logger.log(f"test.{idx}.status", "pass")
            if message:
                logger.log(f"test.{idx}.message", message)
        else:
            logger.log(f"test.{idx}.status", "fail")
            logger.log(f"test.{idx}.error", message)
            passed = False
    logger.log("check", "pass" if passed else "fail")
    return EXIT_OK if passed else EXIT_FAIL


def run_benchmarking(logger: PopcornOutput, runner: Runner, tests: List[TestCase], leaderboard: bool,
                     baseline_runner: Optional[Runner] = None, json_path: Optional[str] = None,
                     max_repeats: int = 100) -> int:
    runner.benchmark(tests[0], False, max_repeats, 1e7 if leaderboard else 1e8)  # warm-up
    logger.log("benchmark-count", len(tests))
    passed = True
    rows = []
    for idx, test in enumerate(tests):
        logger.log(f"benchmark.{idx}.spec", test.spec)
        result = runner.benchmark(test, leaderboard, max_repeats, 30e9 if leaderboard else 10e9)
        if isinstance(result, Stats):
            base = None
            if baseline_runner is not None:
                b = baseline_runner.benchmark(test, False, max_repeats, 10e9)
                base = b if isinstance(b, Stats) else None
            row = _log_stats(logger, idx, result, runner.task or guess_task(test.args), test.args, base)
            rows.append({"spec": test.spec, **row})
        else:
            passed = False
            logger.log(f"benchmark.{idx}.status", "fail")
            logger.log(f"benchmark.{idx}.error", str(result))
            rows.append({"spec": test.spec, "error": str(result)})
            if leaderboard:
                break
    timed = [r for r in rows if "max_rank_us" in r]
    if timed and len(timed) == len(rows):
        # the ranking quantity of the reference: geometric mean of the benchmark means (task.yml:79)
        geo = math.exp(sum(math.log(r["max_rank_us"]) for r in timed) / len(timed))
        logger.log("geomean_us", geo)
        if all("baseline_us" in r for r in timed):
            base = math.exp(sum(math.log(r["baseline_us"]) for r in timed) / len(timed))
            logger.log("baseline_geomean_us", base)
            logger.log("geomean_speedup", base / geo)
    if json_path:
        Path(json_path).write_text(json.dumps(rows, indent=1))
    logger.log("check", "pass" if passed else "fail")
    return EXIT_OK if passed else EXIT_FAIL


def run_profiling(logger: PopcornOutput, runner: Runner, tests: List[TestCase]) -> int:
    logger.log("benchmark-count", len(tests))
    for idx, test in enumerate(tests):
        logger.log(f"benchmark.{idx}.spec", test.spec)
        report = runner.profile(test)
        logger.log(f"benchmark.{idx}.report", base64.b64encode(report.encode("utf-8"), b"+*").decode("utf-8"))
    logger.log("check", "pass")
    return EXIT_OK


def main(argv: Optional[List[str]] = None) -> int:
    fd = os.getenv("POPCORN_FD")
    if not fd:
        return EXIT_NO_FD
    ap = argparse.ArgumentParser(prog="kernel_b200.harness.eval", add_help=True)
    ap.add_argument("mode", nargs="?")
    ap.add_argument("tests_file", nargs="?")
    ap.add_argument("--task", choices=["all2all", "gemm_rs", "ag_gemm"])
    ap.add_argument("--impl", choices=["fused", "baseline"], default="fused")
    ap.add_argument("--submission", default=None, help="module (pkg.mod) or file (path/to/file.py) with a custom_kernel to evaluate instead of --impl")
    ap.add_argument("--backend", choices=["nccl", "gloo"], default="nccl" if torch.cuda.is_available() else "gloo")
    ap.add_argument("--yaml")
    ap.add_argument("--section", default=None)
    ap.add_argument("--world", type=int, default=None, help="override world_size of every case")
    ap.add_argument("--with-baseline", action="store_true", help="benchmark modes: also time the NCCL+cuBLAS baseline and log baseline_us / speedup")
    ap.add_argument("--json", default=None, help="benchmark modes: also write the rows to this file")
    ap.add_argument("--max-repeats", type=int, default=100,
                    help="benchmark modes: timed calls per case at most (the reference's evaluator uses 100, eval.py:338)")
    try:
        ns = ap.parse_args(argv)
    except SystemExit:
        return EXIT_USAGE
    if ns.mode is None or (ns.tests_file is None and ns.yaml is None):
        return EXIT_USAGE
    if ns.mode not in ("test", "benchmark", "leaderboard", "profile"):
        return EXIT_USAGE

    seed_env = os.getenv("POPCORN_SEED")
    os.environ.pop("POPCORN_SEED", None)
    seed = int(seed_env) if seed_env else None
    n_gpus = int(os.getenv("POPCORN_GPUS", "1"))
    set_seed(seed or 42)
    try:
        if ns.yaml:
            section = ns.section or ("tests" if ns.mode == "test" else "benchmarks")
            tests = cases_from_yaml(ns.yaml, section, seed)
        else:
            tests = parse_tests(Path(ns.tests_file).read_text(), seed)
    except (OSError, SpecError) as e:
        print(f"Could not read test cases: {e}", file=sys.stderr)
        return EXIT_BAD_TESTS
    if not tests:
        print("no test cases", file=sys.stderr)
        return EXIT_BAD_TESTS
    if ns.world is not None:
        for t in tests:
            if "world_size" in t.args:
                t.args["world_size"] = ns.world

    def _terminated(signum, frame):
        # leave through the context managers below: the pool's workers (and what they
        # hold on the GPUs) must not outlive an evaluator that was told to stop
        raise SystemExit(128 + signum)

    try:
        signal.signal(signal.SIGTERM, _terminated)
    except ValueError:  # not the main thread
        pass
    with PopcornOutput(int(fd)) as logger:
        with WorkerPool(n_gpus) as pool:
            runner = Runner(pool, n_gpus, ns.task, ns.submission or ns.impl, ns.backend)
            if ns.mode == "test":
                return run_testing(logger, runner, tests)
            base_runner = Runner(pool, n_gpus, ns.task, "baseline", ns.backend) if ns.with_baseline else None
            if ns.mode == "benchmark":
                return run_benchmarking(logger, runner, tests, False, base_runner, ns.json, max(3, ns.max_repeats))
            if ns.mode == "leaderboard":
                return run_benchmarking(logger, runner, tests, True, base_runner, ns.json, max(3, ns.max_repeats))
            return run_profiling(logger, runner, tests)


if __name__ == "__main__":
    sys.exit(main())
