#!/usr/bin/env python
"""Headline benchmark: per-call device time of the three fused ops.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One *step* calls each op once on its flagship configuration:

  a2a      MoE dispatch + combine, 256 experts, top-8, hidden 7168, 2048 tokens
           in total (256 per rank on 8 GPUs), bf16
  gemm_rs  GEMM + reduce-scatter, M=8192 N=8192 K=29568 sharded N-way, bf16, bias
  ag_gemm  all-gather + GEMM, M=8192 K=8192 N=29568 sharded N-way, bf16, bias

Before anything is timed every op runs once and its result goes through the
task's own checker (collective, outside the timed region), as the reference's
evaluator checks before it times (``eval.py:327-334``); a failed check or a
device status word left non-zero after the timed loops ends the run with a
non-zero exit code.

Every op call is timed on the device (CUDA events on the launching stream, L2
flushed and the ranks aligned by a tiny in-stream all-reduce just before the
start event), the maximum over ranks is taken per call, and ``value`` is the
geometric mean of the three mean per-call times in microseconds (the reference
ranks by geometric mean, ``task.yml:79``); medians are printed beside the means.
``e2e`` repeats the measurement with the per-step activations in pinned host
memory and the result wanted there, copies inside the timed region: the GEMM
ops through ``GemmRS.run_from_host`` / ``AGGemm.run_from_host`` (chunks of rows
copied in and out while the fused kernel works on the chunk between them), the
MoE op through ``custom_kernel`` bracketed by its copies.

``--impl reference`` runs the unmodified reference (installed under
``baseline/_ref``) through its own ``custom_kernel`` functions on the same
configurations; the all-gather + GEMM, which the reference does not have, is
``all_gather_into_tensor`` + ``matmul`` there.

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N``.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import signal
import socket
import sys
import threading
import time
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

A2A = dict(num_experts=256, experts_per_token=8, hidden_dim=7168)
A2A_TOTAL_TOKENS = 2048  # 256 per rank on 8 GPUs; the total is fixed as N changes
GEMM_RS = dict(m=8192, n=8192, k=29568)
AG_GEMM = dict(m=8192, n=29568, k=8192)
# Published reference numbers (8xMI300X speed-of-light tables, task.yml:55 and
# gemm_rs/task.yml:54); the reference publishes nothing for ag_gemm.
PUBLISHED_US = {"a2a": 104.36, "gemm_rs": 379.43}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    return ap.parse_args()


# ------------------------------------------------------------------ clocks ----
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML (read-only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.005):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.power, self.stamps, self.masks, self.reasons, self.max_mhz = [], [], [], [], set(), None
        self.window = [None, None, None]
        self._stop_evt = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        while not self._stop_evt.is_set():
            try:
                clock = self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)
                power = self.nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.samples.append(clock)
                self.power.append(power)
                self.masks.append(mask)
                self.stamps.append(time.perf_counter())
            except Exception:
                pass
            self._stop_evt.wait(self.period)

    def mark(self, which: int) -> None:
        """Start (0) or end (1) of the timed region, start of its warm-up (2); the summary covers the
        samples between 0 and 1, or, when those are fewer than three, between 2 and 1."""
        self.window[which] = time.perf_counter()

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=2)
        t0, t1, tw = self.window

        def between(lo, hi):
            return [i for i, t in enumerate(self.stamps) if (lo is None or t >= lo) and (hi is None or t <= hi)]

        keep = between(t0, t1)
        if len(keep) < 3:  # a region shorter than a few sampling periods: the warm-up steps (same work) count too
            keep = between(tw, t1)
        if len(keep) < 3:
            keep = list(range(len(self.stamps)))
        clocks = [self.samples[i] for i in keep]
        power = [self.power[i] for i in keep]
        for i in keep:
            for bit, name in self.REASONS.items():
                if self.masks[i] & bit:
                    self.reasons.add(name)
        s = sorted(clocks)
        # "under load": the samples taken while the board drew more than half of its peak draw in this window
        peak = max(power) if power else 0.0
        loaded = sorted(c for c, w in zip(clocks, power) if w >= 0.5 * peak) if peak > 0 else s
        return {"sm_mhz": loaded[len(loaded) // 2] if loaded else (s[len(s) // 2] if s else None),
                "sm_mhz_all_samples_median": s[len(s) // 2] if s else None, "sm_mhz_min": s[0] if s else None,
                "sm_max_mhz": self.max_mhz, "power_w_max": round(peak, 1), "reasons": sorted(self.reasons), "samples": len(s)}


# ---------------------------------------------------------------- plumbing ----
def init_dist(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}; launch with torch.distributed.run --nproc-per-node {n_gpus}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MASTER_PORT" not in os.environ:
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            os.environ["MASTER_PORT"] = str(s.getsockname()[1])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    return rank, world, dev


class L2Flush:
    def __init__(self, dev):
        self.buf = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def __call__(self):
        self.buf.fill_(1)


def geomean(vals):
    return math.exp(sum(math.log(v) for v in vals) / len(vals))


# ------------------------------------------------------------------- inputs ----
def make_inputs(rank: int, world: int, dev):
    """Seeded synthetic inputs of the flagship shapes (host-generated so that both
    arms and every run see identical data), on the device and in pinned memory."""
    g = torch.Generator().manual_seed(1234 + rank)
    T, E, k, H = A2A_TOTAL_TOKENS // world, A2A["num_experts"], A2A["experts_per_token"], A2A["hidden_dim"]
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    idx = torch.rand(T, E, generator=g).argsort(dim=1)[:, :k].to(torch.int32).contiguous()
    w = torch.softmax(torch.randn(T, k, generator=g), dim=-1)
    kl = GEMM_RS["k"] // world
    a_rs = torch.randn(GEMM_RS["m"], kl, generator=g).to(torch.bfloat16)
    w_rs = (torch.randn(GEMM_RS["n"], kl, generator=g) / GEMM_RS["k"] ** 0.5).to(torch.bfloat16)
    gb = torch.Generator().manual_seed(99)
    b_rs = (torch.randn(GEMM_RS["n"], generator=gb) * 0.02).to(torch.bfloat16)
    ml, nl = AG_GEMM["m"] // world, AG_GEMM["n"] // world
    a_ag = torch.randn(ml, AG_GEMM["k"], generator=g).to(torch.bfloat16)
    w_ag = (torch.randn(nl, AG_GEMM["k"], generator=g) / AG_GEMM["k"] ** 0.5).to(torch.bfloat16)
    b_ag = (torch.randn(nl, generator=g) * 0.02).to(torch.bfloat16)
    host = dict(x=x, idx=idx, w=w, a_rs=a_rs, a_ag=a_ag)
    host = {k_: v.pin_memory() for k_, v in host.items()}
    devt = {k_: v.to(dev) for k_, v in host.items()}
    devt.update(w_rs=w_rs.to(dev), b_rs=b_rs.to(dev), w_ag=w_ag.to(dev), b_ag=b_ag.to(dev))
    return host, devt


# ---------------------------------------------------------------- our arm ----
class OursArm:
    name = "ours"

    def __init__(self, rank, world, dev):
        from kernel_b200.ops import dispatch_combine, gemm
        from kernel_b200.tasks.ag_gemm import reference as ag_ref
        from kernel_b200.tasks.ag_gemm import submission as ag
        from kernel_b200.tasks.all2all import reference as a2a_ref
        from kernel_b200.tasks.all2all import submission as a2a
        from kernel_b200.tasks.gemm_rs import reference as rs_ref
        from kernel_b200.tasks.gemm_rs import submission as rs
        from kernel_b200.tasks.gemm_rs.task import GemmRSInput

        self.mods = (dispatch_combine, gemm)
        self.a2a, self.rs, self.ag = a2a, rs, ag
        self.a2a_ref, self.rs_ref, self.ag_ref = a2a_ref, rs_ref, ag_ref
        self.rs_input = lambda a, w, b: GemmRSInput((a, w, b), "once")  # bias added once, as the flagship config says
        self.rank, self.world, self.dev = rank, world, dev
        self.cfg = a2a_ref.MoEConfig(**A2A, max_num_tokens=A2A_TOTAL_TOKENS // world, in_dtype=torch.bfloat16,
                                     out_dtype=torch.bfloat16, expert_scale=2)

    def _a2a_data(self, x, idx, w):
        rd = object.__new__(self.a2a_ref.RankTestData)
        rd.num_tokens, rd.x, rd.indices, rd.weights = x.shape[0], x, idx, w
        return self.cfg, rd, self.rank, self.world

    def a2a_call(self, x, idx, w, fresh_inputs=False):
        return self.a2a.custom_kernel(self._a2a_data(x, idx, w))

    def rs_call(self, a, w, b):
        return self.rs.custom_kernel(self.rs_input(a, w, b))

    def ag_call(self, a, w, b):
        return self.ag.custom_kernel((a, w, b))

    # activations in pinned host memory, result into pinned host memory
    def rs_from_host(self, a_host, w, b, out_host):
        return self.rs.get_context(a_host.shape[0], w.shape[0], w.device).run_from_host(a_host, w, b, bias_scale=1.0,
                                                                                        out_host=out_host)

    def ag_from_host(self, a_host, w, b, out_host):
        return self.ag.get_context(a_host.shape[0] * self.world, a_host.shape[1], w.device).run_from_host(
            a_host, w, b, out_host=out_host)

    def check(self, name, inputs, out):
        """The task's own checker (collective)."""
        if name == "a2a":
            return self.a2a_ref.check_implementation(self._a2a_data(*inputs), out)
        if name == "gemm_rs":
            return self.rs_ref.check_implementation(self.rs_input(*inputs), out)
        return self.ag_ref.check_implementation(tuple(inputs), out)

    def device_status(self) -> int:
        """First non-zero device status word of any cached workspace (0 = healthy)."""
        torch.cuda.synchronize()
        for mod in (self.a2a, self.rs, self.ag):
            for ctx in mod._contexts.values():
                subs = [ctx] + [sub for sub, _ in getattr(ctx, "_stream_state", {}).values()]
                for c in subs:
                    st = getattr(c, "status", None)
                    if st is not None and int(st[0]) != 0:
                        return int(st[0])
        return 0

    def launches(self) -> int:
        return self.mods[0].launch_count + self.mods[1].launch_count

    def close(self):
        self.a2a.release_contexts()
        self.rs.release_contexts()
        self.ag.release_contexts()


# ----------------------------------------------------------- reference arm ----
class ReferenceArm:
    """The unmodified reference, imported from ``baseline/_ref``."""

    name = "reference"

    def __init__(self, rank, world, dev):
        ref_root = ROOT / "baseline" / "_ref" / "sss_kernel_ref"
        if not (ref_root / "submission.py").exists():
            raise FileNotFoundError("baseline/_ref is not installed")
        self.rank, self.world, self.dev = rank, world, dev

        def load(dirpath):
            for name in ("task", "reference", "submission"):
                sys.modules.pop(name, None)
            sys.path.insert(0, str(dirpath))
            try:
                import reference as r  # noqa: the reference's own module names
                import submission as s
            finally:
                sys.path.pop(0)
            for name in ("task", "reference", "submission"):
                sys.modules.pop(name, None)
            return r, s

        self.notes = {}
        self.a2a_ref, self.a2a_sub = load(ref_root)
        self.rs_ref, self.rs_sub = load(ref_root / "gemm_rs")
        self.cfg = self.a2a_ref.MoEConfig(**A2A, max_num_tokens=A2A_TOTAL_TOKENS // world, in_dtype=torch.bfloat16,
                                          out_dtype=torch.bfloat16)

    def _a2a_data(self, x, idx, w):
        rd = object.__new__(self.a2a_ref.RankTestData)
        rd.num_tokens, rd.x, rd.indices, rd.weights = x.shape[0], x, idx, w
        return self.cfg, rd, self.rank, self.world

    def a2a_call(self, x, idx, w, fresh_inputs=False):
        if fresh_inputs:
            # The reference's custom_kernel works on side streams that do not wait
            # for the stream that produced its inputs (submission.py:16-17,199-201);
            # inputs that were just copied in must have landed before it is called.
            torch.cuda.current_stream().synchronize()
        return self.a2a_sub.custom_kernel(self._a2a_data(x, idx, w))

    def rs_call(self, a, w, b):
        return self.rs_sub.custom_kernel((a, w, b))

    def ag_call(self, a, w, b):
        # The reference has no all-gather + GEMM; this is the same library path
        # (NCCL collective + cuBLAS GEMM + bias add) its gemm_rs submission uses.
        full = torch.empty((a.shape[0] * self.world, a.shape[1]), dtype=a.dtype, device=a.device)
        dist.all_gather_into_tensor(full, a)
        return torch.matmul(full, w.t()) + b

    # The reference has no host-streaming entry point: copy in, its custom_kernel, copy out.
    def rs_from_host(self, a_host, w, b, out_host):
        out_host.copy_(self.rs_call(a_host.to(self.dev, non_blocking=True), w, b), non_blocking=True)
        return out_host

    def ag_from_host(self, a_host, w, b, out_host):
        out_host.copy_(self.ag_call(a_host.to(self.dev, non_blocking=True), w, b), non_blocking=True)
        return out_host

    def check(self, name, inputs, out):
        """The reference's own checkers where it has one (all2all, gemm_rs).  Its
        all2all checker compares in the data type at rtol 1e-2 / atol 5e-3, which its
        own submission misses in bf16 at this size (it accumulates the k weighted rows
        in another order than its oracle); such a result is then compared with the
        closed form out[t] = x[t] * sum_k w[t,k] * (1 + owner rank of expert k) in fp32
        at 3e-2, and the verdict of that comparison is reported with a note."""
        if name == "a2a":
            res = self.a2a_ref.check_implementation(self._a2a_data(*inputs), out)
            ok = bool(res[0]) if isinstance(res, tuple) else not bool(res)
            if not ok:
                x, idx, w = inputs
                owner = (idx.long() // (A2A["num_experts"] // self.world)).float() + 1.0
                expect = x.float() * (w * owner).sum(-1, keepdim=True)
                close = torch.allclose(out.float(), expect, rtol=3e-2, atol=3e-2)
                self.notes["a2a"] = ("the reference's checker rejects the reference's own submission at this size in bf16; "
                                     "compared with the fp32 closed form at rtol = atol = 3e-2 instead")
                return bool(close), "" if close else "a2a differs from the closed form"
            return True, ""
        elif name == "gemm_rs":
            res = self.rs_ref.check_implementation(tuple(inputs), out)
        else:
            a, w, b = inputs
            full = torch.empty((a.shape[0] * self.world, a.shape[1]), dtype=a.dtype, device=a.device)
            dist.all_gather_into_tensor(full, a)
            ok = torch.allclose(out.float(), full.float() @ w.float().t() + b.float(), rtol=1e-2, atol=1e-2)
            res = (bool(ok), "" if ok else "ag_gemm differs from the fp32 product")
        if isinstance(res, tuple):
            return bool(res[0]), str(res[1])
        return (not bool(res)), str(res)

    def device_status(self) -> int:
        return 0

    def launches(self) -> int:
        return 0

    def close(self):
        pass


# ------------------------------------------------------------------ timing ----
def _stop_in_order(signum, frame):
    # A launcher's or a caller's time limit arrives as SIGTERM: leave through the handler of
    # run() below, which waits for this rank's kernels and unbinds the workspaces, instead of
    # dying with memory bound to a multicast object that the other ranks still use.
    signal.signal(signal.SIGTERM, signal.SIG_DFL)
    raise SystemExit(128 + signum)


def run(args):
    signal.signal(signal.SIGTERM, _stop_in_order)
    rank, world, dev = init_dist(args.gpus)
    try:
        arm = OursArm(rank, world, dev) if args.impl == "ours" else ReferenceArm(rank, world, dev)
    except Exception as e:  # the reference arm may be absent
        if args.impl == "reference":
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"}))
            dist.destroy_process_group()
            return 0
        raise
    try:
        return _measure(args, arm, rank, world, dev)
    except BaseException:
        # Leave in order even when something failed: wait for this rank's kernels and
        # release the workspaces (which unbinds their memory from the multicast
        # object) without waiting for peers that may be gone.
        try:
            torch.cuda.synchronize()
            for mod in (getattr(arm, "a2a", None), getattr(arm, "rs", None), getattr(arm, "ag", None)):
                for ctx in list(getattr(mod, "_contexts", {}).values()):
                    for sub, _ in getattr(ctx, "_stream_state", {}).values():
                        if sub is not ctx and sub.heap is not None:
                            sub.heap.close(collective=False)
                    if ctx.heap is not None:
                        ctx.heap.close(collective=False)
        except Exception:
            pass
        raise


def _measure(args, arm, rank, world, dev):
    # The sampler starts before the inputs are made: the first NVML queries of a process take tens of
    # milliseconds (eight ranks initialise the library at once), longer than a whole timed region at 8 GPUs.
    sampler = ClockSampler(dev.index, period_s=0.002)
    sampler.start()
    host, d = make_inputs(rank, world, dev)
    flush = L2Flush(dev)
    align = torch.zeros(1, device=dev)
    T_rank = A2A_TOTAL_TOKENS // world
    pinned_out = {
        "a2a": torch.empty((T_rank, A2A["hidden_dim"]), dtype=torch.bfloat16).pin_memory(),
        "gemm_rs": torch.empty((GEMM_RS["m"] // world, GEMM_RS["n"]), dtype=torch.bfloat16).pin_memory(),
        "ag_gemm": torch.empty((AG_GEMM["m"], AG_GEMM["n"] // world), dtype=torch.bfloat16).pin_memory(),
    }
    inputs = {
        "a2a": (d["x"], d["idx"], d["w"]),
        "gemm_rs": (d["a_rs"], d["w_rs"], d["b_rs"]),
        "ag_gemm": (d["a_ag"], d["w_ag"], d["b_ag"]),
    }
    ops = {
        "a2a": (lambda: arm.a2a_call(*inputs["a2a"]), ("x", "idx", "w")),
        "gemm_rs": (lambda: arm.rs_call(*inputs["gemm_rs"]), ("a_rs",)),
        "ag_gemm": (lambda: arm.ag_call(*inputs["ag_gemm"]), ("a_ag",)),
    }

    def e2e_call(name):
        # host -> device copies of this step's activations, the op, device -> host
        # copy of the result: all inside the events.
        if name == "a2a":
            out = arm.a2a_call(host["x"].to(dev, non_blocking=True), host["idx"].to(dev, non_blocking=True),
                               host["w"].to(dev, non_blocking=True), fresh_inputs=True)
            pinned_out[name].copy_(out, non_blocking=True)
        elif name == "gemm_rs":
            arm.rs_from_host(host["a_rs"], d["w_rs"], d["b_rs"], pinned_out[name])
        else:
            arm.ag_from_host(host["a_ag"], d["w_ag"], d["b_ag"], pinned_out[name])

    # ---- correctness gate: every op once, through the checker, before any timing ----
    def all_ranks(ok: bool) -> bool:
        t = torch.tensor([0 if ok else 1], device=dev)
        dist.all_reduce(t)
        return int(t.item()) == 0

    def run_check(name, out):
        try:
            return arm.check(name, inputs[name], out)
        except Exception as e:  # a checker that cannot run is a failed check, not a crash of the bench
            return False, f"checker raised {type(e).__name__}: {e}"

    checked, checked_e2e, errors = {}, {}, []
    for name, (fn, _) in ops.items():
        out = fn()
        torch.cuda.synchronize()
        ok, msg = run_check(name, out)
        checked[name] = all_ranks(ok)
        if not ok:
            errors.append(f"rank {rank} {name}: {msg}"[:300])
        e2e_call(name)
        torch.cuda.synchronize()
        ok, msg = run_check(name, pinned_out[name].to(dev))
        checked_e2e[name] = all_ranks(ok)
        if not ok:
            errors.append(f"rank {rank} {name} (from host): {msg}"[:300])
        del out

    def timed(fn):
        flush()
        dist.all_reduce(align)  # aligns the ranks on the stream, right before the start event
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        return e0, e1

    def step(collect, e2e):
        for name, (fn, _) in ops.items():
            ev = timed((lambda n=name: e2e_call(n)) if e2e else fn)
            if collect is not None:
                collect[name].append(ev)

    def reduce_times(events):
        out = {}
        for name, evs in events.items():
            t = torch.tensor([a.elapsed_time(b) * 1e3 for a, b in evs], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            out[name] = t.tolist()
        return out

    def measure(e2e: bool, sampler=None):
        if sampler is not None:
            sampler.mark(2)
        for _ in range(args.warmup):
            step(None, e2e)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        before = arm.launches()
        events = {n: [] for n in ops}
        if sampler is not None:
            sampler.mark(0)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            step(events, e2e)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
        if sampler is not None:
            sampler.mark(1)
        return reduce_times(events), arm.launches() - before, wall

    per_call, launches, wall = measure(e2e=False, sampler=sampler)
    clocks = sampler.stop()
    e2e_calls, _, _ = measure(e2e=True)
    status_word = arm.device_status()
    status_t = torch.tensor([status_word], device=dev)
    dist.all_reduce(status_t, op=dist.ReduceOp.MAX)
    status_word = int(status_t.item())

    def median(v):
        s_ = sorted(v)
        return s_[len(s_) // 2] if len(s_) % 2 else 0.5 * (s_[len(s_) // 2 - 1] + s_[len(s_) // 2])

    mean = {n: sum(v) / len(v) for n, v in per_call.items()}
    mean_e2e = {n: sum(v) / len(v) for n, v in e2e_calls.items()}
    value = geomean(list(mean.values()))
    h2d = sum(host[k].numel() * host[k].element_size() for _, (_, keys) in ops.items() for k in keys)
    d2h = sum(t.numel() * t.element_size() for t in pinned_out.values())
    published = geomean([PUBLISHED_US["a2a"], PUBLISHED_US["gemm_rs"]])
    ours_two = geomean([mean["a2a"], mean["gemm_rs"]])
    failed = not (all(checked.values()) and all(checked_e2e.values())) or status_word != 0
    result = {
        "metric": "per-call us (device-timed, max over ranks), geometric mean of dispatch+combine, gemm_rs, ag_gemm",
        "value": round(value, 3),
        "unit": "us",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(sum(mean.values()) / 1e3, 5),
        "higher_is_better": False,
        "scaling": "strong",
        "vs_baseline": round(ours_two / published, 4),
        "vs_baseline_note": "geomean(a2a, gemm_rs) / geomean of the reference's published 8xMI300X speed-of-light "
                            "figures for the same two shapes at 8 ranks (104.36, 379.43 us); nothing is published for ag_gemm",
        "dtype": "bf16",
        "data": "synthetic (seeded N(0,1) activations, N(0,1)/sqrt(K) weights, softmax routing weights; random-init)",
        "impl": args.impl,
        "checked": checked,
        "checked_from_host": checked_e2e,
        **({"checked_notes": arm.notes} if getattr(arm, "notes", None) else {}),
        "device_status": status_word,
        "per_op_us": {n: round(v, 3) for n, v in mean.items()},
        "per_op_median_us": {n: round(median(v), 3) for n, v in per_call.items()},
        "per_op_best_us": {n: round(min(v), 3) for n, v in per_call.items()},
        "config": {
            "model": f"a2a E=256 top-8 H=7168 T={A2A_TOTAL_TOKENS} in total ({T_rank}/rank) bf16 | gemm_rs M=8192 N=8192 "
                     "K=29568 bias | ag_gemm M=8192 N=29568 K=8192 bias",
            "global_batch": A2A_TOTAL_TOKENS,
            "seq_len": GEMM_RS["m"],
            "parallelism": f"ep{world}+tp{world}",
            "l2": "256 MB buffer rewritten before every timed call",
            "scaling_note": "all three problems are fixed in total and sharded N-way (strong)",
        },
        "clocks": clocks,
        "e2e": {
            "value": round(geomean(list(mean_e2e.values())), 3),
            "unit": "us",
            "per_op_us": {n: round(v, 3) for n, v in mean_e2e.items()},
            "per_op_median_us": {n: round(median(v), 3) for n, v in e2e_calls.items()},
            "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h,
            "note": "per-step activations (x, indices, weights; gemm_rs input; ag_gemm local rows) start in pinned host "
                    "memory and the full output ends there, every copy inside the events; weights and bias are "
                    "resident.  ours: the GEMM ops go through run_from_host (four row chunks, copies on two side "
                    "streams overlapping the fused kernel); reference: copy in, custom_kernel, copy out",
        },
        "gpu_launches": launches,
        "wall_s_timed_region": round(wall, 4),
    }
    if failed:
        result["error"] = "; ".join(errors) if errors else f"device status {status_word} or a failed check on another rank"
    if rank == 0:
        print(json.dumps(result))
    torch.cuda.synchronize()
    arm.close()
    dist.destroy_process_group()
    return 1 if failed and args.impl == "ours" else 0  # the reference arm reports its checks but always ends normally


if __name__ == "__main__":
    sys.exit(run(parse_args()))
