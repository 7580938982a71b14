"""MoE dispatch/combine on ``torch.distributed`` collectives: the baseline.

Two variants of the reference's algorithm:

* ``custom_kernel`` -- count exchange, stable sort by destination rank, separate
  data and metadata all-to-alls per direction, fp32 ``scatter_add`` reduction,
  with the preparation work on a side stream (the scheme of the reference's root
  ``submission.py:37-219``: six collectives and four host syncs per call);
* ``custom_kernel_packed`` -- metadata travels inside the token rows, one
  all-to-all per direction (the scheme of ``all2all/submission_baseline.py:13-185``);
  the integers are bit-cast into extra columns rather than converted to the
  float type, so ids above 2048 survive fp16.

``custom_kernel_timed`` is the first variant with every step timed as a named phase
(the reference's ``all2all/submission_timed.py``).  All run on any backend/device
(NCCL on GPUs, gloo on CPU).
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist

from ..ops.dispatch_combine import expert_scale_vector
from ..utils.timing import PhaseTimer, format_summary

META = 3  # src_token, src_k, global_expert


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _a2a(out, inp, out_splits=None, in_splits=None):
    if _world() > 1:
        dist.all_to_all_single(out, inp, out_splits, in_splits)
    else:
        out.copy_(inp)


class _SideStream:
    """Runs a block on a side CUDA stream ordered after the current one; no-op on CPU."""

    def __init__(self, device):
        self.stream = torch.cuda.Stream(device) if device.type == "cuda" else None

    @contextlib.contextmanager
    def __call__(self):
        if self.stream is None:
            yield
            return
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            yield
        torch.cuda.current_stream().wait_stream(self.stream)


def _route(indices, El, world):
    flat_e = indices.reshape(-1).long()
    dst = flat_e // El
    counts = torch.bincount(dst, minlength=world)
    order = torch.argsort(dst, stable=True)
    return flat_e, counts, order


def _run(data, tm: PhaseTimer):
    cfg, rd, rank, world = data
    dev = rd.x.device
    T, k, H = rd.num_tokens, cfg.experts_per_token, cfg.hidden_dim
    El = cfg.num_experts // world
    side = _SideStream(dev)

    with tm("dispatch_total"):
        with tm("dispatch_count_calculation"):
            flat_e, send_counts, order = _route(rd.indices, El, world)
            recv_counts = torch.empty_like(send_counts)
        with tm("dispatch_count_exchange"):
            _a2a(recv_counts, send_counts)                               # collective 1
        with tm("dispatch_data_preparation"), side():
            tok = torch.arange(T, device=dev).repeat_interleave(k)
            kk = torch.arange(k, device=dev).repeat(T)
            meta = torch.stack([tok, kk, flat_e], dim=1).to(torch.int32)[order].contiguous()
            send_x = rd.x[tok][order].contiguous()
        with tm("dispatch_preparation"):
            rc, sc = recv_counts.tolist(), send_counts.tolist()          # host sync
            recv_x = torch.empty((sum(rc), H), dtype=cfg.in_dtype, device=dev)
            recv_meta = torch.empty((sum(rc), META), dtype=torch.int32, device=dev)
        with tm("dispatch_data_communication"):
            _a2a(recv_x, send_x, rc, sc)                                 # collective 2
        with tm("dispatch_meta_communication"):
            _a2a(recv_meta.view(-1), meta.view(-1), [c * META for c in rc], [c * META for c in sc])  # collective 3

    with tm("expert_computation"):
        scale = expert_scale_vector(cfg.num_experts, world, cfg.expert_scale, dev)[recv_meta[:, 2].long()].unsqueeze(1)
        y = (recv_x.float() * scale).to(cfg.out_dtype)

    # Combine: rows go back in the order they came, so the split sizes are the
    # dispatch's swapped; the reference re-derives them with a second count
    # exchange (collective 4), which is kept here to preserve its cost profile.
    with tm("combine_total"):
        with tm("combine_count_exchange"):
            back_counts = torch.empty_like(recv_counts)
            _a2a(back_counts, recv_counts)                               # collective 4
        with tm("combine_preparation"):
            bc = back_counts.tolist()                                    # host sync
            back = torch.empty((sum(bc), H), dtype=cfg.out_dtype, device=dev)
            back_meta = torch.empty((sum(bc), META), dtype=torch.int32, device=dev)
        with tm("combine_data_communication"):
            _a2a(back, y, bc, rc)                                        # collective 5
        with tm("combine_meta_communication"):
            _a2a(back_meta.view(-1), recv_meta.view(-1), [c * META for c in bc], [c * META for c in rc])  # collective 6
        with tm("combine_aggregation"):
            src_tok = back_meta[:, 0].long()
            w = rd.weights[src_tok, back_meta[:, 1].long()].unsqueeze(1)
            out = torch.zeros((cfg.max_num_tokens, H), dtype=torch.float32, device=dev)
            out.scatter_add_(0, src_tok.unsqueeze(1).expand(-1, H), back.float() * w)
            res = out.to(cfg.out_dtype)[:T]
    return res


_OFF = PhaseTimer(enabled=False)
_timers: dict = {}  # device -> PhaseTimer of custom_kernel_timed


def custom_kernel(data):
    return _run(data, _OFF)


def custom_kernel_timed(data):
    """``custom_kernel`` with every step bracketed by a named phase (the phases of
    the reference's ``all2all/submission_timed.py:46-222``).  The numbers
    accumulate per device across calls; read them with ``timing_summary()``."""
    dev = data[1].x.device
    tm = _timers.get(dev)
    if tm is None:
        tm = _timers[dev] = PhaseTimer(dev)
    return _run(data, tm)


def timing_summary(device=None, reset: bool = False, rank: int = 0, echo: bool = False) -> dict:
    """Per-phase statistics (ms) gathered by ``custom_kernel_timed`` on ``device``
    (the only one in use if omitted); ``echo`` prints the formatted table."""
    if not _timers:
        return {}
    tm = _timers[torch.device(device)] if device is not None else next(iter(_timers.values()))
    s = tm.summary()
    if echo:
        print(format_summary(tm, rank), flush=True)
    if reset:
        tm.reset()
    return s


def custom_kernel_packed(data):
    cfg, rd, rank, world = data
    dev = rd.x.device
    T, k, H = rd.num_tokens, cfg.experts_per_token, cfg.hidden_dim
    El = cfg.num_experts // world
    esize = rd.x.element_size()
    extra = META * 4 // esize  # columns that hold META int32 values bit for bit

    flat_e, send_counts, order = _route(rd.indices, El, world)
    recv_counts = torch.empty_like(send_counts)
    _a2a(recv_counts, send_counts)
    tok = torch.arange(T, device=dev).repeat_interleave(k)
    kk = torch.arange(k, device=dev).repeat(T)
    meta = torch.stack([tok, kk, flat_e], dim=1).to(torch.int32)[order].contiguous()
    packed = torch.empty((T * k, H + extra), dtype=cfg.in_dtype, device=dev)
    packed[:, :H] = rd.x[tok][order]
    packed[:, H:] = meta.view(cfg.in_dtype)
    rc, sc = recv_counts.tolist(), send_counts.tolist()
    recv = torch.empty((sum(rc), H + extra), dtype=cfg.in_dtype, device=dev)
    _a2a(recv, packed, rc, sc)

    recv_meta = recv[:, H:].contiguous().view(torch.int32)
    scale = expert_scale_vector(cfg.num_experts, world, cfg.expert_scale, dev)[recv_meta[:, 2].long()].unsqueeze(1)
    recv[:, :H] = (recv[:, :H].float() * scale).to(cfg.out_dtype)
    back = torch.empty((sum(sc), H + extra), dtype=cfg.out_dtype, device=dev)
    _a2a(back, recv, sc, rc)

    back_meta = back[:, H:].contiguous().view(torch.int32)
    src_tok = back_meta[:, 0].long()
    w = rd.weights[src_tok, back_meta[:, 1].long()].unsqueeze(1)
    out = torch.zeros((cfg.max_num_tokens, H), dtype=torch.float32, device=dev)
    out.index_add_(0, src_tok, back[:, :H].float() * w)
    return out.to(cfg.out_dtype)[:T]
