"""Oracle of the MoE all-to-all task: inputs, reference result, checker.

Same contract as the reference's ``reference.py`` -- ``MoEConfig`` (``:10-17``),
``RankTestData`` (``:21-51``), ``generate_input`` (``:237-253``), ``ref_kernel``
(``:256-272``), ``check_implementation`` (``:275-283``) -- but the device and the
process-group backend are parameters (CPU + gloo works), the oracle is
vectorised (no per-row ``.item()`` loops), and the data distribution is
selectable:

* ``compat`` options reproduce the reference semantics: fp16, a random token
  count in ``[1, max_num_tokens)``, uniform weights, expert = ``x * (1 + rank)``.
* the benchmark options give a fixed token count, softmax weights and a
  per-expert scale ``(expert_id + 1) / num_experts``.

Oracles: ``ref_kernel`` (collective, vectorised), ``ref_kernel_two_step`` (through the
``PyTorchAllToAll`` dispatch/combine class with the reference's expert-major
buffers), ``ref_kernel_loop`` (collective, the reference's row-by-row algorithm,
for tiny cases) and ``ref_closed_form`` (no communication at all).
"""
from __future__ import annotations

import dataclasses
from typing import Optional

import torch
import torch.distributed as dist

from ...ops.dispatch_combine import SCALE_EXPERT, SCALE_IDENTITY, SCALE_RANK, expert_scale_vector
from .task import input_t, output_t

_DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32,
           "float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}
_SCALES = {"identity": SCALE_IDENTITY, "rank": SCALE_RANK, "expert": SCALE_EXPERT}

RTOL, ATOL = 1e-2, 5e-3  # reference.py:279


@dataclasses.dataclass
class MoEConfig:
    num_experts: int
    experts_per_token: int
    hidden_dim: int
    max_num_tokens: int
    in_dtype: torch.dtype = torch.float16
    out_dtype: torch.dtype = torch.float16
    expert_scale: int = SCALE_RANK


def default_device(rank: int) -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", rank % torch.cuda.device_count())
    return torch.device("cpu")


class RankTestData:
    """Tokens, routing table and routing weights of one data-parallel rank."""

    def __init__(self, cfg: MoEConfig, rng: torch.Generator, rank: int, device: Optional[torch.device] = None,
                 fixed_tokens: bool = False, weight_mode: str = "uniform"):
        device = torch.device(device) if device is not None else default_device(rank)
        if fixed_tokens or cfg.max_num_tokens <= 1:
            self.num_tokens = cfg.max_num_tokens
        else:
            self.num_tokens = int(torch.randint(1, cfg.max_num_tokens, [1], generator=rng, device=device).item())
        T, E, k = self.num_tokens, cfg.num_experts, cfg.experts_per_token
        # k distinct experts per token, uniform without replacement: rank random keys.
        keys = torch.rand(T, E, generator=rng, device=device)
        self.indices = keys.argsort(dim=1)[:, :k].to(torch.int32).contiguous()
        if weight_mode == "uniform":
            self.weights = torch.rand(T, k, dtype=torch.float32, generator=rng, device=device)
        elif weight_mode == "softmax":
            self.weights = torch.softmax(torch.randn(T, k, dtype=torch.float32, generator=rng, device=device), dim=-1)
        else:
            raise ValueError(f"unknown weight_mode {weight_mode!r}")
        self.x = torch.randn(T, cfg.hidden_dim, dtype=torch.float32, generator=rng, device=device).to(cfg.in_dtype)


def generate_input(num_experts: int, experts_per_token: int, hidden_dim: int, max_num_tokens: int, seed: int,
                   rank: int, world_size: int, dtype: str = "fp16", fixed_tokens: bool = False,
                   weight_mode: str = "uniform", expert_scale: str = "rank", device=None) -> input_t:
    dev = torch.device(device) if device is not None else default_device(rank)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed + rank)
    dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
    cfg = MoEConfig(num_experts, experts_per_token, hidden_dim, max_num_tokens, in_dtype=dt, out_dtype=dt,
                    expert_scale=_SCALES[expert_scale] if isinstance(expert_scale, str) else int(expert_scale))
    rank_data = RankTestData(cfg, gen, rank, device=dev, fixed_tokens=bool(fixed_tokens), weight_mode=weight_mode)
    return cfg, rank_data, rank, world_size


def _a2a(out: torch.Tensor, inp: torch.Tensor, out_splits, in_splits) -> None:
    if dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_to_all_single(out, inp, out_splits, in_splits)
    else:
        out.copy_(inp)


def ref_kernel(data: input_t) -> output_t:
    """Vectorised collective oracle: group by destination rank, exchange, scale by
    the owning expert, send back, weighted sum in fp32 over k."""
    cfg, rd, rank, world = data
    dev = rd.x.device
    T, k, H = rd.num_tokens, cfg.experts_per_token, cfg.hidden_dim
    El = cfg.num_experts // world
    flat_e = rd.indices.reshape(-1).long()
    dst = flat_e // El
    order = torch.argsort(dst, stable=True)
    send_counts = torch.bincount(dst, minlength=world)
    tok = torch.arange(T, device=dev).repeat_interleave(k)
    send_x = rd.x[tok][order].contiguous()
    send_e = flat_e[order].contiguous()
    recv_counts = torch.empty_like(send_counts)
    _a2a(recv_counts, send_counts, None, None)
    rc, sc = recv_counts.tolist(), send_counts.tolist()
    recv_x = torch.empty((sum(rc), H), dtype=cfg.in_dtype, device=dev)
    recv_e = torch.empty(sum(rc), dtype=torch.long, device=dev)
    _a2a(recv_x, send_x, rc, sc)
    _a2a(recv_e, send_e, rc, sc)
    scale = expert_scale_vector(cfg.num_experts, world, cfg.expert_scale, dev)[recv_e].unsqueeze(1)
    y = (recv_x.float() * scale).to(cfg.out_dtype)
    back = torch.empty((sum(sc), H), dtype=cfg.out_dtype, device=dev)
    _a2a(back, y, sc, rc)
    contrib = torch.empty_like(back)
    contrib[order] = back
    out = (contrib.float() * rd.weights.reshape(-1, 1)).view(T, k, H).sum(1)
    return out.to(cfg.out_dtype)


class PyTorchAllToAll:
    """Dispatch and combine as two collective steps with the reference's
    interface (``PyTorchAllToAll``, reference.py:54-234): ``dispatch`` returns the
    expert-major padded buffers ``(expert_num_tokens [E_local], expert_x [E_local,
    max_recv, H], expert_meta [E_local, max_recv, META_DIM])`` and ``combine``
    accumulates ``weights[token, k] * expert_y`` into ``out_tokens``.  Vectorised
    (no per-row host round trips) and device/backend agnostic."""

    META_DIM = 5  # global expert, source rank, source token, source k, pad

    def __init__(self, cfg: MoEConfig, rank: int, world_size: int):
        self.cfg, self.rank, self.world_size = cfg, rank, world_size
        self.num_local_experts = cfg.num_experts // world_size
        self.max_recv = cfg.max_num_tokens * world_size

    def dispatch(self, dp_x: torch.Tensor, indices: torch.Tensor):
        cfg, dev = self.cfg, dp_x.device
        T, k = indices.shape
        El, world = self.num_local_experts, self.world_size
        flat_e = indices.reshape(-1).long()
        dst = flat_e // El
        order = torch.argsort(dst, stable=True)
        send_counts = torch.bincount(dst, minlength=world)
        tok = torch.arange(T, device=dev).repeat_interleave(k)
        kk = torch.arange(k, device=dev).repeat(T)
        meta = torch.stack([flat_e, torch.full_like(flat_e, self.rank), tok, kk, torch.zeros_like(flat_e)], dim=1)
        send_x = dp_x[tok][order].contiguous()
        send_m = meta[order].contiguous()
        recv_counts = torch.empty_like(send_counts)
        _a2a(recv_counts, send_counts, None, None)
        rc, sc = recv_counts.tolist(), send_counts.tolist()
        recv_x = torch.empty((sum(rc), cfg.hidden_dim), dtype=cfg.in_dtype, device=dev)
        recv_m = torch.empty((sum(rc), self.META_DIM), dtype=torch.long, device=dev)
        _a2a(recv_x, send_x, rc, sc)
        _a2a(recv_m.view(-1), send_m.view(-1), [c * self.META_DIM for c in rc], [c * self.META_DIM for c in sc])
        # expert-major placement: position of a row inside its expert = its rank among the
        # rows of that expert in arrival order
        local_e = recv_m[:, 0] % El
        by_expert = torch.argsort(local_e, stable=True)
        expert_num_tokens = torch.bincount(local_e, minlength=El).to(torch.int32)
        starts = torch.cumsum(expert_num_tokens.long(), 0) - expert_num_tokens.long()
        pos = torch.arange(local_e.numel(), device=dev) - starts[local_e[by_expert]]
        expert_x = torch.zeros((El, self.max_recv, cfg.hidden_dim), dtype=cfg.in_dtype, device=dev)
        expert_meta = torch.zeros((El, self.max_recv, self.META_DIM), dtype=torch.int32, device=dev)
        expert_x[local_e[by_expert], pos] = recv_x[by_expert]
        expert_meta[local_e[by_expert], pos] = recv_m[by_expert].to(torch.int32)
        return expert_num_tokens, expert_x, expert_meta

    def combine(self, out_tokens: torch.Tensor, weights: torch.Tensor, expert_meta: torch.Tensor, expert_y: torch.Tensor,
                expert_num_tokens: torch.Tensor) -> torch.Tensor:
        cfg, dev = self.cfg, out_tokens.device
        El, world = self.num_local_experts, self.world_size
        valid = torch.arange(self.max_recv, device=dev).unsqueeze(0) < expert_num_tokens.long().unsqueeze(1)  # [El, max_recv]
        rows = expert_y[valid]                    # expert-major order
        meta = expert_meta[valid].long()
        dst = meta[:, 1]
        order = torch.argsort(dst, stable=True)
        send_counts = torch.bincount(dst, minlength=world)
        recv_counts = torch.empty_like(send_counts)
        _a2a(recv_counts, send_counts, None, None)
        rc, sc = recv_counts.tolist(), send_counts.tolist()
        recv_y = torch.empty((sum(rc), cfg.hidden_dim), dtype=cfg.out_dtype, device=dev)
        recv_m = torch.empty((sum(rc), self.META_DIM), dtype=torch.long, device=dev)
        _a2a(recv_y, rows[order].contiguous(), rc, sc)
        _a2a(recv_m.view(-1), meta[order].contiguous().view(-1), [c * self.META_DIM for c in rc], [c * self.META_DIM for c in sc])
        w = weights[recv_m[:, 2], recv_m[:, 3]].to(torch.float32).unsqueeze(1)
        acc = torch.zeros(out_tokens.shape, dtype=torch.float32, device=dev)
        acc.index_add_(0, recv_m[:, 2], recv_y.float() * w)
        out_tokens += acc.to(out_tokens.dtype)
        return out_tokens


def ref_kernel_two_step(data: input_t) -> output_t:
    """The oracle through ``PyTorchAllToAll.dispatch`` / ``combine`` (the structure of
    the reference's ``ref_kernel``, reference.py:256-272)."""
    cfg, rd, rank, world = data
    ata = PyTorchAllToAll(cfg, rank, world)
    expert_num, expert_x, expert_meta = ata.dispatch(rd.x, rd.indices)
    scale = expert_scale_vector(cfg.num_experts, world, cfg.expert_scale, rd.x.device)
    local = scale[rank * ata.num_local_experts:(rank + 1) * ata.num_local_experts].view(-1, 1, 1)
    expert_y = (expert_x.float() * local).to(cfg.out_dtype)
    y = torch.zeros(cfg.max_num_tokens, cfg.hidden_dim, dtype=cfg.out_dtype, device=rd.x.device)
    ata.combine(y, rd.weights, expert_meta, expert_y, expert_num)
    return y[: rd.num_tokens]


def ref_closed_form(data: input_t) -> output_t:
    """No communication: ``y[t] = sum_k w[t,k] * scale(e[t,k]) * x[t]`` with the
    expert output rounded to ``out_dtype`` as on the wire."""
    cfg, rd, rank, world = data
    sc = expert_scale_vector(cfg.num_experts, world, cfg.expert_scale, rd.x.device)[rd.indices.long()]  # [T,k]
    y = (rd.x.float().unsqueeze(1) * sc.unsqueeze(-1)).to(cfg.out_dtype).float()  # [T,k,H]
    return (y * rd.weights.unsqueeze(-1)).sum(1).to(cfg.out_dtype)


def ref_kernel_loop(data: input_t) -> output_t:
    """Row-by-row oracle with the reference's structure (expert-major receive
    buffers, metadata travelling with the rows, accumulation in ``out_dtype``
    storage in arrival order; reference.py:68-234).  Slow: tiny cases only."""
    cfg, rd, rank, world = data
    dev = rd.x.device
    k, H = cfg.experts_per_token, cfg.hidden_dim
    El = cfg.num_experts // world
    per_dst_rows = [[] for _ in range(world)]
    per_dst_meta = [[] for _ in range(world)]
    for t, experts in enumerate(rd.indices.tolist()):
        for kk, e in enumerate(experts):
            per_dst_rows[e // El].append(t)
            per_dst_meta[e // El].append([e, rank, t, kk])
    sc = [len(r) for r in per_dst_rows]
    send_counts = torch.tensor(sc, dtype=torch.long, device=dev)
    recv_counts = torch.empty_like(send_counts)
    _a2a(recv_counts, send_counts, None, None)
    rc = recv_counts.tolist()
    rows = [t for r in per_dst_rows for t in r]
    send_x = rd.x[rows] if rows else rd.x[:0]
    send_m = torch.tensor([m for r in per_dst_meta for m in r], dtype=torch.int64, device=dev).view(-1, 4)
    recv_x = torch.empty((sum(rc), H), dtype=cfg.in_dtype, device=dev)
    recv_m = torch.empty((sum(rc), 4), dtype=torch.int64, device=dev)
    _a2a(recv_x, send_x.contiguous(), rc, sc)
    _a2a(recv_m.view(-1), send_m.view(-1), [4 * c for c in rc], [4 * c for c in sc])
    # expert-major placement
    max_recv = cfg.max_num_tokens * world
    ex = torch.zeros((El, max_recv, H), dtype=cfg.in_dtype, device=dev)
    em = torch.zeros((El, max_recv, 4), dtype=torch.int64, device=dev)
    cnt = [0] * El
    for i, m in enumerate(recv_m.tolist()):
        le = m[0] % El
        ex[le, cnt[le]] = recv_x[i]
        em[le, cnt[le]] = recv_m[i]
        cnt[le] += 1
    scale = expert_scale_vector(cfg.num_experts, world, cfg.expert_scale, dev)
    back_rows = [[] for _ in range(world)]
    back_meta = [[] for _ in range(world)]
    for le in range(El):
        s = scale[rank * El + le]
        for j in range(cnt[le]):
            m = em[le, j].tolist()
            back_rows[m[1]].append((ex[le, j].float() * s).to(cfg.out_dtype))
            back_meta[m[1]].append(m)
    bc = [len(r) for r in back_rows]
    bcounts = torch.tensor(bc, dtype=torch.long, device=dev)
    rcounts = torch.empty_like(bcounts)
    _a2a(rcounts, bcounts, None, None)
    rb = rcounts.tolist()
    flat_rows = [r for lst in back_rows for r in lst]
    send_y = torch.stack(flat_rows) if flat_rows else torch.empty((0, H), dtype=cfg.out_dtype, device=dev)
    send_bm = torch.tensor([m for lst in back_meta for m in lst], dtype=torch.int64, device=dev).view(-1, 4)
    recv_y = torch.empty((sum(rb), H), dtype=cfg.out_dtype, device=dev)
    recv_bm = torch.empty((sum(rb), 4), dtype=torch.int64, device=dev)
    _a2a(recv_y, send_y.contiguous(), rb, bc)
    _a2a(recv_bm.view(-1), send_bm.view(-1), [4 * c for c in rb], [4 * c for c in bc])
    out = torch.zeros((cfg.max_num_tokens, H), dtype=cfg.out_dtype, device=dev)
    for i, m in enumerate(recv_bm.tolist()):
        out[m[2]] += (recv_y[i].float() * rd.weights[m[2], m[3]]).to(cfg.out_dtype)
    return out[: rd.num_tokens]


def check_implementation(data: input_t, output: output_t):
    """Collective: every rank must call it (the oracle communicates)."""
    expected = ref_kernel(data)
    if output.device != expected.device:
        return False, f"Output device mismatch: {output.device} != {expected.device}"
    if output.shape != expected.shape:
        return False, f"Output shape mismatch: {tuple(output.shape)} != {tuple(expected.shape)}"
    if not torch.allclose(output.float(), expected.float(), rtol=RTOL, atol=ATOL):
        diff = (output.float() - expected.float()).abs()
        return False, f"Output values mismatch: max abs diff {diff.max().item():.5g} at {int(diff.argmax())}"
    return True, ""
