"""Softmax top-k MoE with a sigmoid-gated shared expert, on fp32 logits (ties to the lower id); each row routes and runs on
its own.  Host-side mirror of the reference module ``tensorfold.cuda.moe`` (cuda/moe.py:41-185)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib
from . import experts as grouped
from .kernels import qmm


def router(x: torch.Tensor, rows: torch.Tensor, out: torch.Tensor | None = None, *, prefill: bool = False) -> torch.Tensor:
    """x [R, D] bf16, rows [E + 1, D] bf16 (router rows, then the shared expert's gate row) -> [R, E + 1] fp32.
    ``prefill`` takes the tensor-core tiles (other bits than the decode form; each form is stable over row counts)."""

    if x.dtype != torch.bfloat16 or rows.dtype != torch.bfloat16 or x.dim() != 2 or rows.dim() != 2 or x.shape[1] != rows.shape[1]:
        raise ValueError("router: x [R, D] and rows [E + 1, D] must be bf16 with the same D")
    if x.stride(1) != 1:
        x = x.contiguous()
    rows = rows.contiguous()
    m, d = x.shape
    ne = rows.shape[0]
    if out is None:
        out = torch.empty((m, ne), dtype=torch.float32, device=x.device)
    stream = _lib.stream_of(x)
    fn = _lib.lib().tf_moe_router_tiles if prefill else _lib.lib().tf_moe_router
    _lib.check(fn(x.data_ptr(), x.stride(0), m, d, rows.data_ptr(), ne, out.data_ptr(), out.stride(0), stream), "router")
    return out


class MoEBuffers:
    """Static scratch for up to ``rows`` rows (CUDA-graph safe); ``prefill`` picks the experts' prefill arithmetic."""

    def __init__(self, rows: int, cfg, device: torch.device | str, *, prefill: bool = False, table_experts: int | None = None) -> None:
        slots = cfg.num_experts_per_tok + 1
        self.rows, self.slots = rows, slots
        self.logits = torch.empty((rows, cfg.num_experts + 1), dtype=torch.float32, device=device)
        self.pick = torch.empty((rows, slots), dtype=torch.int32, device=device)
        self.wts = torch.empty((rows, slots), dtype=torch.float32, device=device)
        experts = cfg.num_experts + 1 if table_experts is None else table_experts
        self.plan = grouped.Plan(rows, slots, experts, device, prefill=prefill)
        self.act = torch.empty((rows, slots, cfg.moe_intermediate_size), dtype=torch.bfloat16, device=device)
        self.y = torch.empty((rows, slots, cfg.hidden_size), dtype=torch.bfloat16 if prefill else torch.float32,
                             device=device)


def select_rows(logits: torch.Tensor, buf: MoEBuffers, top_k: int, experts: int) -> None:
    """Each row's experts and weights, rows in parallel (buf.pick, buf.wts)."""

    rows = logits.shape[0]
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or logits.shape[1] < experts + 1:
        raise ValueError("select_rows: logits must be (R, E + 1) fp32")
    stream = _lib.stream_of(logits)
    _lib.check(_lib.lib().tf_moe_topk(logits.data_ptr(), logits.stride(0), rows, experts, top_k, 1, buf.pick.data_ptr(),
                                      buf.wts.data_ptr(), stream), "select_rows")


def select_local_rows(logits: torch.Tensor, buf: MoEBuffers, top_k: int, experts: int, first: int, count: int) -> None:
    """``select_rows`` for a rank that holds experts [first, first + count): local ids and weights for those, id -1 and
    weight 0 for every other slot (the shared one too).  logits: (R, >= E) fp32."""

    rows = logits.shape[0]
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or logits.shape[1] < experts:
        raise ValueError("select_local_rows: logits must be (R, E) fp32")
    _lib.check(_lib.lib().tf_moe_topk_local(logits.data_ptr(), logits.stride(0), rows, experts, top_k, 1, first, count,
                                            buf.pick.data_ptr(), buf.wts.data_ptr(), _lib.stream_of(logits)), "select_local_rows")


def select(logits: torch.Tensor, buf: MoEBuffers, top_k: int, experts: int) -> None:
    """Each row's experts and weights (rows in parallel), then the (row, slot) pairs grouped by expert."""

    select_rows(logits, buf, top_k, experts)
    grouped.route(buf.pick[:logits.shape[0]], buf.plan)


@dataclass
class SharedExpert:
    """A shared expert of its own width, run as dense projections: ``up`` is a ``qmm.pack_pair`` weight (gate and up
    interleaved), ``down`` a ``qmm.pack`` weight.  (The reference appends the shared expert to the routed table, which
    needs equal widths: families/qwen3_5_moe/cuda/weights.py:41-45.)"""

    up: qmm.Q4
    down: qmm.Q4
    limit: float = 0.0


def moe(x: torch.Tensor, router_rows: torch.Tensor, ex: grouped.Experts, buf: MoEBuffers, top_k: int,
        experts: int, shared: SharedExpert | None = None) -> MoEBuffers:
    """Route x [R, D] and run its experts into buf.y [R, k + 1, D] (bf16 in prefill); slot k is the shared expert."""

    rows = x.shape[0]

    def routed() -> None:
        router(x, router_rows, buf.logits[:rows], prefill=buf.plan.prefill)
        select(buf.logits[:rows], buf, top_k, experts)
        grouped.gate_up(x, ex, buf.plan, buf.act.view(-1, ex.width), rows)
        grouped.down(buf.act.view(-1, ex.width), ex, buf.plan, buf.y.view(-1, ex.dims), rows)

    def dense() -> None:
        if buf.plan.prefill:                                    # prefill arithmetic for the dense shared expert too
            act = qmm.matmul_act(x, shared.up, act="swiglu", limit=shared.limit, prefill=True)
            qmm.prefill_matmul(act, shared.down, f32=buf.y.dtype == torch.float32, out=buf.y[:rows, top_k])
        else:
            act = qmm.matmul_act(x, shared.up, act="swiglu", limit=shared.limit)
            qmm.matmul(act, shared.down, f32=buf.y.dtype == torch.float32, out=buf.y[:rows, top_k])

    if shared is None:
        routed()
    elif buf.plan.prefill:
        routed()
        dense()
    else:
        # decode: the shared expert reads only x and writes its own slot, so it runs beside the routed path (whose
        # router, top-k and plan are short kernels that leave the memory system idle)
        qmm.fork_join([routed, dense])
    return buf


def combine(y: torch.Tensor, wts: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """y [R, S, D] (fp32, or bf16 in prefill) and wts [R, S] fp32 -> [R, D] bf16; a row's bits never depend on R."""

    rows, slots, dims = y.shape
    if not y.is_contiguous() or wts.dtype != torch.float32 or wts.shape != (rows, slots) or not wts.is_contiguous():
        raise ValueError("combine: y [R, S, D] and wts [R, S] fp32 must be contiguous")
    if out is None:
        out = torch.empty((rows, dims), dtype=torch.bfloat16, device=y.device)
    elif out.shape != (rows, dims) or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("combine: out must be a contiguous [R, D] bf16 tensor")
    stream = _lib.stream_of(y)
    _lib.check(_lib.lib().tf_moe_combine(y.data_ptr(), int(y.dtype == torch.bfloat16), wts.data_ptr(), rows, slots, dims,
                                         out.data_ptr(), stream), "combine")
    return out


@dataclass
class Routed:
    """A layer's router rows [E + 1, D] bf16 (the shared expert's gate row last) and its experts: E + 1 table entries
    (shared expert appended), or E entries plus a dense ``shared`` expert of another width."""

    router: torch.Tensor
    experts: grouped.Experts
    top_k: int
    shared: SharedExpert | None = None

    @property
    def count(self) -> int:
        return self.router.shape[0] - 1


class _Shape:
    def __init__(self, m: Routed) -> None:
        self.num_experts_per_tok, self.num_experts = m.top_k, m.count
        self.moe_intermediate_size, self.hidden_size = m.experts.width, m.experts.dims


_scratch: dict[tuple, MoEBuffers] = {}


def run(x: torch.Tensor, m: Routed, *, prefill: bool = False) -> torch.Tensor:
    """x [R, D] bf16 -> [R, D] bf16: its top-k experts by renormalized softmax weight plus the shared expert."""

    rows = x.shape[0]
    size = 1 << max(4, (rows - 1).bit_length())                 # scratch per power of two, reused by every layer
    key = (size, m.count, m.top_k, m.experts.width, m.experts.dims, prefill, x.device, m.experts.count)
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = MoEBuffers(size, _Shape(m), x.device, prefill=prefill, table_experts=m.experts.count)
    moe(x.contiguous(), m.router, m.experts, buf, m.top_k, m.count, m.shared)
    return combine(buf.y[:rows], buf.wts[:rows])
