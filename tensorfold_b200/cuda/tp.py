"""Tensor- and expert-parallel layers over the GPUs of one NVLink/NVSwitch box (1, 2, 4 or 8 ranks, one process each).

Column-parallel projections own whole output rows, row-parallel ones whole quantization groups of the inputs
(families/qwen3_5/cuda/distributed.py of the reference, two ranks there); every partial sum is reduced in rank order
((p0 + p1) + p2 ...) in fp32 and rounded once, so all ranks hold the same bits and a row's bits do not depend on the row
count.  The routed MoE block is expert-parallel without an all-to-all: activations are replicated, every rank routes all
rows, keeps the pairs whose expert it owns, and contributes a partial [M, D] (the reference splits every expert's width
across its two ranks instead, families/nemotron_h/cuda/tp.py:38-51)."""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist

from . import experts as grouped
from . import moe
from .kernels import qmm
from ..families.qwen3_5.cuda import distributed
from ..families.qwen3_5.cuda.weights import QLinear

GATHER_LIMIT = 1 << 20          # partials up to this many bytes take one all-gather; larger ones exchange shares first


def ordered_all_reduce(local: torch.Tensor, group=None, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Sum of every rank's ``local`` [M, N] (fp32 or bf16) in rank order, fp32 adds, one rounding to ``dtype``.

    Small partials: one all-gather, then each rank adds all of them.  Large ones: every rank receives one share of each
    partial (all-to-all), adds its shares in rank order, and the finished shares are all-gathered: the bytes of a ring
    all-reduce with a fixed summation order.  Both give the same bits."""

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local.to(dtype)
    local = local.contiguous()
    total = local.numel()
    if total * local.element_size() <= GATHER_LIMIT or total % world:
        return distributed.gather_rank_partials(local, group, dtype)
    share = total // world
    recv = torch.empty((world, share), dtype=local.dtype, device=local.device)
    dist.all_to_all_single(recv.view(-1), local.view(-1), group=group)
    mine = distributed._ordered_sum(recv, dtype)
    out = torch.empty((total,), dtype=dtype, device=local.device)
    dist.all_gather_into_tensor(out, mine.view(-1), group=group)
    return out.view(local.shape)


def shard_experts(raw_up: list[tuple], raw_down: tuple, rank: int, world: int) -> tuple[list[tuple], tuple, int]:
    """Rank's share of the expert tables: experts [rank * E / world, (rank + 1) * E / world)."""

    e = raw_down[0].shape[0]
    if e % world:
        raise ValueError("experts must divide across the ranks")
    a, b = rank * e // world, (rank + 1) * e // world
    cut = lambda m: tuple(t[a:b] for t in m)
    return [cut(m) for m in raw_up], cut(raw_down), a


@dataclass
class ExpertParallelMoE:
    """One rank's share of a routed layer: the full router, the local experts and their first global id."""

    router: torch.Tensor            # [E (+1), D] bf16: every rank routes every row
    experts: grouped.Experts        # local experts only
    top_k: int
    first: int                      # global id of local expert 0
    total: int                      # experts in the whole layer
    has_shared_row: bool = False    # router carries a shared-expert gate row (slot k), run elsewhere

    def buffers(self, rows: int, device, *, prefill: bool = False) -> moe.MoEBuffers:
        class _Cfg:
            num_experts_per_tok, num_experts = self.top_k, self.total
            moe_intermediate_size, hidden_size = self.experts.width, self.experts.dims
        return moe.MoEBuffers(rows, _Cfg, device, prefill=prefill, table_experts=self.experts.count)

    def partial(self, x: torch.Tensor, buf: moe.MoEBuffers) -> torch.Tensor:
        """This rank's contribution [R, D] bf16: its experts' slots combined, the others weighted zero."""

        rows = x.shape[0]
        logits = buf.logits[:rows]
        form = buf.plan.prefill                                # prompt passes take the tensor-core router, as moe.moe does
        if self.has_shared_row:
            moe.router(x, self.router, logits, prefill=form)
        else:
            moe.router(x, self.router, logits[:, :self.total], prefill=form)
            logits[:, self.total].zero_()
        moe.select_rows(logits, buf, self.top_k, self.total)
        pick, wts = buf.pick[:rows], buf.wts[:rows]
        pick -= self.first                                                   # local ids; others fall outside the table
        local = (pick >= 0) & (pick < self.experts.count)
        wts.mul_(local)
        grouped.route(pick, buf.plan)
        grouped.gate_up(x, self.experts, buf.plan, buf.act.view(-1, self.experts.width), rows)
        grouped.down(buf.act.view(-1, self.experts.width), self.experts, buf.plan, buf.y.view(-1, self.experts.dims), rows)
        return moe.combine(buf.y[:rows], wts)

    def run(self, x: torch.Tensor, buf: moe.MoEBuffers, group=None) -> torch.Tensor:
        return ordered_all_reduce(self.partial(x, buf), group)


@dataclass
class RowParallelLinear:
    """A projection whose inputs are split across ranks in whole groups; ``forward`` reduces the partials."""

    q: qmm.Q4

    @staticmethod
    def shard(q: QLinear, rank: int, world: int) -> "RowParallelLinear":
        part = distributed.split_input(q, rank, world)
        return RowParallelLinear(qmm.pack(part.weight, part.scales, part.biases, part.gs, bits=part.bits))

    def partial(self, x_local: torch.Tensor, *, f32: bool = False) -> torch.Tensor:
        return qmm.matmul(x_local, self.q, f32=f32)

    def forward(self, x_local: torch.Tensor, group=None, *, f32: bool = False) -> torch.Tensor:
        return ordered_all_reduce(self.partial(x_local, f32=f32), group)


@dataclass
class ColumnParallelLinear:
    """A projection whose output rows are split across ranks; no reduction."""

    q: qmm.Q4

    @staticmethod
    def shard(q: QLinear, rank: int, world: int, segments=None, block: int = 1) -> "ColumnParallelLinear":
        part = distributed.split_output(q, rank, world, segments, block)
        return ColumnParallelLinear(qmm.pack(part.weight, part.scales, part.biases, part.gs, bits=part.bits))

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        return qmm.matmul(x, self.q, **kw)
