"""Grouped MoE experts on MLX 4-bit weights; a (row, slot) pair's bits never depend on the other rows of the call.

Host-side mirror of the reference module ``tensorfold.cuda.experts`` (cuda/experts.py:11-149).  The expert tables use the
same tiled units as the dense matmul (one table per projection, experts outermost); gate and up are interleaved in
16-row tiles so one pass yields both halves of a SwiGLU output.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import _lib
from .kernels import qmm

NTW = 4                  # n8 tiles a warp
COLS = 8 * NTW           # output columns a warp
TILE = 16                # pairs an item holds (decode form; 8 while experts see few pairs each, see ``decode_tile``)
PREFILL_TILE = 128       # pairs an item holds (prefill form: one tcgen05 tile of 128 rows; the reference's is 64)
SMALL = 1024             # pairs the one-block plan takes; wider plans rank in blocks of 1024 pairs


def _check(words, scales, biases, gs):
    if gs not in (32, 64, 128):
        raise ValueError(f"groups of 32, 64 or 128 inputs, not {gs}")
    e, n, k8 = words.shape
    k = k8 * 8
    if n % 16 or k % gs or scales.shape != (e, n, k // gs) or biases.shape != scales.shape:
        raise ValueError(f"experts: shape {tuple(words.shape)} with scales {tuple(scales.shape)} does not pack")
    if scales.dtype != torch.bfloat16 or biases.dtype != torch.bfloat16:
        raise ValueError("experts: scales and biases must be bf16")
    return e, n, k


def pack(words: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, gs: int) -> torch.Tensor:
    """MLX words [E, N, K/8], scales and biases [E, N, K/gs] -> tiled units [E, ceil(N/128), K/gs, unit]; ``unpack`` inverts."""

    e, n, k = _check(words, scales, biases, gs)
    parts = [qmm.pack(words[i], scales[i], biases[i], gs).weight for i in range(e)]
    return torch.stack(parts)


def pack_pair(gate: tuple, up: tuple, gs: int) -> torch.Tensor:
    """Gate and up (each words [E, N, K/8], scales, biases) interleaved in 16-row tiles: [E, ceil(2N/128), K/gs, unit]."""

    e, n, k = _check(*gate, gs)
    if _check(*up, gs) != (e, n, k):
        raise ValueError("experts: gate and up must have the same shapes")
    parts = [qmm.pack_pair(tuple(t[i] for t in gate), tuple(t[i] for t in up), gs).weight for i in range(e)]
    return torch.stack(parts)


def unpack(blocks: torch.Tensor, gs: int, n: int | None = None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``pack``'s inverse: units [E, ceil(N/128), K/gs, unit] -> MLX words [E, N, K/8], scales and biases [E, N, K/gs].
    ``n`` defaults to all 128 columns of every super-block."""

    e, nsb, kg, _ = blocks.shape
    n = nsb * 128 if n is None else n
    outs = [qmm.unpack(qmm.Q4(blocks[i], None, None, n, kg * gs, gs)) for i in range(e)]
    return tuple(torch.stack([o[j] for o in outs]) for j in range(3))


def unpack_pair(blocks: torch.Tensor, gs: int, n_each: int):
    """``pack_pair``'s inverse: ((gate words, scales, biases), (up words, scales, biases)), each [E, n_each, ...]."""

    both = unpack(blocks, gs, 2 * n_each)
    rows = torch.arange(2 * n_each, device=blocks.device)
    gate_rows, up_rows = rows[(rows // 16) % 2 == 0], rows[(rows // 16) % 2 == 1]
    return tuple(t[:, gate_rows].contiguous() for t in both), tuple(t[:, up_rows].contiguous() for t in both)


@dataclass
class Experts:
    """One layer's experts (the shared ones included): gate and up (SwiGLU) or up (relu^2), and down."""

    up: torch.Tensor          # [E, ceil(rows/128), D/gs, unit] int32; rows = 2 NI (gate and up interleaved) or NI
    down: torch.Tensor        # [E, ceil(D/128), NI/gs, unit]
    gs: int
    width: int                # NI: the expert's (or this rank's) intermediate width
    dims: int                 # D
    limit: float = 0.0        # SwiGLU clip (0: none)
    gated: bool = True        # gate and up (SwiGLU) rather than up alone (relu^2)

    @property
    def count(self) -> int:
        return self.up.shape[0]

    @property
    def swiglu(self) -> bool:
        return self.gated

    def bytes_per_expert(self) -> int:
        return (self.up[0].numel() + self.down[0].numel()) * 4


def make(up: list[tuple], down: tuple, gs: int, *, limit: float = 0.0) -> Experts:
    """One layer's MLX arrays: ``up`` [gate, up] (SwiGLU) or [up] (relu^2), ``down``, each (words, scales, biases)."""

    if len(up) not in (1, 2):
        raise ValueError("experts take a gate and an up projection, or an up projection alone")
    width, dims = up[0][0].shape[1], up[0][0].shape[2] * 8
    u = pack_pair(up[0], up[1], gs) if len(up) == 2 else pack(*up[0], gs)
    d = pack(*down, gs)
    return Experts(u, d, gs, width, dims, float(limit), len(up) == 2)


def decode_tile(pairs: int, experts: int) -> int:
    """Pairs a decode item holds: 8 while an expert sees four pairs on average at most (an item then costs one row
    tile of MMAs, and an expert with more than 8 pairs gets a second item), else 16.  A load-time choice from the
    buffers' sizes; a pair's bits do not depend on it."""

    return 8 if pairs <= 4 * experts else TILE


def max_items(pairs: int, experts: int, tile: int = TILE) -> int:
    """Items a plan of ``pairs`` can hold: an item per used expert, plus one per ``tile`` pairs past its first."""

    return min(pairs, experts) + pairs // tile


class Plan:
    """Scratch grouping pairs by expert: members, items (expert, first, count), counts [items, distinct experts]."""

    def __init__(self, rows: int, slots: int, experts: int, device: torch.device | str, *,
                 prefill: bool = False) -> None:
        pairs = rows * slots
        self.rows, self.slots, self.experts, self.prefill = rows, slots, experts, prefill
        self.tile = PREFILL_TILE if prefill else decode_tile(pairs, experts)
        self.members = torch.zeros((pairs,), dtype=torch.int32, device=device)
        self.items = torch.zeros((max_items(pairs, experts, self.tile), 3), dtype=torch.int32, device=device)
        self.counts = torch.zeros((2,), dtype=torch.int32, device=device)
        self.rank = torch.zeros((pairs,), dtype=torch.int32, device=device)
        self.hist = torch.zeros((-(-pairs // SMALL) * experts,), dtype=torch.int32, device=device)
        self.sorted = None       # prefill form: the call's rows in member order (made on first use, before any capture)


def route(picks: torch.Tensor, plan: Plan) -> None:
    """``picks`` [R, slots] int32, contiguous: each (row, slot) pair's expert id (shared experts included).  Ids outside
    [0, plan.experts) belong to no table expert and are left out of the plan."""

    rows, slots = picks.shape
    if slots != plan.slots or rows > plan.rows:
        raise ValueError(f"picks {tuple(picks.shape)} do not fit a plan of {plan.rows} x {plan.slots}")
    if picks.dtype != torch.int32 or not picks.is_contiguous():
        raise ValueError("picks must be contiguous int32")
    stream = _lib.stream_of(picks)
    _lib.check(_lib.lib().tf_moe_plan(picks.data_ptr(), rows * slots, plan.experts, plan.tile, plan.members.data_ptr(),
                                      plan.items.data_ptr(), plan.counts.data_ptr(), plan.rank.data_ptr(),
                                      plan.hist.data_ptr(), plan.items.shape[0], stream), "route")


def _grouped(x, slots, table, n, k, ex, plan, out, rows, epi, limit):
    if plan.experts > table.shape[0]:
        # an item may name any expert below plan.experts: the kernels would read past the table
        raise ValueError(f"the plan routes to {plan.experts} experts but the table holds {table.shape[0]}")
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != k or x.stride(1) != 1:
        raise ValueError(f"experts: inputs must be (rows, {k}) bf16 with unit-stride rows")
    if x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    if out.dim() != 2 or out.stride(1) != 1:
        raise ValueError("experts: out must be 2-D with unit-stride rows")
    stream = _lib.stream_of(x)
    items = min(max_items(rows * plan.slots, plan.experts, plan.tile), plan.items.shape[0])
    if plan.prefill:
        if ex.gs not in (32, 64):
            raise ValueError("prefill plans take expert weights with groups of 32 or 64")
        pairs = plan.members.shape[0]
        if plan.sorted is None or plan.sorted.numel() < pairs * k:
            plan.sorted = torch.empty((pairs * max(k, ex.dims, ex.width),), dtype=torch.bfloat16, device=x.device)
        _lib.check(_lib.lib().tf_moe_experts_prefill(
            x.data_ptr(), x.stride(0), slots, table.data_ptr(), table.stride(0), table.shape[0], n, k, ex.gs, plan.items.data_ptr(),
            plan.counts.data_ptr(), plan.members.data_ptr(), rows * plan.slots, items, plan.sorted.data_ptr(), out.data_ptr(),
            out.stride(0), int(out.dtype == torch.float32), epi, float(limit), stream), "experts (prefill)")
        return
    _lib.check(_lib.lib().tf_moe_experts(
        x.data_ptr(), x.stride(0), slots, table.data_ptr(), table.stride(0), table.shape[0], n, k, ex.gs, plan.items.data_ptr(),
        plan.counts.data_ptr(), plan.members.data_ptr(), items, plan.tile, out.data_ptr(), out.stride(0),
        int(out.dtype == torch.float32), epi, float(limit), stream), "experts")


def gate_up(x: torch.Tensor, ex: Experts, plan: Plan, out: torch.Tensor, rows: int) -> None:
    """x [R, D] bf16 (unit-stride rows) -> out [R * slots, NI] bf16, each pair's activation."""

    if out.dtype != torch.bfloat16 or out.shape[1] != ex.width:
        raise ValueError("gate_up: out must be (pairs, NI) bf16")
    n = 2 * ex.width if ex.swiglu else ex.width
    _grouped(x, plan.slots, ex.up, n, ex.dims, ex, plan, out, rows, 2 if ex.swiglu else 1, ex.limit)


def down(act: torch.Tensor, ex: Experts, plan: Plan, out: torch.Tensor, rows: int) -> None:
    """act [R * slots, NI] bf16 -> out [R * slots, D] per pair: fp32, or bf16 when ``out`` is bf16."""

    if out.dtype not in (torch.float32, torch.bfloat16) or out.shape[1] != ex.dims:
        raise ValueError("down: out must be (pairs, D) fp32 or bf16")
    _grouped(act, 0, ex.down, ex.dims, ex.width, ex, plan, out, rows, 0, 0.0)
