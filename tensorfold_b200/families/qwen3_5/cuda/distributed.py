"""Rank shards keep packed rows and quantization-group boundaries; row-parallel partials are gathered and summed in rank
order so every rank holds the same bits.  Mirrors families/qwen3_5/cuda/distributed.py:27-284 of the reference, whose
two-rank guards are widened to any world size that divides the shapes (1, 2, 4, 8 GPUs of one box)."""

from __future__ import annotations

import os
from typing import Sequence

import torch
import torch.distributed as dist

from .... import _lib
from ....cuda.kernels import affine
from dataclasses import dataclass, replace

from .weights import GDN, Attention, Config, Layer, QLinear, Weights


def _rank(rank: int, world_size: int) -> None:
    if world_size < 1 or not 0 <= rank < world_size:
        raise ValueError("rank outside the world")


def output_rows(n: int, rank: int, world_size: int = 2, segments: Sequence[int] | None = None, block: int = 1,
                device: torch.device | str = "cpu") -> torch.Tensor:
    """Rank-local row indices in segment order, preserving concatenated projections and complete head blocks."""

    _rank(rank, world_size)
    lengths = tuple(segments) if segments is not None else (n,)
    if sum(lengths) != n or any(v <= 0 or v % (world_size * block) for v in lengths):
        raise ValueError(f"output segments {lengths} do not split into {world_size} blocks of {block}")
    base, ranges = 0, []
    for length in lengths:
        share = length // world_size
        ranges.append(torch.arange(base + rank * share, base + (rank + 1) * share, device=device))
        base += length
    return torch.cat(ranges)


def split_output(q: QLinear, rank: int, world_size: int = 2, segments: Sequence[int] | None = None,
                 block: int = 1) -> QLinear:
    """Column-parallel QLinear: each rank owns complete output rows."""

    if q.layout == "tiled":
        raise ValueError("split the checkpoint layout before tiling")
    rows = output_rows(q.n, rank, world_size, segments, block, q.weight.device)
    return QLinear(q.weight.index_select(0, rows).contiguous(),
                   q.scales.index_select(0, rows).contiguous() if q.scales is not None else None,
                   q.biases.index_select(0, rows).contiguous() if q.biases is not None else None,
                   layout=q.layout, gs=q.gs, bits=q.bits)


def split_input(q: QLinear, rank: int, world_size: int = 2) -> QLinear:
    """Row-parallel QLinear: each rank owns complete quantization groups and packed words."""

    _rank(rank, world_size)
    if q.layout != "mlx":
        raise ValueError("split the checkpoint layout before tiling")
    (w0, w1), (g0, g1) = affine.input_slice(q.k, q.bits, q.gs, rank, world_size)
    return QLinear(q.weight[:, w0:w1].contiguous(), q.scales[:, g0:g1].contiguous(), q.biases[:, g0:g1].contiguous(),
                   gs=q.gs, bits=q.bits)


def local_input(x: torch.Tensor, rank: int, world_size: int = 2, *, group_size: int = 64) -> torch.Tensor:
    """Select the activation columns corresponding to ``split_input``."""

    _rank(rank, world_size)
    if group_size not in (1, 32, 64, 128) or x.ndim != 2 or x.shape[1] % (group_size * world_size):
        raise ValueError("activation input must be 2-D and group-aligned")
    share = x.shape[1] // world_size
    return x[:, rank * share:(rank + 1) * share].contiguous()


def row_partial(x: torch.Tensor, q: QLinear, sk: int | None = None, xs: torch.Tensor | None = None) -> torch.Tensor:
    """Row-parallel projection, returning an fp32 (rows, outputs) partial."""

    from . import qmm_fast

    if sk is not None and q.layout == "tiled":
        raise ValueError("tiled row partials use the shape's own split")
    return qmm_fast.matmul_partial(x, q, xs)


def sum_rank_partials(partials: Sequence[torch.Tensor], dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Rank-ordered sum ((p0 + p1) + p2) + ... in fp32, one rounding.  On a CUDA device this is one kernel; CPU tensors
    (the gloo tests of the host logic) are added with torch."""

    if len(partials) < 1 or any(p.dtype not in (torch.float32, torch.bfloat16) or p.shape != partials[0].shape for p in partials):
        raise ValueError("expected equally shaped fp32 or bf16 partials in rank order")
    return _ordered_sum(torch.stack([p.contiguous() for p in partials]), dtype)


def _ordered_sum(stacked: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    world = stacked.shape[0]
    if not stacked.is_cuda:
        total = stacked[0].float()
        for r in range(1, world):
            total = total + stacked[r].float()
        return total.to(dtype)
    stream = _lib.stream_of(stacked)
    out = torch.empty(stacked.shape[1:], dtype=dtype, device=stacked.device)
    _lib.check(_lib.lib().tf_sum_ranks(stacked.data_ptr(), world, out.numel(), int(stacked.dtype == torch.bfloat16),
                                       out.data_ptr(), int(dtype == torch.float32), stream), "sum_rank_partials")
    return out


def gather_rank_partials(local: torch.Tensor, group=None, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Add every rank's partial, rank 0 first, in fp32 and round once; an all-reduce leaves the order to NCCL
    (``TF_TP_REDUCE=allreduce``)."""

    if not dist.is_initialized():
        raise RuntimeError("a process group must be initialized")
    if local.dtype not in (torch.float32, torch.bfloat16) or local.ndim != 2:
        raise ValueError("local partial must be a 2-D fp32 or bf16 tensor")
    if dist.get_backend(group) == "nccl" and not local.is_cuda:
        raise ValueError("NCCL partial must be on CUDA")
    world = dist.get_world_size(group)
    local = local.contiguous()
    if world == 1:
        return local.to(dtype)
    if os.environ.get("TF_TP_REDUCE") == "allreduce":
        local = local.clone()
        dist.all_reduce(local, op=dist.ReduceOp.SUM, group=group)
        return local.to(dtype)
    gathered = torch.empty((world, *local.shape), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(gathered.view(-1), local.view(-1), group=group)
    return _ordered_sum(gathered, dtype)


@dataclass
class LayerShard:
    """One rank's share of a layer and the head counts it holds (families/qwen3_5/cuda/distributed.py:90-99)."""

    layer: Layer
    rank: int
    world_size: int
    q_heads: int
    kv_heads: int
    k_heads: int
    v_heads: int


def split_layer(layer: Layer, cfg: Config, rank: int, world_size: int = 2) -> LayerShard:
    """One rank's share of a layer, cut along heads and the MLP width without touching a checkpoint word
    (families/qwen3_5/cuda/distributed.py:101-133): q/k/v, gate/up and the GDN inputs by whole output rows (whole
    heads), o, down and the GDN output by whole groups of inputs; the per-head GDN tensors follow their heads."""

    _rank(rank, world_size)
    counts = [cfg.intermediate] + ([cfg.heads, cfg.kv_heads] if layer.attn is not None else []) + \
             ([cfg.k_heads, cfg.v_heads] if layer.gdn is not None else [])
    if any(v % world_size for v in counts):
        raise ValueError("head count and MLP width must be divisible by rank count")
    attn = None
    if layer.attn is not None:
        a = layer.attn
        attn = Attention(q=split_output(a.q, rank, world_size, block=2 * cfg.head_dim),
                         k=split_output(a.k, rank, world_size, block=cfg.head_dim),
                         v=split_output(a.v, rank, world_size, block=cfg.head_dim),
                         o=split_input(a.o, rank, world_size), q_norm=a.q_norm, k_norm=a.k_norm)
    gdn = None
    if layer.gdn is not None:
        g = layer.gdn
        kd, vd = cfg.k_heads * cfg.dk, cfg.v_heads * cfg.dv
        rows = output_rows(g.qkv.n, rank, world_size, segments=(kd, kd, vd), device=g.conv.device)
        vh = cfg.v_heads // world_size
        lo, hi = rank * vh, (rank + 1) * vh
        gdn = GDN(qkv=split_output(g.qkv, rank, world_size, segments=(kd, kd, vd)),
                  z=split_output(g.z, rank, world_size, block=cfg.dv),
                  b=split_output(g.b, rank, world_size), a=split_output(g.a, rank, world_size),
                  out=split_input(g.out, rank, world_size),
                  conv=g.conv.index_select(0, rows).contiguous(),
                  A_log=g.A_log[lo:hi].contiguous(), dt_bias=g.dt_bias[lo:hi].contiguous(), norm=g.norm)
    cut = lambda q, fn: fn(q, rank, world_size) if q is not None else None
    local = Layer(linear=layer.linear, input_norm=layer.input_norm, post_norm=layer.post_norm, gdn=gdn, attn=attn,
                  gate=cut(layer.gate, split_output), up=cut(layer.up, split_output), down=cut(layer.down, split_input),
                  moe=layer.moe)
    return LayerShard(local, rank, world_size, cfg.heads // world_size, cfg.kv_heads // world_size,
                      cfg.k_heads // world_size, cfg.v_heads // world_size)


def split_weights(w: Weights, rank: int, world_size: int = 2, *, tiled: bool = False, fuse: bool = False,
                  split_head: bool = False) -> Weights:
    """One rank's share of a model's projections, cut in the stored layout and only then (optionally) tiled
    (families/qwen3_5/cuda/distributed.py:136-165); ``split_head`` also cuts the head's vocabulary rows (every rank then
    holds whole dot products of its rows, so logits keep their bits and candidates can be merged)."""

    _rank(rank, world_size)
    c = w.config
    local_cfg = replace(c, heads=c.heads // world_size, kv_heads=c.kv_heads // world_size, k_heads=c.k_heads // world_size,
                        v_heads=c.v_heads // world_size, intermediate=c.intermediate // world_size)
    layers = []
    for layer in w.layers:
        local = split_layer(layer, c, rank, world_size).layer
        if tiled:
            from .qmm_fast import stack_small, tile_layer

            if fuse:
                stack_small(local)
            tile_layer(local)
        layers.append(local)
    head = split_output(w.head, rank, world_size) if split_head and w.head is not None else w.head
    if tiled and head is not None:
        from .qmm_fast import tile

        head = tile(head)
    return Weights(local_cfg, w.embed, layers, w.norm, head, w.inv_freq)
