"""The projection record the kernels' callers pass around.  Mirrors ``QLinear`` of the reference
(families/qwen3_5/cuda/weights.py:14-40); ``tensorfold_b200.cuda.checkpoint`` fills it from safetensors files."""

from __future__ import annotations

from dataclasses import dataclass, field
from functools import cached_property
from typing import Any

import torch


@dataclass
class QLinear:
    weight: torch.Tensor      # original MLX words, or the tiled units (``qmm_fast.tile``)
    scales: torch.Tensor | None
    biases: torch.Tensor | None
    layout: str = "mlx"       # "mlx" as stored, or "tiled"
    rows: int = 0             # N when tiled (the tiled units are padded to 128 columns)
    gs: int = 64              # inputs per quantization group
    bits: int = 4
    cols: int = 0             # K when tiled

    @property
    def n(self) -> int:
        return self.rows if self.layout == "tiled" else int(self.weight.shape[0])

    @property
    def k(self) -> int:
        if self.layout == "dense":
            return int(self.weight.shape[1])
        return self.cols if self.layout == "tiled" else int(self.scales.shape[1]) * self.gs

    def nbytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.weight, self.scales, self.biases) if t is not None)

    @cached_property
    def fast(self) -> bool:
        if self.layout == "tiled":
            return True
        return (self.bits, self.gs) == (4, 64) and self.layout != "dense" and all(
            t.dtype == torch.bfloat16 for t in (self.scales, self.biases))


# The layer containers the sharding and packing helpers walk (families/qwen3_5/cuda/weights.py:107-215 of the
# reference).  Only the fields those helpers touch are kept: the projections, and the per-head tensors that are cut
# with them.  Attention, the GDN recurrence and the norms themselves are outside this library.

@dataclass
class Config:
    hidden: int
    intermediate: int
    heads: int
    kv_heads: int
    head_dim: int
    k_heads: int = 0          # GDN key heads
    v_heads: int = 0          # GDN value heads
    dk: int = 0
    dv: int = 0
    vocab: int = 0


@dataclass
class GDN:
    qkv: QLinear
    z: QLinear
    b: QLinear
    a: QLinear
    out: QLinear
    conv: torch.Tensor        # (conv_dim, kernel)
    A_log: torch.Tensor       # (Hv,)
    dt_bias: torch.Tensor     # (Hv,)
    norm: torch.Tensor | None = None
    zba: QLinear | None = None  # [z | b | a] stacked into one projection (``qmm_fast.stack``)


@dataclass
class Attention:
    q: QLinear                # (heads * head_dim * 2, hidden): [q_h | gate_h] per head
    k: QLinear
    v: QLinear
    o: QLinear
    q_norm: torch.Tensor | None = None
    k_norm: torch.Tensor | None = None
    kv: QLinear | None = None   # [k | v] stacked


@dataclass
class Layer:
    linear: bool = False
    input_norm: torch.Tensor | None = None
    post_norm: torch.Tensor | None = None
    gdn: GDN | None = None
    attn: Attention | None = None
    gate: QLinear | None = None
    up: QLinear | None = None
    down: QLinear | None = None
    moe: Any = None


@dataclass
class Weights:
    config: Config
    embed: Any
    layers: list = field(default_factory=list)
    norm: torch.Tensor | None = None
    head: Any = None
    inv_freq: torch.Tensor | None = None
