"""The projection record the kernels' callers pass around.  Mirrors ``QLinear`` of the reference
(families/qwen3_5/cuda/weights.py:14-40); ``tensorfold_b200.cuda.checkpoint`` fills it from safetensors files."""

from __future__ import annotations

from dataclasses import dataclass
from functools import cached_property

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
