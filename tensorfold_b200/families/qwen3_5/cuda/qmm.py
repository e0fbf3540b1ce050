"""Stored-layout entry points of the 27B family: the lane matmul on MLX words and the diagnostic dequantiser.
Mirrors families/qwen3_5/cuda/qmm.py:14-149 of the reference; both run the shared tiled kernel, so they give the bits of
``tensorfold_b200.cuda.kernels.qmm.matmul`` by construction."""

from __future__ import annotations

import torch

from .... import _lib
from ....cuda.kernels import affine, qmm as shared
from .weights import QLinear

BN = 64


def bucket(m: int) -> int:
    if m < 1:
        raise ValueError("lane matmul takes at least one row")
    for b in (16, 32, 64):
        if m <= b:
            return b
    return 128


def split_k(n: int, k: int) -> int:
    return shared.split_k(n, k, 64)


def group_sums(x: torch.Tensor) -> torch.Tensor:
    return shared.group_sums(x, 64)


def lane_matmul(x: torch.Tensor, weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor,
                xs: torch.Tensor | None = None, sk: int | None = None, bm: int | None = None) -> torch.Tensor:
    """x (M, K) bf16 times the packed 4-bit ``weight`` (N, K/8) transposed -> (M, N) bf16 (row tile ``bm`` is accepted
    and ignored: tiles never change bits)."""

    if x.dtype != torch.bfloat16 or x.dim() != 2:
        raise ValueError("lane_matmul: x must be a 2-D bf16 tensor")
    if weight.shape[1] * 8 != x.shape[1] or x.shape[1] % 64:
        raise ValueError(f"lane_matmul: weight {tuple(weight.shape)} does not match K={x.shape[1]}")
    if bm is not None and int(bm) not in (16, 32, 64, 128):
        raise ValueError("lane_matmul: row tile must be 16, 32, 64 or 128")
    q = affine.tiled(QLinear(weight, scales, biases))
    return shared.matmul(x, q, xs, sk=sk)


def dequantize(weight: torch.Tensor, scales: torch.Tensor | None, biases: torch.Tensor | None,
               bits: int = 4, gs: int = 64) -> torch.Tensor:
    """Diagnostic reference only: fp32 ``q * scale + bias`` of every row."""

    if scales is None:
        return weight.float()
    n, k = affine.packed_shape(weight.shape, scales.shape, biases.shape, bits, gs)
    meta = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[scales.dtype]
    stream = _lib.stream_of(weight)
    out = torch.empty((n, k), dtype=torch.float32, device=weight.device)
    w, s, b = weight.contiguous(), scales.contiguous(), biases.contiguous()
    for a in range(0, n, 65535):
        rows = min(65535, n - a)
        _lib.check(_lib.lib().tf_affine_rows(None, 0, rows, w[a:].data_ptr(), s[a:].data_ptr(), b[a:].data_ptr(), meta, n - a,
                                             k, bits, gs, out[a:].data_ptr(), 1, stream), "dequantize")
    return out
