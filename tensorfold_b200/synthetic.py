"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.  Everything is drawn
on the CPU from a ``torch.Generator`` so a checker on the host and a kernel on the device see identical bits."""

from __future__ import annotations

import torch

DENSE_27B = {          # name -> (n, k): hidden 5120, MLX affine 4-bit / group 64
    "q_proj": (6144, 5120), "k_proj": (1024, 5120), "v_proj": (1024, 5120), "o_proj": (5120, 6144),
    "gate_proj": (17408, 5120), "up_proj": (17408, 5120), "down_proj": (5120, 17408),
}


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """(n, k) integer codes -> (n, k * bits / 32) int32 words, code j at bits [j * bits, j * bits + bits) of the row."""

    n, k = codes.shape
    if (k * bits) % 32:
        raise ValueError("rows must fill whole words")
    pos = torch.arange(k, dtype=torch.int64) * bits
    out = torch.zeros((n, k * bits // 32 + 1), dtype=torch.int64)
    c = codes.to(torch.int64)
    lo = (c << (pos % 32)) & 0xFFFFFFFF
    hi = (c << (pos % 32)) >> 32
    out.scatter_add_(1, (pos // 32).expand(n, k), lo)          # fields never overlap, so adding equals or-ing
    out.scatter_add_(1, (pos // 32 + 1).expand(n, k), hi)
    out = out[:, :-1]
    return torch.where(out >= 2 ** 31, out - 2 ** 32, out).to(torch.int32)


def affine_weight(n: int, k: int, bits: int = 4, gs: int = 64, seed: int = 0, *, centred: bool = True):
    """Codes uniform over [0, 2^bits), scale |N(0, 0.01)| + 1e-4, bias -(2^(bits-1)) * scale + N(0, 0.002).
    Returns (words int32 [n, k*bits/32], scales bf16 [n, k/gs], biases bf16 [n, k/gs])."""

    g = torch.Generator().manual_seed(seed)
    codes = torch.randint(0, 1 << bits, (n, k), generator=g)
    scales = (torch.randn((n, k // gs), generator=g) * 0.01).abs() + 1e-4
    biases = -(2 ** (bits - 1)) * scales + (torch.randn((n, k // gs), generator=g) * 0.002 if centred else 0)
    return pack_codes(codes, bits), scales.to(torch.bfloat16), biases.to(torch.bfloat16)


def raw_weight(n: int, k: int, bits: int, gs: int, seed: int):
    """Raw random words (every bit pattern), scales U(0.001, 0.021), biases N(0, 0.05): the reference tests' weights
    (tests/cuda/test_qmm.py:14-19)."""

    g = torch.Generator().manual_seed(seed)
    words = torch.randint(-(2 ** 31), 2 ** 31 - 1, (n, k * bits // 32), generator=g, dtype=torch.int64).to(torch.int32)
    scales = (torch.rand((n, k // gs), generator=g) * 0.02 + 0.001).to(torch.bfloat16)
    biases = (torch.randn((n, k // gs), generator=g) * 0.05).to(torch.bfloat16)
    return words, scales, biases


def activations(m: int, k: int, seed: int = 0, std: float = 1.0) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed + 7919)
    return (torch.randn((m, k), generator=g) * std).to(torch.bfloat16)


def bf16_bits(t: torch.Tensor):
    """bf16 tensor -> numpy uint16 bit patterns."""

    import numpy as np

    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)
