"""Keep one tiled path for every affine format and the helpers the family's loaders and forwards use.
Mirrors families/qwen3_5/cuda/qmm_fast.py:13-115 of the reference."""

from __future__ import annotations

import torch

from ....cuda.kernels import affine, qmm as shared
from .weights import QLinear, Weights


def tile(q: QLinear) -> QLinear:
    """Stored MLX words -> tiled units (every width and group; bf16 scales and biases)."""

    if q.layout == "tiled" or q.layout == "dense":
        return q
    if q.scales.dtype != torch.bfloat16 or q.biases.dtype != torch.bfloat16:
        return q
    p = shared.pack(q.weight, q.scales, q.biases, q.gs, bits=q.bits)
    return QLinear(p.weight, None, None, layout="tiled", rows=p.n, gs=q.gs, bits=q.bits, cols=p.k)


def _q4(q: QLinear) -> shared.Q4:
    return shared.Q4(q.weight, None, None, q.n, q.k, q.gs, q.bits)


def untile(q: QLinear) -> QLinear:
    """The stored MLX layout again (for the fp32 reference, TP sharding or slicing rows)."""

    if q.layout != "tiled":
        return q
    w, s, b = shared.unpack(_q4(q))
    return QLinear(w, s, b, gs=q.gs, bits=q.bits)


def rows(q: QLinear, a: int, b: int) -> QLinear:
    """Rows [a, b) of a tiled weight: a view when they start on a 128-row super-block, else a small copy."""

    if a % 128 == 0 and (b - a) > 0:
        return QLinear(q.weight[a // 128:-(-b // 128)], None, None, layout="tiled", rows=b - a, gs=q.gs, bits=q.bits, cols=q.k)
    t0, t1 = a // 128, -(-b // 128)
    part = shared.Q4(q.weight[t0:t1].contiguous(), None, None, min(q.n, t1 * 128) - t0 * 128, q.k, q.gs, q.bits)
    w, s, bias = shared.unpack(part)
    lo, hi = a - t0 * 128, b - t0 * 128
    return tile(QLinear(w[lo:hi].contiguous(), s[lo:hi].contiguous(), bias[lo:hi].contiguous(), gs=q.gs, bits=q.bits))


def matmul_rows(x: torch.Tensor, parts: list[QLinear]) -> torch.Tensor:
    """``x`` against row blocks of one weight, with the bits of the stacked weight's matmul."""

    sk = shared.default_split(sum(p.n for p in parts), parts[0].k, parts[0].gs)
    xs = shared.group_sums(x, parts[0].gs)
    return torch.cat([shared.matmul(x, _q4(p), xs, sk=sk) for p in parts], dim=1)


def matmul(x: torch.Tensor, q: QLinear, xs: torch.Tensor | None = None) -> torch.Tensor:
    """The lane matmul for either layout; both give the same bits."""

    if q.layout == "tiled":
        return shared.matmul(x, _q4(q), xs)
    return shared.matmul(x, affine.tiled(q), xs) if xs is not None else affine.matmul(x, q)


def matmul_partial(x: torch.Tensor, q: QLinear, xs: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 sums, unrounded: a row-parallel rank's share of a projection."""

    if q.layout == "tiled":
        return shared.matmul(x, _q4(q), xs, f32=True)
    return affine.matmul(x, q, f32=True)


def stack(parts: list[QLinear]) -> QLinear:
    """Several projections of the same input as one: stored-layout rows concatenated in order."""

    if any(q.layout != "mlx" for q in parts):
        raise ValueError("stack the stored layout, then tile")
    if len({(q.bits, q.gs, q.k, q.scales.dtype, q.biases.dtype) for q in parts}) != 1:
        raise ValueError("stacked projections must share an affine format and input width")
    return QLinear(torch.cat([q.weight for q in parts]).contiguous(), torch.cat([q.scales for q in parts]).contiguous(),
                   torch.cat([q.biases for q in parts]).contiguous(), gs=parts[0].gs, bits=parts[0].bits)


def _stackable(parts: list[QLinear]) -> bool:
    return (all(q is not None and q.layout == "mlx" for q in parts)
            and len({(q.bits, q.gs, q.k, q.scales.dtype, q.biases.dtype) for q in parts}) == 1)


def stack_small(layer) -> None:
    """[z | b | a] and [k | v] as one projection each (families/qwen3_5/cuda/qmm_fast.py:89-95): the gates and k/v are too
    narrow to fill the GPU alone.  Stacking changes the K split, hence the bits: a load-time decision.  (With
    ``shared.matmul_set`` the same projections share a launch WITHOUT changing bits; stacking stays for engines that
    want one output tensor.)"""

    if layer.gdn is not None and layer.gdn.zba is None and _stackable([layer.gdn.z, layer.gdn.b, layer.gdn.a]):
        layer.gdn.zba = stack([layer.gdn.z, layer.gdn.b, layer.gdn.a])
    if layer.attn is not None and layer.attn.kv is None and _stackable([layer.attn.k, layer.attn.v]):
        layer.attn.kv = stack([layer.attn.k, layer.attn.v])


PROJECTIONS = ((None, ("gate", "up", "down")), ("gdn", ("qkv", "z", "b", "a", "out", "zba")), ("attn", ("q", "k", "v", "o", "kv")))


def tile_layer(layer) -> None:
    """Tile every projection a layer holds, in place (stacked ones included)."""

    for owner_name, names in PROJECTIONS:
        owner = layer if owner_name is None else getattr(layer, owner_name)
        if owner is None:
            continue
        for name in names:
            q = getattr(owner, name, None)
            if q is not None:
                setattr(owner, name, tile(q))


def prepare(w: Weights, *, fuse: bool = False) -> None:
    """Pack every projection and the head in place (families/qwen3_5/cuda/qmm_fast.py:98-115); ``fuse`` stacks the
    narrow projections first, which changes K splits and bits, so every run of a model must share it."""

    for layer in w.layers:
        if fuse:
            stack_small(layer)
        tile_layer(layer)
    if w.head is not None:
        w.head = tile(w.head)
    if torch.cuda.is_available():
        torch.cuda.empty_cache()
