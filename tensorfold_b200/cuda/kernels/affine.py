"""Packed MLX affine projections without dense weight copies or row-dependent arithmetic.

Host-side mirror of the reference module ``tensorfold.cuda.kernels.affine`` (cuda/kernels/affine.py:5-87).  Every width
(2/3/4/5/6/8 bits) and group (32/64/128) runs the same tiled kernel as the 4-bit lane matmul; a projection still in the
stored MLX layout is repacked once (same size, no dense copy) the first time it is used and the tiled form is kept.
"""

from __future__ import annotations

import weakref

BITS = (2, 3, 4, 5, 6, 8)
GROUPS = (32, 64, 128)


def packed_shape(weight, scales, biases, bits: int, group: int) -> tuple[int, int]:
    if bits not in BITS or group not in GROUPS:
        raise ValueError("CUDA affine weights require 2/3/4/5/6/8 bits and groups of 32/64/128")
    if len(weight) != 2 or len(scales) != 2 or tuple(scales) != tuple(biases):
        raise ValueError("affine projections need 2-D weights and matching scales and biases")
    n, groups = map(int, scales)
    k = groups * group
    if n <= 0 or groups <= 0 or tuple(weight) != (n, k * bits // 32):
        raise ValueError("packed affine words do not match their declared bit width and group metadata")
    return n, k


def input_slice(k: int, bits: int, group: int, rank: int, world: int = 2):
    """Split only whole quantization groups and packed words, without changing any values (any world size)."""

    if world < 1 or not 0 <= rank < world or bits not in BITS or group not in GROUPS or k % (world * group):
        raise ValueError("tensor parallel affine inputs must split into complete group-aligned shares")
    count = k // (world * group)
    a, b = rank * count, (rank + 1) * count
    if (a * group * bits) % 32 or (b * group * bits) % 32:
        raise ValueError("a rank's share must start and end on a packed word")
    return (a * group * bits // 32, b * group * bits // 32), (a, b)


_tiled: dict[tuple, object] = {}


def tiled(q):
    """The tiled form of a stored-layout projection (``Q4``), made on first use and kept while the words live."""

    import torch

    from . import qmm

    if q.layout == "tiled":
        return qmm.Q4(q.weight, None, None, q.n, q.k, q.gs, q.bits)
    key = (q.weight.data_ptr(), q.scales.data_ptr(), q.biases.data_ptr(), tuple(q.weight.shape), q.bits, q.gs)
    hit = _tiled.get(key)
    if hit is not None and hit[0]() is q.weight:
        return hit[1]
    if q.scales.dtype != torch.bfloat16 or q.biases.dtype != torch.bfloat16:
        raise ValueError("this build tiles affine projections with bf16 scales and biases only")
    packed = qmm.pack(q.weight, q.scales, q.biases, q.gs, bits=q.bits)
    _tiled[key] = (weakref.ref(q.weight), packed)
    return packed


def _validate(x, q):
    import torch

    if q.layout == "dense":
        raise ValueError("unquantized (dense) projections are outside this build: it serves packed affine weights")
    if q.layout == "tiled":
        n, k = q.n, q.k
    else:
        if q.layout != "mlx":
            raise ValueError("generic affine kernels read the original MLX word layout")
        n, k = packed_shape(q.weight.shape, q.scales.shape, q.biases.shape, q.bits, q.gs)
        if q.weight.dtype != torch.int32 or any(t.dtype not in (torch.bfloat16, torch.float16, torch.float32)
                                               for t in (q.scales, q.biases)):
            raise ValueError("affine words must be int32 with floating-point scales and biases")
        if any(t is not None and not t.is_contiguous() for t in (q.weight, q.scales, q.biases)):
            raise ValueError("affine weights and group metadata must be contiguous")
    if x.ndim != 2 or x.shape[1] != k or x.dtype != torch.bfloat16 or x.shape[0] < 1:
        raise ValueError("affine inputs must be nonempty BF16 rows of the declared input width")
    if not x.is_cuda or q.weight.device != x.device:
        raise ValueError("affine operands must share a CUDA device")
    return n, k


def matmul(x, q, *, f32: bool = False):
    from . import qmm

    _validate(x, q)
    return qmm.matmul(x, tiled(q), f32=f32)


def embed(ids, q):
    import torch

    from ... import _lib

    if ids.ndim != 1 or ids.dtype not in (torch.int32, torch.int64) or ids.device != q.weight.device:
        raise ValueError("embedding IDs must be a vector on the weights' CUDA device")
    if q.layout != "mlx" or q.weight.dtype != torch.int32:
        raise ValueError("generic embeddings require original int32 MLX packed words")
    n, k = packed_shape(q.weight.shape, q.scales.shape, q.biases.shape, q.bits, q.gs)
    meta = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}.get(q.scales.dtype)
    if meta is None or q.biases.dtype != q.scales.dtype:
        raise ValueError("scales and biases must share a floating-point dtype")
    stream = _lib.stream_of(ids)
    ids = ids.contiguous()
    out = torch.empty((ids.shape[0], k), dtype=torch.bfloat16, device=ids.device)
    for a in range(0, ids.shape[0], 65535):
        part = ids[a:a + 65535]
        _lib.check(_lib.lib().tf_affine_rows(part.data_ptr(), int(ids.dtype == torch.int64), part.shape[0], q.weight.data_ptr(),
                                             q.scales.data_ptr(), q.biases.data_ptr(), meta, n, k, q.bits, q.gs,
                                             out[a:a + 65535].data_ptr(), 0, stream), "embed")
    return out
