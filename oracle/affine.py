"""CPU restatement of the MLX-affine packed-row format and its matmul.  Test infrastructure only (see package doc).

Every function names the reference lines it follows (paths inside the reference project).  Integer work is numpy and
exact; floating-point references are float64 unless a function says otherwise.
"""

from __future__ import annotations

import numpy as np

BITS = (2, 3, 4, 5, 6, 8)          # cuda/kernels/affine.py:5
GROUPS = (32, 64, 128)             # cuda/kernels/affine.py:6


# ----------------------------------------------------------------------------------------------------------------------
# bf16 helpers (numpy has no bfloat16: values travel as float32 that are exactly representable in bf16, or as uint16 bits)
# ----------------------------------------------------------------------------------------------------------------------

def bf16_round(a) -> np.ndarray:
    """float32 -> nearest bf16 (ties to even), returned as float32.  NaNs are kept quiet."""

    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    rounded = ((u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000).astype(np.uint32)
    out = rounded.view(np.float32).copy()
    nan = np.isnan(a)
    if nan.any():
        out[nan] = np.float32("nan")
    return out.reshape(a.shape)


def bf16_bits(a) -> np.ndarray:
    """float32 values (already bf16-representable or not) -> uint16 bf16 bit patterns, round-to-nearest-even."""

    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(u) -> np.ndarray:
    return (np.asarray(u, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------------------------------------------------------------
# the packed format
# ----------------------------------------------------------------------------------------------------------------------

def packed_shape(weight, scales, biases, bits: int, group: int) -> tuple[int, int]:
    """Shape check of (weight, scales, biases) shapes -> (n, k).  Follows cuda/kernels/affine.py:9-18."""

    if bits not in BITS or group not in GROUPS:
        raise ValueError("affine weights require 2/3/4/5/6/8 bits and groups of 32/64/128")
    if len(weight) != 2 or len(scales) != 2 or tuple(scales) != tuple(biases):
        raise ValueError("affine projections need 2-D weights and matching scales and biases")
    n, groups = map(int, scales)
    k = groups * group
    if n <= 0 or groups <= 0 or tuple(weight) != (n, k * bits // 32):
        raise ValueError("packed affine words do not match their declared bit width and group metadata")
    return n, k


def input_slice(k: int, bits: int, group: int, rank: int, world: int = 2):
    """Word and group ranges of rank's share of K: whole groups and whole words only.

    Follows cuda/kernels/affine.py:21-27, which fixes world = 2; here any world that divides K into whole groups whose
    boundaries fall on word boundaries (the generalisation the 4- and 8-GPU shard maps need).
    """

    if world < 1 or not 0 <= rank < world or bits not in BITS or group not in GROUPS or k % (world * group):
        raise ValueError("tensor parallel affine inputs must split into complete group-aligned shares")
    count = k // (world * group)
    a, b = rank * count, (rank + 1) * count
    if (a * group * bits) % 32 or (b * group * bits) % 32:
        raise ValueError("a rank's share must start and end on a packed word")
    return (a * group * bits // 32, b * group * bits // 32), (a, b)


def pack_codes(values, bits: int) -> np.ndarray:
    """(N, K) integer codes in [0, 2^bits) -> (N, K*bits/32) uint32: code k occupies bits [k*bits, k*bits+bits) of the
    row's little-endian bit stream (it may straddle two words).  Inverse of ``codes``."""

    values = np.asarray(values, dtype=np.uint64)
    n, k = values.shape
    if (k * bits) % 32:
        raise ValueError("a row must fill whole 32-bit words")
    nw = k * bits // 32
    out = np.zeros((n, nw + 1), dtype=np.uint64)
    pos = np.arange(k, dtype=np.uint64) * np.uint64(bits)
    word, shift = (pos >> np.uint64(5)).astype(np.int64), pos & np.uint64(31)
    lo = (values << shift) & np.uint64(0xFFFFFFFF)
    hi = (values << shift) >> np.uint64(32)
    for j in range(k):                                   # k is small in tests; exactness matters, not speed
        out[:, word[j]] |= lo[:, j]
        out[:, word[j] + 1] |= hi[:, j]
    return out[:, :nw].astype(np.uint32)


def codes(words, bits: int) -> np.ndarray:
    """(N, W) uint32 (or int32) packed rows -> (N, 32*W/bits) uint32 codes.

    Follows the bit-stream rule of cuda/kernels/affine_kernels.py:7-14 (low word shifted right, the straddling high word
    shifted left by 32 - shift, masked to ``bits``) and kernels/qwen/dense/v1/affine_rows.py:14-21 (``code_at``).
    """

    w = np.ascontiguousarray(words).view(np.uint32).astype(np.uint64)
    n, nw = w.shape
    k = nw * 32 // bits
    padded = np.concatenate([w, np.zeros((n, 1), dtype=np.uint64)], axis=1)
    bit = np.arange(k, dtype=np.uint64) * np.uint64(bits)
    word, shift = (bit >> np.uint64(5)).astype(np.int64), bit & np.uint64(31)
    both = padded[:, word] | (padded[:, word + 1] << np.uint64(32))
    return ((both >> shift) & np.uint64((1 << bits) - 1)).astype(np.uint32)


def dequantize(words, scales, biases, bits: int = 4, gs: int = 64, dtype=np.float64) -> np.ndarray:
    """w[n, k] = scales[n, k // gs] * q[n, k] + biases[n, k // gs].

    Follows families/qwen3_5/cuda/qmm.py:132-149 (which computes in float32; pass ``dtype=np.float32`` for its bits).
    """

    q = codes(words, bits).astype(dtype)
    s = np.repeat(np.asarray(scales, dtype=dtype), gs, axis=1)
    b = np.repeat(np.asarray(biases, dtype=dtype), gs, axis=1)
    return q * s + b


def quantized_matmul(x, words, scales, biases, gs: int = 64, bits: int = 4) -> np.ndarray:
    """float64 ``x @ dequantize(w).T``: the affine definition every kernel is judged against.

    Follows the references the reference's own tests use: tests/cuda/test_qmm.py:22-26,64-70 and
    tests/cuda/test_experts.py:26-30 (MLX ``quantized_matmul(..., transpose=True)`` semantics, lane_qmm.py:366-370).
    """

    return np.asarray(x, dtype=np.float64) @ dequantize(words, scales, biases, bits, gs).T


def group_sums(x, gs: int = 64) -> np.ndarray:
    """xs[m, g] = sum of x[m, g*gs:(g+1)*gs] (float64 sum rounded to float32).  cuda/kernels/qmm.py:122-137."""

    x = np.asarray(x, dtype=np.float64)
    m, k = x.shape
    return x.reshape(m, k // gs, gs).sum(-1).astype(np.float32)


def split_k(n: int, k: int, gs: int = 64, target: int = 192) -> int:
    """K slices of an (n, k) weight, from the shape alone.  Follows cuda/kernels/qmm.py:105-111."""

    tiles, groups, sk = -(-n // 64), k // gs, 1
    while sk < 8 and tiles * sk < target and groups % (sk * 2) == 0 and groups // (sk * 2) >= 8:
        sk *= 2
    return sk


def bucket(m: int) -> int:
    """Row tile of the lane matmul: 16, 32, else 64.  Follows cuda/kernels/qmm.py:114-119."""

    if m < 1:
        raise ValueError("the lane matmul takes at least one row")
    return 16 if m <= 16 else 32 if m <= 32 else 64


def lane_matmul(x, words, scales, biases, gs: int = 64, bits: int = 4, sk: int | None = None,
                f32: bool = False, reduce: bool = True) -> np.ndarray:
    """Model of the decode/verify arithmetic: per K slice, for each group in order
    ``acc = xs*b + (P*s + acc)`` with ``P`` the exact group dot of x with the integer codes, slices added in slice order,
    one rounding to bf16 at the end.  Follows cuda/kernels/qmm.cu:83-93,173-201,221-226 and the Triton twin
    families/qwen3_5/cuda/qmm.py:63-73.  The tensor-core dot is modelled as an exact dot rounded to float32 and each
    fma as a float64 operation rounded to float32, so this is a tolerance model of a GPU kernel, not a bit model.
    """

    x = np.asarray(x, dtype=np.float64)
    q = codes(words, bits).astype(np.float64)
    m, k = x.shape
    n = q.shape[0]
    kg = k // gs
    sk = sk or split_k(n, k, gs)
    s = np.asarray(scales, dtype=np.float64)
    b = np.asarray(biases, dtype=np.float64)
    xs = group_sums(x, gs).astype(np.float64)
    per = kg // sk
    slices = np.zeros((sk, m, n), dtype=np.float32)
    for sl in range(sk):
        acc = np.zeros((m, n), dtype=np.float32)
        for g in range(sl * per, (sl + 1) * per):
            p = (x[:, g * gs:(g + 1) * gs] @ q[:, g * gs:(g + 1) * gs].T).astype(np.float32).astype(np.float64)
            inner = (p * s[None, :, g] + acc.astype(np.float64)).astype(np.float32)
            acc = (xs[:, g, None] * b[None, :, g] + inner.astype(np.float64)).astype(np.float32)
        slices[sl] = acc
    if not reduce:
        return slices
    total = slices[0]
    for sl in range(1, sk):
        total = (total + slices[sl]).astype(np.float32)
    return total if f32 else bf16_round(total)


def embed(ids, words, scales, biases, gs: int, bits: int) -> np.ndarray:
    """Rows ``ids`` of the dequantised table as bf16 (float32 holding bf16 values): ``bf16(q*s + b)`` in float32.
    Follows cuda/kernels/affine.py:71-87 and cuda/kernels/affine_kernels.py:49-60."""

    ids = np.asarray(ids, dtype=np.int64)
    w = np.ascontiguousarray(words).view(np.uint32)[ids]
    q = codes(w, bits).astype(np.float32)
    s = np.repeat(np.asarray(scales, dtype=np.float32)[ids], gs, axis=1)
    b = np.repeat(np.asarray(biases, dtype=np.float32)[ids], gs, axis=1)
    return bf16_round(q * s + b)


# ----------------------------------------------------------------------------------------------------------------------
# tensor-parallel shard map (CPU restatement)
# ----------------------------------------------------------------------------------------------------------------------

def output_rows(n: int, rank: int, world: int = 2, segments=None, block: int = 1) -> np.ndarray:
    """Rank-local output row indices in segment order.  Follows families/qwen3_5/cuda/distributed.py:27-42 with the
    two-rank guard (:22-24) widened to any world size."""

    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    lengths = tuple(segments) if segments is not None else (n,)
    if sum(lengths) != n or any(v <= 0 or v % (world * block) for v in lengths):
        raise ValueError(f"output segments {lengths} do not split into {world} blocks of {block}")
    base, ranges = 0, []
    for length in lengths:
        share = length // world
        ranges.append(np.arange(base + rank * share, base + (rank + 1) * share))
        base += length
    return np.concatenate(ranges)


def sum_rank_partials(partials, f32: bool = False) -> np.ndarray:
    """Rank-ordered float32 sum ``((p0 + p1) + p2) + ...`` then one rounding to bf16.
    Follows families/qwen3_5/cuda/distributed.py:259-264 (two ranks) extended left to right."""

    total = np.asarray(partials[0], dtype=np.float32)
    for p in partials[1:]:
        total = (total + np.asarray(p, dtype=np.float32)).astype(np.float32)
    return total if f32 else bf16_round(total)
