"""CPU restatement of the routed-MoE layer over affine 4-bit experts.  Test infrastructure only (see package doc).

float64 models of the value every device kernel must stay within tolerance of, plus the exact integer plan.
"""

from __future__ import annotations

import numpy as np

from .affine import bf16_round, dequantize


def router_logits(x, rows) -> np.ndarray:
    """float32 ``x @ rows.T`` of bf16 inputs (float64 accumulate, one rounding).  cuda/moe.py:23-55."""

    return (np.asarray(x, dtype=np.float64) @ np.asarray(rows, dtype=np.float64).T).astype(np.float32)


def select_rows(logits, top_k: int, experts: int, shared: bool = True):
    """Each row's ``top_k`` experts by float32 logit, largest first, the lower id among equal logits; weights
    ``bf16(exp(l_k - l_0) / sum)`` (a softmax over the chosen k); with ``shared`` one more slot: expert id ``experts``
    weighted ``bf16(sigmoid(bf16(logit[experts])))``.  Follows cuda/moe.py:58-85.  Returns (picks int32, wts float32).
    """

    logits = np.asarray(logits, dtype=np.float32)
    r = logits.shape[0]
    slots = top_k + (1 if shared else 0)
    picks = np.zeros((r, slots), dtype=np.int32)
    wts = np.zeros((r, slots), dtype=np.float32)
    for i in range(r):
        v = logits[i, :experts].copy()
        order = np.lexsort((np.arange(experts), -v.astype(np.float64)))[:top_k]     # by value desc, then id asc
        top = v[order[0]]
        ex = np.exp((v[order] - top).astype(np.float32)).astype(np.float32)
        total = np.float32(0.0)
        for e in ex:
            total = np.float32(total + e)
        picks[i, :top_k] = order
        wts[i, :top_k] = bf16_round((ex / total).astype(np.float32))
        if shared:
            sg = bf16_round(logits[i, experts:experts + 1])[0]
            picks[i, top_k] = experts
            wts[i, top_k] = bf16_round(np.asarray([1.0 / (1.0 + np.exp(-np.float64(sg)))], dtype=np.float32))[0]
    return picks, wts


def plan(picks, experts: int, tile: int):
    """Stable counting sort of the (row, slot) pairs by expert: ``members`` (pair ids grouped by expert, pair order
    kept), ``items`` rows (expert, first, count <= tile), and the number of distinct experts.
    Follows tests/cuda/test_experts.py:107-115 (``want_plan``), the specification of cuda/experts.cu:157-334."""

    flat = np.asarray(picks).reshape(-1)
    items, members = [], []
    for e in range(experts):
        pairs = np.nonzero(flat == e)[0].tolist()
        for j in range(0, len(pairs), tile):
            items.append([e, len(members) + j, min(tile, len(pairs) - j)])
        members += pairs
    return np.asarray(items, dtype=np.int32).reshape(-1, 3), np.asarray(members, dtype=np.int32), len(set(flat.tolist()))


def max_items(pairs: int, experts: int, tile: int = 16) -> int:
    """cuda/experts.py:95-98."""

    return min(pairs, experts) + pairs // tile


def silu_mul(g, u, limit: float = 0.0) -> np.ndarray:
    """SwiGLU as the families define it: ``bf16(bf16(silu(bf16 g)) * bf16 u)``, clipped first when limit > 0.
    Follows cuda/experts.cuh:57-65 (device) and tests/cuda/test_experts.py:150-156 (the float64 reference)."""

    g = bf16_round(np.asarray(g, dtype=np.float32)).astype(np.float64)
    u = bf16_round(np.asarray(u, dtype=np.float32)).astype(np.float64)
    if limit > 0:
        g, u = np.minimum(g, limit), np.clip(u, -limit, limit)
    act = bf16_round((g / (1.0 + np.exp(-g))).astype(np.float32)).astype(np.float64)
    return act * u


def expert_pairs(x, picks, gate, up, down, gs: int, limit: float = 0.0, weight_bf16: bool = False):
    """float64 reference of the per-pair activation and down projection.

    ``gate``/``up``/``down`` are (words [E, N, K/8], scales, biases) triples; pair p = row * slots + slot uses expert
    picks[p].  Returns (act [P, NI] float64 before the final bf16 rounding, y [P, D] float64 computed from the bf16-rounded
    activation).  Follows tests/cuda/test_experts.py:136-165.
    """

    x = np.asarray(x, dtype=np.float64)
    picks = np.asarray(picks)
    rows, slots = picks.shape
    pe = picks.reshape(-1)

    def weights(m, e):
        w = dequantize(m[0][e], m[1][e], m[2][e], 4, gs)
        return bf16_round(w.astype(np.float32)).astype(np.float64) if weight_bf16 else w

    ni, d = gate[0].shape[1], down[0].shape[1]
    act = np.zeros((rows * slots, ni))
    y = np.zeros((rows * slots, d))
    cache: dict[int, tuple] = {}
    for p, e in enumerate(pe):
        e = int(e)
        if e not in cache:
            cache[e] = (weights(gate, e), weights(up, e), weights(down, e))
        wg, wu, wd = cache[e]
        xr = x[p // slots]
        a = silu_mul((wg @ xr).astype(np.float32), (wu @ xr).astype(np.float32), limit)
        act[p] = a
        y[p] = wd @ bf16_round(a.astype(np.float32)).astype(np.float64)
    return act, y


def down_pairs(act, picks, down, gs: int, weight_bf16: bool = False) -> np.ndarray:
    """float64 down projection of given (bf16-valued) activations, pair p using expert picks[p]; ``weight_bf16`` rounds
    the dequantised weights to bf16 first (the prefill form, tests/cuda/test_experts.py:146-148)."""

    act = np.asarray(act, dtype=np.float64)
    pe = np.asarray(picks).reshape(-1)
    y = np.zeros((act.shape[0], down[0].shape[1]))
    cache: dict[int, np.ndarray] = {}
    for p, e in enumerate(pe):
        e = int(e)
        if e not in cache:
            w = dequantize(down[0][e], down[1][e], down[2][e], 4, gs)
            cache[e] = bf16_round(w.astype(np.float32)).astype(np.float64) if weight_bf16 else w
        y[p] = cache[e] @ act[p]
    return y


def expert_pairs_relu2(x, picks, up, down, gs: int, weight_bf16: bool = False):
    """The relu^2 form: act = relu(bf16(up x))^2 (before its bf16 rounding), then the down projection.
    Follows cuda/experts.cuh:67-70 and tests/cuda/test_experts.py:157-158."""

    x = np.asarray(x, dtype=np.float64)
    picks = np.asarray(picks)
    rows, slots = picks.shape
    pe = picks.reshape(-1)
    act = np.zeros((rows * slots, up[0].shape[1]))
    for p, e in enumerate(pe):
        w = dequantize(up[0][int(e)], up[1][int(e)], up[2][int(e)], 4, gs)
        if weight_bf16:
            w = bf16_round(w.astype(np.float32)).astype(np.float64)
        v = bf16_round((w @ x[p // slots]).astype(np.float32)).astype(np.float64)
        act[p] = np.maximum(v, 0.0) ** 2
    return act, down_pairs(bf16_round(act.astype(np.float32)), picks, down, gs, weight_bf16)


def combine(y, wts) -> np.ndarray:
    """Slot-ordered ``sum_k w[r, k] * y[r, k, :]`` in float32, rounded once to bf16.  cuda/moe.py:130-141."""

    y = np.asarray(y, dtype=np.float32)
    wts = np.asarray(wts, dtype=np.float32)
    acc = np.zeros((y.shape[0], y.shape[2]), dtype=np.float32)
    for k in range(y.shape[1]):
        acc = (acc + (wts[:, k, None] * y[:, k]).astype(np.float32)).astype(np.float32)
    return bf16_round(acc)
