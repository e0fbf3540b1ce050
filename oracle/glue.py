"""CPU restatement of the row-wise glue (test infrastructure only, like the rest of ``oracle``): float64 arithmetic on
the bf16 inputs, outputs rounded to bf16.  Follows families/qwen3_5/cuda/glue.py:10-29 (``_add_rmsnorm``) and
:130-143 (``_swiglu``) of the reference, and the plain-torch formulas its test checks them against
(tests/cuda/test_qwen27_glue.py:24-44)."""

from __future__ import annotations

import numpy as np

from .affine import bf16_round


def add_rmsnorm(x, r, w, eps: float, gs: int = 64):
    """(h, y, xs): h = bf16(x + r) (x when r is None), y = bf16(h / sqrt(mean(h^2) + eps) * w), xs = group sums of y."""

    x = np.asarray(x, dtype=np.float64)
    h = x if r is None else bf16_round((x + np.asarray(r, dtype=np.float64)).astype(np.float32)).astype(np.float64)
    inv = 1.0 / np.sqrt((h * h).mean(axis=1, keepdims=True) + eps)
    y = bf16_round((h * inv * np.asarray(w, dtype=np.float64)[None, :]).astype(np.float32)).astype(np.float64)
    rows, d = y.shape
    return h.astype(np.float32), y.astype(np.float32), y.reshape(rows, d // gs, gs).sum(-1).astype(np.float32)


def swiglu(gate, up, gs: int = 64):
    """(out, xs): out = bf16(g * sigmoid(g) * u), xs = group sums of out."""

    g, u = np.asarray(gate, dtype=np.float64), np.asarray(up, dtype=np.float64)
    out = bf16_round((g / (1.0 + np.exp(-g)) * u).astype(np.float32)).astype(np.float64)
    rows, n = out.shape
    return out.astype(np.float32), out.reshape(rows, n // gs, gs).sum(-1).astype(np.float32)
