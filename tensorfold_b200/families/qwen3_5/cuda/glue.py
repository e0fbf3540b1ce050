"""Row-wise glue that feeds the quantized matmuls: residual add + RMSNorm and SwiGLU, each returning the fp32 group sums
of its bf16 output (a matmul's ``xs``).  Mirrors ``add_rmsnorm`` and ``swiglu`` of the reference
(families/qwen3_5/cuda/glue.py:31-40,146-151); each row is computed on its own, in a fixed order of operations."""

from __future__ import annotations

import torch

from .... import _lib


def _rows(t: torch.Tensor, who: str) -> torch.Tensor:
    if t.dim() != 2 or t.dtype != torch.bfloat16 or not t.is_cuda:
        raise ValueError(f"{who}: rows must be a 2-D bf16 CUDA tensor")
    return t if t.is_contiguous() else t.contiguous()


def add_rmsnorm(x: torch.Tensor, r: torch.Tensor | None, w: torch.Tensor, eps: float, gs: int = 64):
    """h = x + r (bf16), y = rmsnorm(h) * w (bf16), xs = y's group sums (fp32).  Returns (h, y, xs); h is x when r is None."""

    x = _rows(x, "add_rmsnorm")
    rows, d = x.shape
    if r is not None:
        r = _rows(r, "add_rmsnorm")
        if r.shape != x.shape:
            raise ValueError("add_rmsnorm: x and r must have the same shape")
    if w.dtype != torch.bfloat16 or w.shape != (d,) or not w.is_cuda:
        raise ValueError("add_rmsnorm: w must be a bf16 CUDA vector of the row length")
    w = w.contiguous()
    h = torch.empty_like(x) if r is not None else x
    y = torch.empty_like(x)
    xs = torch.empty((rows, d // gs), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().tf_add_rmsnorm(x.data_ptr(), r.data_ptr() if r is not None else None, w.data_ptr(), rows, d, float(eps),
                                         h.data_ptr() if r is not None else None, y.data_ptr(), xs.data_ptr(), gs,
                                         _lib.stream_of(x)), "add_rmsnorm")
    return h, y, xs


def swiglu(gate: torch.Tensor, up: torch.Tensor, gs: int = 64):
    """out = bf16(gate * sigmoid(gate) * up), xs = out's group sums (fp32).  Returns (out, xs)."""

    gate, up = _rows(gate, "swiglu"), _rows(up, "swiglu")
    if gate.shape != up.shape:
        raise ValueError("swiglu: gate and up must have the same shape")
    rows, n = gate.shape
    out = torch.empty_like(gate)
    xs = torch.empty((rows, n // gs), dtype=torch.float32, device=gate.device)
    _lib.check(_lib.lib().tf_swiglu(gate.data_ptr(), up.data_ptr(), rows, n, out.data_ptr(), xs.data_ptr(), gs,
                                    _lib.stream_of(gate)), "swiglu")
    return out, xs
