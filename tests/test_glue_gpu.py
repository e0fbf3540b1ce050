"""The row-wise glue on a B200 against the CPU restatement: residual add + RMSNorm and SwiGLU with the group sums a
matmul takes as ``xs``.  Rows keep their bits whatever the row count (reference: families/qwen3_5/cuda/glue.py:1)."""

import numpy as np
import pytest
import torch

from oracle import glue as oglue
from tensorfold_b200 import synthetic
from tensorfold_b200.cuda.kernels import qmm
from tensorfold_b200.families.qwen3_5.cuda import glue

from gpu_util import DEV, to_dev

pytestmark = pytest.mark.gpu


def ulps(got: torch.Tensor, ref: np.ndarray) -> float:
    """Largest error in units of 2^-8 of the reference: neighbouring bf16 values are between 1 and 2 of these apart."""

    g = got.float().cpu().numpy().astype(np.float64)
    return float(np.max(np.abs(g - ref) / np.maximum(np.abs(ref) * 2.0 ** -8, 1e-30)))


@pytest.mark.parametrize("rows,d,gs,residual", [(1, 64, 64, True), (5, 5120, 64, True), (33, 2688, 64, False), (16, 6144, 128, True),
                                                (7, 1536, 32, True)])
def test_add_rmsnorm_matches_the_oracle(rows, d, gs, residual):
    g = torch.Generator().manual_seed(rows + d)
    x = synthetic.activations(rows, d, 1)
    r = synthetic.activations(rows, d, 2) if residual else None
    w = (1 + 0.1 * torch.randn((d,), generator=g)).to(torch.bfloat16)
    h, y, xs = glue.add_rmsnorm(x.to(DEV), r.to(DEV) if residual else None, w.to(DEV), 1e-6, gs)
    rh, ry, _ = oglue.add_rmsnorm(x.float().numpy(), r.float().numpy() if residual else None, w.float().numpy(), 1e-6, gs)
    assert torch.equal(h.cpu(), torch.from_numpy(rh).to(torch.bfloat16))        # the sum of two bf16 values, rounded once
    assert ulps(y, ry.astype(np.float64)) <= 2.0                                  # fp32 against float64: one bf16 spacing
    sums = y.float().cpu().numpy().astype(np.float64).reshape(rows, d // gs, gs).sum(-1)      # of the kernel's own y
    assert np.abs(xs.cpu().numpy() - sums).max() <= 1e-5 * max(1.0, np.abs(sums).max())
    one = glue.add_rmsnorm(x[rows // 2:rows // 2 + 1].to(DEV), r[rows // 2:rows // 2 + 1].to(DEV) if residual else None,
                           w.to(DEV), 1e-6, gs)
    for a, b in zip(one, (h, y, xs)):
        assert torch.equal(a, b[rows // 2:rows // 2 + 1])                        # a row alone: the same bits


@pytest.mark.parametrize("rows,n,gs", [(1, 64, 64), (16, 17408, 64), (9, 1856, 64), (3, 4096, 128), (40, 2720, 32)])
def test_swiglu_matches_the_oracle(rows, n, gs):
    gate, up = synthetic.activations(rows, n, 3) * 2, synthetic.activations(rows, n, 4)
    gate = gate.to(torch.bfloat16)
    out, xs = glue.swiglu(gate.to(DEV), up.to(DEV), gs)
    ref, _ = oglue.swiglu(gate.float().numpy(), up.float().numpy(), gs)
    assert ulps(out, ref.astype(np.float64)) <= 2.0
    sums = out.float().cpu().numpy().astype(np.float64).reshape(rows, n // gs, gs).sum(-1)
    assert np.abs(xs.cpu().numpy() - sums).max() <= 1e-5 * max(1.0, np.abs(sums).max())
    one = glue.swiglu(gate[rows - 1:].to(DEV), up[rows - 1:].to(DEV), gs)
    assert torch.equal(one[0], out[rows - 1:]) and torch.equal(one[1], xs[rows - 1:])


def test_group_sums_feed_the_matmul():
    """The glue's sums stand in for the matmul's own (``xs=``): same result within the bf16 tolerance, rows bit-stable."""

    n, k, gs = 512, 1024, 64
    q = qmm.pack(*to_dev(*synthetic.affine_weight(n, k, 4, gs, seed=5)), gs)
    x = synthetic.activations(6, k, 7).to(DEV)
    w = torch.ones((k,), dtype=torch.bfloat16, device=DEV)
    _, y, xs = glue.add_rmsnorm(x, None, w, 1e-6, gs)
    with_sums, own = qmm.matmul(y, q, xs), qmm.matmul(y, q)
    assert (with_sums.float() - own.float()).abs().max() <= 2 ** -7 * own.float().abs().max()
    assert torch.equal(qmm.matmul(y[2:3], q, xs[2:3]), with_sums[2:3])


def test_bad_arguments_are_refused():
    x = torch.zeros((2, 96), dtype=torch.bfloat16, device=DEV)
    w = torch.ones((96,), dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError):
        glue.add_rmsnorm(x, None, w, 1e-6, 64)                   # 96 is not a multiple of the group
    with pytest.raises(ValueError):
        glue.swiglu(x, x[:, :64], 32)
    with pytest.raises(ValueError):
        glue.add_rmsnorm(x.float(), None, w, 1e-6, 32)
