"""Dense-27B-shaped projections (hidden 5120, affine 4-bit / group 64) at M = 1, 4, 16 and 2048: rows bit-identical at
every row count through the one entry point, and within the bf16 tolerance of the oracle."""

import pytest
import torch

from tensorfold_b200 import synthetic
from tensorfold_b200.cuda.kernels import qmm

from gpu_util import DEV, assert_close_bf16, oracle_f64, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", list(synthetic.DENSE_27B))
def test_projection_rows_are_bit_exact_across_row_counts_and_accurate(name):
    n, k = synthetic.DENSE_27B[name]
    words, scales, biases = synthetic.affine_weight(n, k, 4, 64, seed=sum(map(ord, name)))
    q = qmm.pack(*to_dev(words, scales, biases), 64)
    x = synthetic.activations(2048, k, 1)
    xd = x.to(DEV)
    big = qmm.matmul(xd, q)                                      # M = 2048 (prefill chunk) through the same entry point
    for m in (1, 4, 16):
        assert torch.equal(qmm.matmul(xd[:m], q), big[:m]), f"{name}: M={m} rows differ from M=2048"
    for r in (0, 15, 777, 2047):
        assert torch.equal(qmm.matmul(xd[r:r + 1], q), big[r:r + 1]), f"{name}: row {r} alone differs"
    # accuracy on a bounded sample of columns (the float64 oracle over all of gate_proj would take minutes)
    cols = 1024
    ref = oracle_f64(x[:16], words[:cols], scales[:cols], biases[:cols], 64, 4)
    assert_close_bf16(big[:16, :cols], ref, name)
    # linearity in x, a size-independent property: f32 outputs of 2x are exactly twice those of x
    y1 = qmm.matmul(xd[:16], q, f32=True)
    y2 = qmm.matmul(xd[:16] * 2, q, f32=True)
    assert torch.equal(y2, y1 * 2), f"{name}: scaling x by 2 must scale every fp32 sum exactly"
