"""The tcgen05 prefill matmul on a B200: weights rounded once to bf16, one fp32 chain over K; rows do not depend on how
the prompt is chunked.  Mirrors the reference's contract for ``prefill_matmul`` (cuda/kernels/qmm.py:160-171)."""

import numpy as np
import pytest
import torch

from oracle import affine as oaff
from tensorfold_b200 import _lib, synthetic
from tensorfold_b200.cuda.kernels import qmm

from gpu_util import DEV, to_dev

pytestmark = pytest.mark.gpu


def reference(x, words, scales, biases, gs):
    """float64 x @ bf16(q * s + b).T: the weight is rounded once to bf16 (q * s + b is exact in float64)."""

    w = oaff.dequantize(words.numpy(), scales.float().numpy(), biases.float().numpy(), 4, gs)
    w = oaff.bf16_round(w.astype(np.float32)).astype(np.float64)
    return x.float().numpy().astype(np.float64) @ w.T


@pytest.mark.parametrize("n,k,gs,m", [(128, 64, 64, 8), (128, 256, 64, 256), (1024, 5120, 64, 300), (384, 2048, 32, 70),
                                      (200, 1024, 32, 1), (5120, 6144, 64, 512)])
def test_matches_the_oracle(n, k, gs, m):
    w = synthetic.affine_weight(n, k, 4, gs, seed=n + k + m)
    q = qmm.pack(*to_dev(*w), gs)
    x = synthetic.activations(m, k, 1)
    y = qmm.prefill_matmul(x.to(DEV), q)
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    ref = reference(x, *w, gs)
    err = np.abs(y.float().cpu().numpy() - ref).max()
    assert err <= np.abs(ref).max() * 2 ** -7, f"max abs error {err} vs {np.abs(ref).max()}"
    f32 = qmm.prefill_matmul(x.to(DEV), q, f32=True)
    assert torch.equal(f32.to(torch.bfloat16), y)
    assert np.abs(f32.cpu().numpy() - ref).max() <= np.abs(ref).max() * 2 ** -12
    assert _lib.device_error(y) == 0


def test_exact_integer_case_is_bit_exact():
    rng = np.random.default_rng(7)
    n, k, gs, m = 140, 128, 64, 19
    values = rng.integers(0, 16, size=(n, k), dtype=np.uint32)
    words = torch.from_numpy(oaff.pack_codes(values, 4).view(np.int32))
    scales, biases = torch.full((n, 2), 0.25).bfloat16(), torch.full((n, 2), -0.5).bfloat16()
    xf = rng.integers(-2, 3, size=(m, k)).astype(np.float32) * 0.5
    want = np.sum(xf[:, None, :] * (values.astype(np.float32) * 0.25 - 0.5)[None, :, :], axis=2)
    q = qmm.pack(*to_dev(words, scales, biases), gs)
    got = qmm.prefill_matmul(torch.from_numpy(xf).bfloat16().to(DEV), q, f32=True)
    np.testing.assert_array_equal(got.cpu().numpy(), want)


@pytest.mark.parametrize("n,k,gs", [(1024, 5120, 64), (512, 2048, 32)])
def test_rows_do_not_depend_on_the_chunk(n, k, gs):
    q = qmm.pack(*to_dev(*synthetic.raw_weight(n, k, 4, gs, 3 * n + k)), gs)
    x = synthetic.activations(700, k, 5).to(DEV)
    whole = qmm.prefill_matmul(x, q)
    for a, b in ((0, 1), (255, 257), (699, 700), (0, 256), (100, 612), (3, 4)):
        assert torch.equal(qmm.prefill_matmul(x[a:b], q), whole[a:b]), (a, b)
    perm = torch.randperm(700, generator=torch.Generator().manual_seed(3)).to(DEV)
    assert torch.equal(qmm.prefill_matmul(x[perm], q), whole[perm])
    wide = torch.zeros((700, k + 64), dtype=torch.bfloat16, device=DEV)
    wide[:, :k] = x
    assert torch.equal(qmm.prefill_matmul(wide[:, :k], q), whole)             # strided rows


def test_blocks_that_run_several_tiles_keep_the_bits():
    """360 tiles on at most 148 persistent blocks: a block runs two or three tiles back to back on alternating
    accumulators.  Every 256-row chunk run on its own (40 tiles: one per block) must give the same bits, and the whole
    must match the oracle."""

    n, k, gs, m = 5120, 256, 64, 2304
    w = synthetic.affine_weight(n, k, 4, gs, seed=77)
    q = qmm.pack(*to_dev(*w), gs)
    x = synthetic.activations(m, k, 9)
    whole = qmm.prefill_matmul(x.to(DEV), q)
    for a in range(0, m, 256):
        assert torch.equal(qmm.prefill_matmul(x[a:a + 256].to(DEV), q), whole[a:a + 256]), a
    ref = reference(x, *w, gs)
    assert np.abs(whole.float().cpu().numpy() - ref).max() <= np.abs(ref).max() * 2 ** -7
    pair = qmm.pack_pair(to_dev(*w), to_dev(*synthetic.affine_weight(n, k, 4, gs, seed=78)), gs)
    act = qmm.matmul_act(x.to(DEV), pair, act="swiglu", prefill=True)       # 80 x 9 tiles through the SwiGLU drain
    for a in (0, 1024, 2048):
        assert torch.equal(qmm.matmul_act(x[a:a + 256].to(DEV), pair, act="swiglu", prefill=True), act[a:a + 256]), a
    assert _lib.device_error(whole) == 0


def test_other_formats_fall_back_to_the_exact_matmul():
    w = synthetic.affine_weight(256, 1024, 3, 128, seed=4)
    q = qmm.pack(*to_dev(*w), 128, bits=3)
    x = synthetic.activations(40, 1024, 2).to(DEV)
    assert torch.equal(qmm.prefill_matmul(x, q), qmm.matmul(x, q))
