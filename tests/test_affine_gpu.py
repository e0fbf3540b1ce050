"""The generic affine entry points on a B200: every width and group through ``affine.matmul`` on stored MLX words, the
quantised embedding gather, the diagnostic dequantiser, the 27B family's stored-layout lane matmul and row helpers."""

import numpy as np
import pytest
import torch

from oracle import affine as oaff
from tensorfold_b200 import synthetic
from tensorfold_b200.cuda.kernels import affine, qmm
from tensorfold_b200.families.qwen3_5.cuda import qmm as lane, qmm_fast
from tensorfold_b200.families.qwen3_5.cuda.weights import QLinear

from gpu_util import DEV, assert_close_bf16, oracle_f64, to_dev

pytestmark = pytest.mark.gpu
FORMATS = [(b, g) for b in affine.BITS for g in affine.GROUPS]


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_matmul_on_stored_words_every_format(bits, gs):
    n, k = 200, gs * 12
    w = synthetic.affine_weight(n, k, bits, gs, seed=bits + gs)
    q = QLinear(*to_dev(*w), gs=gs, bits=bits)
    x = synthetic.activations(16, k, 3)
    y = affine.matmul(x.to(DEV), q)
    assert_close_bf16(y, oracle_f64(x, *w, gs, bits), f"{bits}b/g{gs}")
    assert torch.equal(affine.matmul(x[7:8].to(DEV), q), y[7:8])
    f32 = affine.matmul(x.to(DEV), q, f32=True)
    assert f32.dtype == torch.float32 and torch.equal(f32.to(torch.bfloat16), y)
    tiled = qmm_fast.tile(q)
    assert tiled.layout == "tiled" and torch.equal(qmm_fast.matmul(x.to(DEV), tiled), y)
    back = qmm_fast.untile(tiled)
    assert all(torch.equal(a, b.to(DEV)) for a, b in zip((back.weight, back.scales, back.biases), w))


@pytest.mark.parametrize("bits,gs", [(2, 32), (3, 64), (4, 64), (5, 128), (6, 32), (8, 64)])
def test_embed_and_dequantize_are_exact(bits, gs):
    n, k = 300, gs * 6
    w = synthetic.raw_weight(n, k, bits, gs, 5 * bits + gs)
    q = QLinear(*to_dev(*w), gs=gs, bits=bits)
    ids = torch.tensor([0, 299, 17, 17, 123], dtype=torch.int64)
    got = affine.embed(ids.to(DEV), q)
    want = oaff.embed(ids.numpy(), w[0].numpy(), w[1].float().numpy(), w[2].float().numpy(), gs, bits)
    np.testing.assert_array_equal(got.float().cpu().numpy(), want)
    assert torch.equal(affine.embed(ids.to(torch.int32).to(DEV), q), got)
    deq = lane.dequantize(q.weight, q.scales, q.biases, bits=bits, gs=gs)
    ref = oaff.dequantize(w[0].numpy(), w[1].float().numpy(), w[2].float().numpy(), bits, gs, dtype=np.float32)
    np.testing.assert_array_equal(deq.cpu().numpy(), ref)
    with pytest.raises(ValueError):
        affine.embed(ids.float().to(DEV), q)


def test_embed_accepts_fp16_and_fp32_metadata():
    n, k, gs, bits = 64, 256, 64, 8
    w, s, b = synthetic.raw_weight(n, k, bits, gs, 9)
    ids = torch.arange(0, n, 7).to(DEV)
    for dt in (torch.float16, torch.float32):
        q = QLinear(w.to(DEV), s.to(dt).to(DEV), b.to(dt).to(DEV), gs=gs, bits=bits)
        got = affine.embed(ids, q)
        want = oaff.embed(ids.cpu().numpy(), w.numpy(), s.to(dt).float().numpy(), b.to(dt).float().numpy(), gs, bits)
        np.testing.assert_array_equal(got.float().cpu().numpy(), want)


def test_stored_layout_lane_matmul_gives_the_tiled_bits():
    for n, k in [(48, 5120), (1024, 5120), (5120, 6144)]:
        w = to_dev(*synthetic.raw_weight(n, k, 4, 64, 5 * n + k))
        q = qmm.pack(*w, 64)
        x = synthetic.activations(128, k, 2).to(DEV)
        for m in (1, 7, 16, 17, 64, 128):
            assert torch.equal(qmm.matmul(x[:m], q), lane.lane_matmul(x[:m], *w)), (n, k, m)


def test_row_blocks_and_stacks():
    k, gs = 2048, 64
    parts = [QLinear(*to_dev(*synthetic.raw_weight(n, k, 4, gs, n)), gs=gs) for n in (256, 128, 384)]
    whole = qmm_fast.tile(qmm_fast.stack(parts))
    x = synthetic.activations(9, k, 1).to(DEV)
    full = qmm_fast.matmul(x, whole)
    blocks = [qmm_fast.rows(whole, 0, 256), qmm_fast.rows(whole, 256, 384), qmm_fast.rows(whole, 384, 768)]
    assert torch.equal(qmm_fast.matmul_rows(x, blocks), full)                 # views on super-block boundaries
    odd = qmm_fast.rows(whole, 100, 300)                                       # a copy: rows 100..299
    sk = qmm.default_split(whole.n, k, gs)
    assert torch.equal(qmm.matmul(x, qmm_fast._q4(odd), sk=sk), full[:, 100:300])
    assert torch.equal(qmm_fast.matmul_partial(x, whole).to(torch.bfloat16), full)
    with pytest.raises(ValueError):
        qmm_fast.stack([whole])


def test_refusals():
    q = QLinear(torch.zeros((4, 16), dtype=torch.int32, device=DEV), torch.zeros((4, 2), dtype=torch.bfloat16, device=DEV),
                torch.zeros((4, 2), dtype=torch.bfloat16, device=DEV))
    with pytest.raises(ValueError):
        affine.matmul(torch.zeros((2, 64), dtype=torch.bfloat16, device=DEV), q)           # wrong K
    with pytest.raises(ValueError):
        affine.matmul(torch.zeros((2, 128), dtype=torch.float32, device=DEV), q)           # not bf16
    dense = QLinear(torch.zeros((4, 128), dtype=torch.bfloat16, device=DEV), None, None, layout="dense")
    with pytest.raises(ValueError):
        affine.matmul(torch.zeros((2, 128), dtype=torch.bfloat16, device=DEV), dense)
