"""The benchmark configurations at their full shapes, each against the CPU oracle on the same seeded inputs and through
the size-independent properties the kernels promise (a row's bits ignore the row count and the chunk):

* a single 4096 -> 4096 4-bit/g64 matmul at M = 4 (seed 0);
* the dense-27B projections at M = 2048 in the prefill arithmetic (the decode arithmetic at M = 1..2048 is in
  test_dense27b_gpu.py);
* the routed layer (hidden 2688, 128 experts of width 1856, top 6, shared width 3712) at M = 2048 in prefill form;
* the mixed-width sweep on 4096 -> 14336: widths 2, 3, 5, 6, 8 and groups 32, 64, 128 at M = 1 and 16;
* the tensor-parallel MoE block (hidden 6144, 160 experts of width 1536, top 8, o_proj 8192 -> 6144) split over 8
  ranks, the ranks run in turn on one GPU and reduced in rank order, at M = 16 and M = 2048."""

import numpy as np
import pytest
import torch

from oracle import affine as oaff
from oracle import moe as omoe
from tensorfold_b200 import _lib, synthetic
from tensorfold_b200.cuda import experts, moe, tp
from tensorfold_b200.cuda.kernels import qmm
from tensorfold_b200.families.qwen3_5.cuda import distributed
from tensorfold_b200.families.qwen3_5.cuda.weights import QLinear

from gpu_util import DEV, assert_close_bf16, oracle_f64, to_dev

pytestmark = pytest.mark.gpu


def prefill_reference(x, words, scales, biases, gs):
    """float64 x @ bf16(q * s + b).T: the prefill contract rounds the weight once to bf16 (cuda/kernels/qmm.py:160-171)."""

    w = oaff.dequantize(words.numpy(), scales.float().numpy(), biases.float().numpy(), 4, gs)
    w = oaff.bf16_round(w.astype(np.float32)).astype(np.float64)
    return x.float().numpy().astype(np.float64) @ w.T


def test_single_matmul_4096_m4_seed0():
    n = k = 4096
    w = synthetic.affine_weight(n, k, 4, 64, seed=0)
    q = qmm.pack(*to_dev(*w), 64)
    x = synthetic.activations(4, k, 0)
    y = qmm.matmul(x.to(DEV), q)
    assert y.shape == (4, n) and y.dtype == torch.bfloat16
    assert_close_bf16(y, oracle_f64(x, *w, 64, 4), "4096x4096 M=4")
    for r in range(4):
        assert torch.equal(qmm.matmul(x[r:r + 1].to(DEV), q), y[r:r + 1])


@pytest.mark.parametrize("name", list(synthetic.DENSE_27B))
def test_dense27b_prefill_chunk_of_2048(name):
    n, k = synthetic.DENSE_27B[name]
    words, scales, biases = synthetic.affine_weight(n, k, 4, 64, seed=sum(map(ord, name)))
    q = qmm.pack(*to_dev(words, scales, biases), 64)
    x = synthetic.activations(2048, k, 1)
    xd = x.to(DEV)
    big = qmm.prefill_matmul(xd, q)
    assert big.shape == (2048, n)
    for a, b in ((0, 256), (1000, 1001), (1792, 2048)):          # any chunking of the prompt gives the same rows
        assert torch.equal(qmm.prefill_matmul(xd[a:b], q), big[a:b]), (name, a, b)
    # a bounded sample for the float64 oracle, in the prefill form's own arithmetic (weights rounded once to bf16)
    for rows, cols in ((slice(0, 16), slice(0, 1024)), (slice(2040, 2048), slice(n - 256, n))):
        ref = prefill_reference(x[rows], words[cols], scales[cols], biases[cols], 64)
        got = big[rows, cols].float().cpu().numpy()
        assert np.abs(got - ref).max() <= np.abs(ref).max() * 2 ** -7, (name, rows, cols)
    assert _lib.device_error(big) == 0


@pytest.mark.parametrize("bits", [2, 3, 5, 6, 8])
@pytest.mark.parametrize("gs", [32, 64, 128])
def test_mixed_width_sweep_4096_to_14336(bits, gs):
    n, k = 14336, 4096
    words, scales, biases = synthetic.affine_weight(n, k, bits, gs, seed=100 * bits + gs, centred=False)
    q = qmm.pack(*to_dev(words, scales, biases), gs, bits=bits)
    x = synthetic.activations(16, k, bits + gs)
    xd = x.to(DEV)
    y = qmm.matmul(xd, q)
    for r in (0, 7, 15):                                         # M = 1: the bits of the same row at M = 16
        assert torch.equal(qmm.matmul(xd[r:r + 1], q), y[r:r + 1]), (bits, gs, r)
    lo, hi = (0, 1024), (n - 512, n)                             # a bounded sample of columns: the first and the last
    for a, b in (lo, hi):
        ref = oracle_f64(x, words[a:b], scales[a:b], biases[a:b], gs, bits)
        assert_close_bf16(y[:, a:b], ref, f"{bits} bits, groups of {gs}, columns {a}:{b}")
    y1 = qmm.matmul(xd, q, f32=True)                             # linearity in x, exact in fp32
    assert torch.equal(qmm.matmul(xd * 2, q, f32=True), y1 * 2)
    assert _lib.device_error(y) == 0


def rolled(w, count, first=0):
    """``count`` distinct experts made by rolling one matrix's rows (cheap to make; the oracle sees the same tensors)."""

    return tuple(torch.stack([torch.roll(t, 7 * (first + i) + 1, 0) for i in range(count)]) for t in w)


def npz(m):
    return tuple(t.numpy() if t.dtype == torch.int32 else t.float().numpy() for t in m)


def test_routed_layer_at_2048_rows_in_prefill_form():
    d, e, ni, sni, gs, top_k = 2688, 128, 1856, 3712, 64, 6
    g = torch.Generator().manual_seed(11)
    one = lambda n, k, s: synthetic.affine_weight(n, k, 4, gs, seed=s)
    gate, up, down = rolled(one(ni, d, 1), e), rolled(one(ni, d, 2), e), rolled(one(d, ni, 3), e)
    sg, su, sd = one(sni, d, 4), one(sni, d, 5), one(d, sni, 6)
    wr = (torch.randn((e + 1, d), generator=g) * 0.05).to(torch.bfloat16)
    dev = lambda m: tuple(t.to(DEV) for t in m)
    layer = moe.Routed(wr.to(DEV), experts.make([dev(gate), dev(up)], dev(down), gs), top_k,
                       moe.SharedExpert(qmm.pack_pair(dev(sg), dev(su), gs), qmm.pack(*dev(sd), gs)))
    x = synthetic.activations(2048, d, 3)
    big = moe.run(x.to(DEV), layer, prefill=True)
    assert big.shape == (2048, d)
    for a, b in ((0, 7), (1023, 1024), (1900, 2048)):            # rows route and run on their own
        assert torch.equal(moe.run(x[a:b].to(DEV), layer, prefill=True), big[a:b]), (a, b)
    from test_moe_gpu import oracle_layer

    ref, _ = oracle_layer(x[:3], (wr, gate, up, down, sg, su, sd), gs, top_k)
    assert np.abs(big[:3].float().cpu().numpy() - ref).max() <= 2 ** -6 * np.abs(ref).max()
    assert _lib.device_error(big) == 0


@pytest.mark.parametrize("rows", [16, 2048])
def test_tensor_parallel_moe_block_over_eight_ranks(rows):
    d, e, ni, top_k, ko, gs, world = 6144, 160, 1536, 8, 8192, 64, 8
    prefill = rows > 128
    g = torch.Generator().manual_seed(21)
    one = lambda n, k, s: synthetic.affine_weight(n, k, 4, gs, seed=s)
    base = [one(ni, d, 1), one(ni, d, 2), one(d, ni, 3)]
    wr = (torch.randn((e, d), generator=g) * 0.05).to(torch.bfloat16)
    wo = one(d, ko, 30)
    attn = synthetic.activations(rows, ko, 50)
    dev = lambda m: tuple(t.to(DEV) for t in m)

    # attention output projection, inputs split in whole groups.  Decode: fp32 partials, rank-ordered fp32 adds, one
    # rounding (the reference's decode form).  Prompt pass: bf16 partials added in fp32 (its prefill form,
    # families/qwen3_5/cuda/prefill.py:36-41): eight roundings of partials, so the bound is on the absolute error only.
    o_full = QLinear(*dev(wo), gs=gs)
    parts = []
    for r in range(world):
        lin = tp.RowParallelLinear.shard(o_full, r, world)
        x_local = distributed.local_input(attn.to(DEV), r, world, group_size=gs)
        parts.append(qmm.prefill_matmul(x_local, lin.q) if prefill else lin.partial(x_local))
    assert parts[0].dtype == (torch.bfloat16 if prefill else torch.float32)
    h = distributed.sum_rank_partials(parts)
    ref_h = oracle_f64(attn[:4], *wo, gs, 4)
    if prefill:
        assert np.abs(h[:4].float().cpu().numpy() - ref_h).max() <= 2 ** -6 * np.abs(ref_h).max()
    else:
        assert_close_bf16(h[:4], ref_h, "o_proj over 8 ranks")

    # the experts, 20 a rank: every rank routes all rows, runs its own experts, contributes a partial [rows, d]
    parts = []
    for r in range(world):
        local = e // world
        gate, up, down = (rolled(w, local, r * local) for w in base)
        layer = tp.ExpertParallelMoE(wr.to(DEV), experts.make([dev(gate), dev(up)], dev(down), gs), top_k, r * local, e)
        parts.append(layer.partial(h, layer.buffers(rows, DEV, prefill=prefill)).clone())
        if r == 3:                                               # a few rows alone through one rank: the same bits
            alone = layer.partial(h[5:7], layer.buffers(2, DEV, prefill=prefill))
            assert torch.equal(alone, parts[-1][5:7])
    out = distributed.sum_rank_partials(parts)
    assert out.shape == (rows, d) and out.dtype == torch.bfloat16

    sample = 3                                                   # the float64 oracle on the first rows
    hf = h[:sample].float().cpu().numpy()
    logits = omoe.router_logits(hf, wr.float().numpy())
    picks, wts = omoe.select_rows(np.concatenate([logits, np.zeros((sample, 1), np.float32)], 1), top_k, e, shared=True)
    whole = [npz(rolled(w, e)) for w in base]
    _, y = omoe.expert_pairs(hf, picks[:, :top_k], *whole, gs)
    ref = (wts[:, :top_k, None].astype(np.float64) * y.reshape(sample, top_k, d)).sum(1)
    assert np.abs(out[:sample].float().cpu().numpy() - ref).max() <= 2 ** -6 * np.abs(ref).max()
    assert _lib.device_error(out) == 0
