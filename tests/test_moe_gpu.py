"""The routed-MoE layer on a B200 against the CPU oracle: router logits, top-k with renormalised weights and the
sigmoid-gated shared slot, slot-ordered combine, and the whole layer (routed table + a wider dense shared expert)."""

import numpy as np
import pytest
import torch

from oracle import affine as oaff
from oracle import moe as omoe
from tensorfold_b200 import _lib, synthetic
from tensorfold_b200.cuda import experts, moe
from tensorfold_b200.cuda.kernels import qmm

from gpu_util import DEV

pytestmark = pytest.mark.gpu


def expert_weights(e, n, k, gs, seed):
    ws = [synthetic.affine_weight(n, k, 4, gs, seed=seed * 1000 + i) for i in range(e)]
    return tuple(torch.stack([w[j] for w in ws]) for j in range(3))


def npz(m):
    return tuple(t.numpy() if t.dtype == torch.int32 else t.float().numpy() for t in m)


def test_router_and_topk_match_the_oracle():
    g = torch.Generator().manual_seed(3)
    rows, d, e, k = 33, 2688, 128, 6
    x = synthetic.activations(rows, d, 1)
    wr = (torch.randn((e + 1, d), generator=g) * 0.05).to(torch.bfloat16)
    logits = moe.router(x.to(DEV), wr.to(DEV))
    ref = omoe.router_logits(x.float().numpy(), wr.float().numpy())
    assert np.abs(logits.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()
    assert torch.equal(moe.router(x[5:6].to(DEV), wr.to(DEV)), logits[5:6])             # a row alone: same bits
    tiles = moe.router(x.to(DEV), wr.to(DEV), prefill=True)                              # tensor-core tiles: its own bits,
    assert np.abs(tiles.cpu().numpy() - ref).max() <= 1e-4 * np.abs(ref).max()          # ragged rows (33) and experts (129)
    assert torch.equal(moe.router(x[17:18].to(DEV), wr.to(DEV), prefill=True), tiles[17:18])
    assert torch.equal(moe.router(x[:32].to(DEV), wr[:16].to(DEV), prefill=True), tiles[:32, :16])
    wide = torch.zeros((rows, d + 2), dtype=torch.bfloat16)            # rows 4 bytes off the 16-byte grid: the kernel
    wide[:, :d] = x                                                    # that reads fragments straight from global memory
    assert torch.equal(moe.router(wide.to(DEV)[:, :d], wr.to(DEV), prefill=True), tiles)   # gives the staged kernel's bits

    class Cfg:
        num_experts_per_tok, num_experts, moe_intermediate_size, hidden_size = k, e, 64, 64
    buf = moe.MoEBuffers(rows, Cfg, DEV)
    lg = logits.clone()
    lg[0, 7] = lg[0, 3] = lg[0].max() + 1                      # a tie: the lower id wins slot 0
    moe.select_rows(lg, buf, k, e)
    picks, wts = omoe.select_rows(lg.cpu().numpy(), k, e, shared=True)
    assert buf.pick.cpu().numpy().tolist() == picks.tolist()
    assert buf.pick[0, 0] == 3 and buf.pick[0, 1] == 7
    # One bf16 spacing is allowed here and only here: the kernel's expf and NumPy's exp may differ in the last fp32 bit,
    # which moves the bf16 rounding of a quotient that sits within 2^-16 of a tie.  The rule itself (order, ties,
    # normalisation, roundings) is held to equality below, on the vectors made from the reference's kernel body.
    np.testing.assert_allclose(buf.wts.cpu().numpy(), wts, rtol=2 ** -7, atol=0)
    assert torch.equal(buf.wts, buf.wts.to(torch.bfloat16).float())                      # weights are bf16 values


def test_top_k_and_combine_equal_the_references_kernel_bodies(golden):
    """``tf_moe_topk`` and ``tf_moe_combine`` on the golden vectors (the reference's ``_topk_rows`` and ``_combine`` bodies
    run over NumPy): same experts in the same order, same bf16 weights, same combined rows, bit for bit."""

    rows, ne, top_k = map(int, golden["topk_case"])

    class Cfg:
        num_experts_per_tok, num_experts, moe_intermediate_size, hidden_size = top_k, ne, 64, 64
    buf = moe.MoEBuffers(rows, Cfg, DEV)
    moe.select_rows(torch.from_numpy(golden["topk_logits"]).to(DEV), buf, top_k, ne)
    assert buf.pick.cpu().numpy().tolist() == golden["topk_picks"].tolist()
    assert np.array_equal(buf.wts.cpu().numpy(), golden["topk_wts"])
    y, w = torch.from_numpy(golden["combine_y"]).to(DEV), torch.from_numpy(golden["combine_w"]).to(DEV)
    assert np.array_equal(moe.combine(y, w).float().cpu().numpy(), golden["combine_out"])


def test_combine_is_slot_ordered_fp32():
    g = torch.Generator().manual_seed(5)
    y = torch.randn((19, 7, 333), generator=g)
    w = torch.rand((19, 7), generator=g).to(torch.bfloat16).float()
    out = moe.combine(y.to(DEV), w.to(DEV))
    ref = omoe.combine(y.numpy(), w.numpy())
    assert np.abs(out.float().cpu().numpy() - ref).max() <= 2 ** -8 * np.abs(ref).max()
    out16 = moe.combine(y.to(torch.bfloat16).to(DEV), w.to(DEV))
    assert torch.equal(out16[3:4], moe.combine(y[3:4].to(torch.bfloat16).to(DEV), w[3:4].to(DEV)))
    w[:, 2] = 0                                                        # a slot that is skipped
    for dtype in (torch.float32, torch.bfloat16):                      # 336 columns: 16-byte loads; 337: the scalar kernel
        wide = torch.randn((19, 7, 337), generator=g).to(dtype)
        a = moe.combine(wide[:, :, :336].contiguous().to(DEV), w.to(DEV))
        b = moe.combine(wide.to(DEV), w.to(DEV))
        assert torch.equal(a, b[:, :336])


def layer(d, e, ni, shared_ni, gs, top_k, seed):
    """Routed table of e experts plus a dense shared expert of its own width (the benchmark's MoE layer in small)."""

    g = torch.Generator().manual_seed(seed)
    gate, up, down = expert_weights(e, ni, d, gs, seed), expert_weights(e, ni, d, gs, seed + 1), expert_weights(e, d, ni, gs, seed + 2)
    sg, su = synthetic.affine_weight(shared_ni, d, 4, gs, seed=seed + 50), synthetic.affine_weight(shared_ni, d, 4, gs, seed=seed + 51)
    sd = synthetic.affine_weight(d, shared_ni, 4, gs, seed=seed + 52)
    wr = (torch.randn((e + 1, d), generator=g) * 0.05).to(torch.bfloat16)
    dev = lambda m: tuple(t.to(DEV) for t in m)
    ex = experts.make([dev(gate), dev(up)], dev(down), gs)
    shared = moe.SharedExpert(qmm.pack_pair(dev(sg), dev(su), gs), qmm.pack(*dev(sd), gs))
    return moe.Routed(wr.to(DEV), ex, top_k, shared), (wr, gate, up, down, sg, su, sd)


def oracle_layer(x, raw, gs, top_k):
    wr, gate, up, down, sg, su, sd = raw
    e = wr.shape[0] - 1
    xf = x.float().numpy()
    logits = omoe.router_logits(xf, wr.float().numpy())
    picks, wts = omoe.select_rows(logits, top_k, e, shared=True)
    _, y = omoe.expert_pairs(xf, picks[:, :top_k], npz(gate), npz(up), npz(down), gs)
    y = y.reshape(x.shape[0], top_k, -1)
    g = oaff.quantized_matmul(xf, sg[0].numpy(), sg[1].float().numpy(), sg[2].float().numpy(), gs, 4)
    u = oaff.quantized_matmul(xf, su[0].numpy(), su[1].float().numpy(), su[2].float().numpy(), gs, 4)
    act = oaff.bf16_round(omoe.silu_mul(g.astype(np.float32), u.astype(np.float32)).astype(np.float32))
    ys = oaff.quantized_matmul(act, sd[0].numpy(), sd[1].float().numpy(), sd[2].float().numpy(), gs, 4)
    full = np.concatenate([y, ys[:, None, :]], axis=1)
    out = np.zeros((x.shape[0], full.shape[2]))
    for k in range(top_k + 1):
        out += wts[:, k, None].astype(np.float64) * full[:, k]
    return out, picks


@pytest.mark.parametrize("prefill", [False, True])
def test_layer_matches_the_oracle(prefill):
    d, e, ni, sni, gs, top_k = 512, 24, 192, 384, 64, 4
    m, raw = layer(d, e, ni, sni, gs, top_k, 7)
    x = synthetic.activations(21, d, 2)
    out = moe.run(x.to(DEV), m, prefill=prefill)
    ref, _ = oracle_layer(x, raw, gs, top_k)
    assert out.shape == (21, d) and out.dtype == torch.bfloat16
    assert np.abs(out.float().cpu().numpy() - ref).max() <= 2 ** -6 * np.abs(ref).max()
    for r in (0, 9, 20):                                        # a row alone routes and runs to the same bits
        assert torch.equal(moe.run(x[r:r + 1].to(DEV), m, prefill=prefill), out[r:r + 1]), r


def test_prompt_sized_layer_runs_many_tiles_a_block():
    """1200 rows, top 4 of 16 experts: about 50 plan items x 4 column blocks, more tiles than SMs, so the persistent
    prefill kernel runs several (item, column block) tiles a block.  Rows must keep the bits of a small call and the
    first rows must match the oracle."""

    d, e, ni, sni, gs, top_k = 512, 16, 256, 512, 64, 4
    m, raw = layer(d, e, ni, sni, gs, top_k, 19)
    x = synthetic.activations(1200, d, 4)
    out = moe.run(x.to(DEV), m, prefill=True)
    for a, b in ((0, 5), (600, 601), (1100, 1200)):
        assert torch.equal(moe.run(x[a:b].to(DEV), m, prefill=True), out[a:b]), (a, b)
    ref, _ = oracle_layer(x[:6], raw, gs, top_k)
    assert np.abs(out[:6].float().cpu().numpy() - ref).max() <= 2 ** -6 * np.abs(ref).max()
    assert _lib.device_error(out) == 0


def test_benchmark_moe_layer_shapes_rows_are_bit_stable():
    """Hidden 2688, 128 experts of width 1856, top 6, shared width 3712 (group 64): rows of a 16-row call keep their bits
    inside a 256-row call; the first rows are checked against the oracle."""

    d, e, ni, sni, gs, top_k = 2688, 128, 1856, 3712, 64, 6
    g = torch.Generator().manual_seed(11)
    one = lambda n, k, s: synthetic.affine_weight(n, k, 4, gs, seed=s)
    rep = lambda w: tuple(torch.stack([torch.roll(t, i, 0) for i in range(e)]) for t in w)   # distinct experts, cheap to make
    gate, up, down = rep(one(ni, d, 1)), rep(one(ni, d, 2)), rep(one(d, ni, 3))
    sg, su, sd = one(sni, d, 4), one(sni, d, 5), one(d, sni, 6)
    wr = (torch.randn((e + 1, d), generator=g) * 0.05).to(torch.bfloat16)
    dev = lambda m: tuple(t.to(DEV) for t in m)
    ex = experts.make([dev(gate), dev(up)], dev(down), gs)
    m = moe.Routed(wr.to(DEV), ex, top_k, moe.SharedExpert(qmm.pack_pair(dev(sg), dev(su), gs), qmm.pack(*dev(sd), gs)))
    x = synthetic.activations(256, d, 3)
    big = moe.run(x.to(DEV), m)
    small = moe.run(x[:16].to(DEV), m)
    assert torch.equal(small, big[:16])
    ref, _ = oracle_layer(x[:3], (wr, gate, up, down, sg, su, sd), gs, top_k)
    assert np.abs(big[:3].float().cpu().numpy() - ref).max() <= 2 ** -6 * np.abs(ref).max()
