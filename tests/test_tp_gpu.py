"""Tensor- and expert-parallel layers on one GPU: the shards of every rank are run in turn and reduced in rank order, which
is what the ranks of a box compute (the collectives themselves are covered by the gloo tests and the multi-GPU run)."""

import numpy as np
import pytest
import torch

from oracle import affine as oaff
from tensorfold_b200 import synthetic
from tensorfold_b200.cuda import experts, moe, tp
from tensorfold_b200.cuda.kernels import qmm
from tensorfold_b200.families.qwen3_5.cuda import distributed
from tensorfold_b200.families.qwen3_5.cuda.weights import QLinear

from gpu_util import DEV, assert_close_bf16, oracle_f64, to_dev

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_parallel_partials_sum_to_the_projection(world):
    n, k, gs = 1024, 8192, 64                                   # o_proj-like: K splits into whole groups a rank
    w = synthetic.affine_weight(n, k, 4, gs, seed=world)
    q = QLinear(*to_dev(*w), gs=gs)
    x = synthetic.activations(24, k, 1)
    xd = x.to(DEV)
    parts = []
    for r in range(world):
        lin = tp.RowParallelLinear.shard(q, r, world)
        parts.append(lin.partial(distributed.local_input(xd, r, world, group_size=gs), f32=True))
    y = distributed.sum_rank_partials(parts)
    assert_close_bf16(y, oracle_f64(x, *w, gs, 4), f"world {world}")
    alone = [tp.RowParallelLinear.shard(q, r, world).partial(distributed.local_input(xd[5:6], r, world, group_size=gs), f32=True)
             for r in range(world)]
    assert torch.equal(distributed.sum_rank_partials(alone), y[5:6])            # a row's bits ignore the row count
    bf = distributed.sum_rank_partials([p.to(torch.bfloat16) for p in parts])    # bf16 partials (prefill): fp32 adds
    want = oaff.sum_rank_partials([p.to(torch.bfloat16).float().cpu().numpy() for p in parts])
    assert torch.equal(bf.float().cpu(), torch.from_numpy(want))


@pytest.mark.parametrize("world", [2, 4])
def test_column_parallel_rows_are_the_projections_rows(world):
    n, k, gs = 1024, 2048, 64
    w = synthetic.affine_weight(n, k, 4, gs, seed=7)
    q = QLinear(*to_dev(*w), gs=gs)
    x = synthetic.activations(8, k, 2).to(DEV)
    ref = oracle_f64(x.cpu(), *w, gs, 4)
    for r in range(world):
        y = tp.ColumnParallelLinear.shard(q, r, world).forward(x)
        rows = distributed.output_rows(n, r, world).numpy()
        assert_close_bf16(y, ref[:, rows], f"rank {r}")


@pytest.mark.parametrize("world,prefill", [(1, False), (2, False), (4, False), (4, True)])
def test_expert_parallel_partials_sum_to_the_layer(world, prefill):
    d, e, ni, gs, top_k, rows = 512, 16, 128, 64, 4, 19
    g = torch.Generator().manual_seed(3)
    stackw = lambda n, k, s: tuple(torch.stack([synthetic.affine_weight(n, k, 4, gs, seed=s * 100 + i)[j] for i in range(e)]) for j in range(3))
    gate, up, down = stackw(ni, d, 1), stackw(ni, d, 2), stackw(d, ni, 3)
    wr = (torch.randn((e, d), generator=g) * 0.05).to(torch.bfloat16)
    x = synthetic.activations(rows, d, 4).to(DEV)
    dev = lambda m: tuple(t.to(DEV) for t in m)
    parts = []
    for r in range(world):
        lu, ld, first = tp.shard_experts([gate, up], down, r, world)
        layer = tp.ExpertParallelMoE(wr.to(DEV), experts.make([dev(m) for m in lu], dev(ld), gs), top_k, first, e)
        parts.append(layer.partial(x, layer.buffers(rows, DEV, prefill=prefill)))
    got = distributed.sum_rank_partials(parts)
    # oracle: the whole layer on the host
    from oracle import moe as omoe
    npz = lambda m: tuple(t.numpy() if t.dtype == torch.int32 else t.float().numpy() for t in m)
    xf = x.float().cpu().numpy()
    logits = omoe.router_logits(xf, wr.float().numpy())
    picks, wts = omoe.select_rows(np.concatenate([logits, np.zeros((rows, 1), np.float32)], 1), top_k, e, shared=True)
    _, y = omoe.expert_pairs(xf, picks[:, :top_k], npz(gate), npz(up), npz(down), gs)
    ref = (wts[:, :top_k, None].astype(np.float64) * y.reshape(rows, top_k, d)).sum(1)
    assert np.abs(got.float().cpu().numpy() - ref).max() <= 2 ** -6 * np.abs(ref).max()
    if world > 1 and not prefill:
        one = tp.ExpertParallelMoE(wr.to(DEV), experts.make([dev(gate), dev(up)], dev(down), gs), top_k, 0, e)
        whole = one.partial(x, one.buffers(rows, DEV)).float()
        assert (got.float() - whole).abs().max() <= 2 ** -6 * whole.abs().max()


def test_forward_hands_unrounded_partials_to_the_reduction(monkeypatch):
    """``RowParallelLinear.forward`` with its defaults: the partial that meets the other ranks' is fp32 and the result is
    the rank-ordered sum rounded once, the bits ``sum_rank_partials`` gives for the fp32 partials."""

    n, k, gs, world = 512, 4096, 64, 2
    q = QLinear(*to_dev(*synthetic.affine_weight(n, k, 4, gs, seed=11)), gs=gs)
    x = synthetic.activations(9, k, 3).to(DEV)
    lins = [tp.RowParallelLinear.shard(q, r, world) for r in range(world)]
    xs = [distributed.local_input(x, r, world, group_size=gs) for r in range(world)]
    theirs = lins[1].partial(xs[1])
    assert theirs.dtype == torch.float32
    seen = []

    def two_ranks(local, group=None, dtype=torch.bfloat16):      # rank 0's view of the reduction: its partial, then rank 1's
        seen.append(local)
        return distributed.sum_rank_partials([local, theirs], dtype)

    monkeypatch.setattr(tp, "ordered_all_reduce", two_ranks)
    got = lins[0].forward(xs[0])
    assert seen[0].dtype == torch.float32
    assert torch.equal(got, distributed.sum_rank_partials([lins[0].partial(xs[0], f32=True), theirs]))
    rounded = distributed.sum_rank_partials([lins[0].partial(xs[0], f32=False), lins[1].partial(xs[1], f32=False)])
    assert got.dtype == rounded.dtype == torch.bfloat16        # the bf16-partial form stays an explicit option
