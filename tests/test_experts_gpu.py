"""Grouped-expert kernels on a B200 against the CPU oracle: a pair's bits ignore the call's other rows; outputs track
float64; the plan equals a Python counting sort.  Mirrors the reference's tests/cuda/test_experts.py."""

import numpy as np
import pytest
import torch

from oracle import moe as omoe
from tensorfold_b200 import synthetic
from tensorfold_b200.cuda import experts

from gpu_util import DEV

pytestmark = pytest.mark.gpu

# (group size, SwiGLU, limit, experts incl. shared, D, NI, shared slots): three families in small
CASES = [(32, True, 0.0, 41, 256, 96, 1), (64, True, 10.0, 19, 512, 128, 1), (64, False, 0.0, 12, 384, 192, 2)]


def mlx(e, n, k, gs, seed):
    g = torch.Generator().manual_seed(seed)
    words = torch.randint(-(2 ** 31), 2 ** 31 - 1, (e, n, k // 8), generator=g, dtype=torch.int64).to(torch.int32)
    scales = (torch.rand((e, n, k // gs), generator=g) * 0.02 + 0.001).to(torch.bfloat16)
    biases = (torch.randn((e, n, k // gs), generator=g) * 0.02).to(torch.bfloat16)
    return words, scales, biases


def build(case, seed):
    gs, swiglu, limit, e, d, ni, _ = case
    up = [mlx(e, ni, d, gs, seed + i) for i in range(2 if swiglu else 1)]
    down = mlx(e, d, ni, gs, seed + 7)
    dev = lambda m: tuple(t.to(DEV) for t in m)
    return experts.make([dev(m) for m in up], dev(down), gs, limit=limit), up, down


def picks_for(rows, case, seed, *, hot=None):
    _, _, _, e, _, _, shared = case
    routed = e - shared
    k = min(6, routed)
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(rows):
        r = torch.arange(k) if hot is not None else torch.randperm(routed, generator=g)[:k]
        out.append(torch.cat([r, torch.arange(routed, e)]))
    return torch.stack(out).to(torch.int32).to(DEV)


def run(ex, x, picks, *, prefill=False, y_dtype=torch.float32):
    rows, slots = picks.shape
    plan = experts.Plan(rows, slots, ex.count, DEV, prefill=prefill)
    experts.route(picks.contiguous(), plan)
    act = torch.empty((rows * slots, ex.width), dtype=torch.bfloat16, device=DEV)
    y = torch.empty((rows * slots, ex.dims), dtype=y_dtype, device=DEV)
    experts.gate_up(x, ex, plan, act, rows)
    experts.down(act, ex, plan, y, rows)
    return act, y, plan


@pytest.mark.parametrize("gs", [32, 64])
def test_pack_round_trip(gs):
    w = tuple(t.to(DEV) for t in mlx(3, 96, 256, gs, 61))
    back = experts.unpack(experts.pack(*w, gs), gs, 96)
    assert all(torch.equal(a, b) for a, b in zip(back, w))
    u = tuple(t.to(DEV) for t in mlx(3, 96, 256, gs, 62))
    g2, u2 = experts.unpack_pair(experts.pack_pair(w, u, gs), gs, 96)
    assert all(torch.equal(a, b) for a, b in zip(g2, w)) and all(torch.equal(a, b) for a, b in zip(u2, u))


@pytest.mark.parametrize("case", CASES)
def test_pairs_do_not_depend_on_the_window(case):
    ex, _, _ = build(case, 11)
    rows = 40
    x = synthetic.activations(rows, ex.dims, 1, std=0.5).to(DEV)
    picks = picks_for(rows, case, 3)
    slots = picks.shape[1]
    act, y, _ = run(ex, x, picks)
    alone = [run(ex, x[r:r + 1], picks[r:r + 1]) for r in range(rows)]
    assert torch.equal(act, torch.cat([a[0] for a in alone])) and torch.equal(y, torch.cat([a[1] for a in alone]))
    for m in (2, 3, 8, 9, 16, 17, 33):
        a_m, y_m, _ = run(ex, x[:m], picks[:m])
        assert torch.equal(a_m, act[:m * slots]) and torch.equal(y_m, y[:m * slots]), m
    perm = torch.randperm(rows, generator=torch.Generator().manual_seed(5)).to(DEV)
    a_p, y_p, _ = run(ex, x[perm], picks[perm])
    idx = (perm[:, None] * slots + torch.arange(slots, device=DEV)).reshape(-1)
    assert torch.equal(a_p, act[idx]) and torch.equal(y_p, y[idx])


@pytest.mark.parametrize("case", CASES)
def test_an_expert_shared_by_many_rows(case):
    """Every row picks the same experts: items of 16 pairs, several an expert, same bits as alone."""

    ex, _, _ = build(case, 21)
    rows = 37
    x = synthetic.activations(rows, ex.dims, 2, std=0.5).to(DEV)
    picks = picks_for(rows, case, 4, hot=0)
    _, y, plan = run(ex, x, picks)
    slots = picks.shape[1]
    alone = torch.cat([run(ex, x[r:r + 1], picks[r:r + 1])[1] for r in range(rows)])
    assert torch.equal(y, alone)
    assert int(plan.counts[1]) == slots
    assert int(plan.counts[0]) == slots * 3                    # 37 pairs an expert: items of 16, 16 and 5


@pytest.mark.parametrize("rows,prefill", [(23, False), (23, True), (300, False), (300, True), (1500, True)])
def test_plan_groups_pairs_by_expert(rows, prefill):
    slots, e = 7, 50
    g = torch.Generator().manual_seed(9)
    picks = torch.stack([torch.randperm(e, generator=g)[:slots] for _ in range(rows)]).to(torch.int32)
    picks[:, 0] = 3                                            # one expert with a pair in every row
    plan = experts.Plan(rows, slots, e, DEV, prefill=prefill)
    experts.route(picks.to(DEV), plan)
    want_items, want_members, distinct = omoe.plan(picks.numpy(), e, plan.tile)
    n = int(plan.counts[0])
    assert n == len(want_items) and int(plan.counts[1]) == distinct
    assert plan.items[:n].cpu().tolist() == want_items.tolist()
    assert plan.members.cpu().tolist() == want_members.tolist()


def test_plan_equals_the_references_expected_plan(golden):
    """The plan kernel against the plans the reference's own test expects (golden vectors made from its ``want_plan``)."""

    for tag in "abc":
        rows, slots, e, tile, distinct = map(int, golden[f"plan_{tag}_case"])
        picks = torch.from_numpy(golden[f"plan_{tag}_picks"]).to(torch.int32)
        plan = experts.Plan(rows, slots, e, DEV, prefill=False)
        plan.tile = tile
        plan.items = torch.zeros((experts.max_items(rows * slots, e, tile), 3), dtype=torch.int32, device=DEV)
        experts.route(picks.to(DEV), plan)
        n = int(plan.counts[0])
        assert n == len(golden[f"plan_{tag}_items"]) and int(plan.counts[1]) == distinct
        assert plan.items[:n].cpu().tolist() == golden[f"plan_{tag}_items"].tolist()
        assert plan.members.cpu().tolist() == golden[f"plan_{tag}_members"].tolist()


@pytest.mark.parametrize("prefill", [False, True])
@pytest.mark.parametrize("case", CASES)
def test_matches_fp64(case, prefill):
    """Against float64 over the dequantized weights (rounded to bf16 first for the prefill form): activations within 2^-6, the fp32 down projection within 1e-5
    of the largest value (tests/cuda/test_experts.py:136-165)."""

    gs, swiglu, limit = case[0], case[1], case[2]
    ex, up, down = build(case, 31)
    rows = 5
    x = synthetic.activations(rows, ex.dims, 3, std=0.5)
    picks = picks_for(rows, case, 6)
    act, y, _ = run(ex, x.to(DEV), picks, prefill=prefill)
    npz = lambda m: tuple(t.numpy() if t.dtype == torch.int32 else t.float().numpy() for t in m)
    if swiglu:
        ref_act, ref_y = omoe.expert_pairs(x.float().numpy(), picks.cpu().numpy(), npz(up[0]), npz(up[1]), npz(down), gs, limit,
                                           weight_bf16=prefill)
    else:
        ref_act, ref_y = omoe.expert_pairs_relu2(x.float().numpy(), picks.cpu().numpy(), npz(up[0]), npz(down), gs,
                                                 weight_bf16=prefill)
    assert np.abs(act.float().cpu().numpy() - ref_act).max() <= 2 ** -6 * np.abs(ref_act).max()
    # y is computed from the device's own bf16 activations so the down projection is judged alone
    yref = omoe.down_pairs(act.float().cpu().numpy(), picks.cpu().numpy(), npz(down), gs, weight_bf16=prefill)
    assert np.abs(y.cpu().numpy() - yref).max() <= 1e-5 * np.abs(yref).max()


def test_graph_replay_follows_the_picks():
    case = CASES[1]
    ex, _, _ = build(case, 41)
    rows = 9
    picks = picks_for(rows, case, 7).contiguous()
    slots = picks.shape[1]
    plan = experts.Plan(rows, slots, ex.count, DEV)
    x = synthetic.activations(rows, ex.dims, 4, std=0.5).to(DEV)
    act = torch.empty((rows * slots, ex.width), dtype=torch.bfloat16, device=DEV)
    y = torch.empty((rows * slots, ex.dims), dtype=torch.float32, device=DEV)

    def step():
        experts.route(picks, plan)
        experts.gate_up(x, ex, plan, act, rows)
        experts.down(act, ex, plan, y, rows)

    step()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for seed in (8, 9):
        picks.copy_(picks_for(rows, case, seed))
        g.replay()
        _, want, _ = run(ex, x, picks)
        assert torch.equal(y, want)


@pytest.mark.parametrize("case", CASES)
def test_prefill_rows_do_not_depend_on_the_chunk(case):
    ex, _, _ = build(case, 71)
    rows = 200
    x = synthetic.activations(rows, ex.dims, 5, std=0.5).to(DEV)
    picks = picks_for(rows, case, 13)
    slots = picks.shape[1]
    assert rows * slots > experts.SMALL
    act, y, _ = run(ex, x, picks, prefill=True)
    for a, b in ((0, 1), (77, 78), (199, 200), (0, 7), (5, 22), (0, 64), (100, 200)):
        a1, y1, _ = run(ex, x[a:b], picks[a:b], prefill=True)
        assert torch.equal(a1, act[a * slots:b * slots]) and torch.equal(y1, y[a * slots:b * slots]), (a, b)
    perm = torch.randperm(rows, generator=torch.Generator().manual_seed(5)).to(DEV)
    a_p, y_p, _ = run(ex, x[perm], picks[perm], prefill=True)
    idx = (perm[:, None] * slots + torch.arange(slots, device=DEV)).reshape(-1)
    assert torch.equal(a_p, act[idx]) and torch.equal(y_p, y[idx])
    _, y16, _ = run(ex, x, picks, prefill=True, y_dtype=torch.bfloat16)
    assert torch.equal(y16, y.to(torch.bfloat16))
    a_d, y_d, _ = run(ex, x, picks, prefill=False)                      # the decode form: other bits, same values
    assert (a_d.float() - act.float()).abs().max() <= 2 ** -5 * act.float().abs().max()
    assert (y_d - y).abs().max() <= 2 ** -5 * y.abs().max()


def test_many_items_keep_the_bits():
    case = (64, True, 0.0, 257, 2048, 128, 1)
    ex, _, _ = build(case, 81)
    rows = 64
    x = synthetic.activations(rows, ex.dims, 6, std=0.5).to(DEV)
    g = torch.Generator().manual_seed(12)
    picks = torch.stack([torch.cat([torch.randperm(256, generator=g)[:8], torch.tensor([256])])
                         for _ in range(rows)]).to(torch.int32).to(DEV)
    _, y, plan = run(ex, x, picks)
    assert int(plan.counts[0]) >= 200
    for r in (0, 31, 63):
        assert torch.equal(run(ex, x[r:r + 1], picks[r:r + 1])[1], y[9 * r:9 * r + 9]), r


@pytest.mark.parametrize("case", CASES)
def test_persistent_and_tiled_kernels_give_the_same_pairs(case):
    """The decode form runs the persistent kernel's grouped mode; the tiled kernel (one block an item and column block)
    stays behind a tuning switch.  Same arithmetic: every pair has the same bits through both, for items of 8 and of 16."""

    from tensorfold_b200 import _lib

    ex, _, _ = build(case, 31)
    rows = 29
    x = synthetic.activations(rows, ex.dims, 6, std=0.5).to(DEV)
    picks = picks_for(rows, case, 8)
    slots = picks.shape[1]
    results = {}
    try:
        for tiled in (0, 1):
            _lib.check(_lib.lib().tf_tune(b"grouped_tiled", tiled), "tune")
            for tile in (8, 16):
                plan = experts.Plan(rows, slots, ex.count, DEV)
                plan.tile = tile
                plan.items = torch.zeros((experts.max_items(rows * slots, ex.count, tile), 3), dtype=torch.int32, device=DEV)
                experts.route(picks.contiguous(), plan)
                act = torch.zeros((rows * slots, ex.width), dtype=torch.bfloat16, device=DEV)
                y = torch.zeros((rows * slots, ex.dims), dtype=torch.float32, device=DEV)
                experts.gate_up(x, ex, plan, act, rows)
                experts.down(act, ex, plan, y, rows)
                results[(tiled, tile)] = (act, y)
    finally:
        _lib.lib().tf_tune(b"grouped_tiled", 0)
    first = results[(0, 8)]
    for key, (act, y) in results.items():
        assert torch.equal(act, first[0]) and torch.equal(y, first[1]), key
    assert _lib.device_error(x) == 0
