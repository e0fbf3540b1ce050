"""Host-side logic without a GPU: shard maps on CPU tensors, refusals, and the rank-ordered reduction over a
two-process gloo group (the N > 1 path of the tensor-parallel layers)."""

import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import affine as oaff
from tensorfold_b200 import synthetic
from tensorfold_b200.cuda.kernels import affine
from tensorfold_b200.families.qwen3_5.cuda import distributed
from tensorfold_b200.families.qwen3_5.cuda.weights import QLinear


def test_shapes_and_slices_match_the_oracle(golden):
    for bits, gs, rank, a, b, g0, g1 in golden["input_slice"].tolist():
        assert affine.input_slice(gs * 4, bits, gs, rank) == ((a, b), (g0, g1))
    with pytest.raises(ValueError):
        affine.input_slice(384, 5, 128, 0)
    for bits, gs, shape in [(1, 64, (4, 16)), (8, 16, (4, 64)), (3, 32, (4, 4))]:
        with pytest.raises(ValueError):
            affine.packed_shape(shape, (4, 2), (4, 2), bits, gs)
    assert affine.packed_shape((5, 24), (5, 4), (5, 4), 3, 64) == (5, 256)
    for world in (4, 8):
        for rank in range(world):
            assert affine.input_slice(8192, 4, 64, rank, world) == oaff.input_slice(8192, 4, 64, rank, world)


def test_partition_map_on_cpu_tensors(golden):
    assert distributed.output_rows(16, 1).tolist() == golden["rows_plain_r1"].tolist()
    assert distributed.output_rows(40, 0, segments=(8, 8, 24)).tolist() == golden["rows_seg_r0"].tolist()
    assert distributed.output_rows(32, 1, block=8).tolist() == golden["rows_block_r1"].tolist()
    words, scales, biases = synthetic.raw_weight(64, 512, 4, 64, 3)
    q = QLinear(words, scales, biases)
    for world in (2, 4, 8):
        cols = [distributed.split_output(q, r, world) for r in range(world)]
        assert torch.equal(torch.cat([c.weight for c in cols]), words)
        rows = [distributed.split_input(q, r, world) for r in range(world)]
        assert torch.equal(torch.cat([c.weight for c in rows], dim=1), words)
        assert torch.equal(torch.cat([c.scales for c in rows], dim=1), scales)
        full = oaff.dequantize(words.numpy(), scales.float().numpy(), biases.float().numpy(), 4, 64)
        part = oaff.dequantize(rows[1].weight.numpy(), rows[1].scales.float().numpy(), rows[1].biases.float().numpy(), 4, 64)
        np.testing.assert_array_equal(part, full[:, 512 // world:2 * 512 // world])     # values never change
    x = torch.arange(2 * 512, dtype=torch.float32).view(2, 512)
    assert torch.equal(distributed.local_input(x, 3, 4), x[:, 384:512])
    with pytest.raises(ValueError):
        distributed.split_output(q, 0, 3)
    with pytest.raises(ValueError):
        distributed.local_input(x, 0, 3)


def test_rank_sum_rounds_after_the_fp32_add(golden):
    p0, p1 = torch.from_numpy(golden["rank_p0"]), torch.from_numpy(golden["rank_p1"])
    got = distributed.sum_rank_partials([p0, p1])
    assert synthetic.bf16_bits(got).tolist() == golden["rank_sum_bf16"].tolist()
    four = [p0, p1, p0 * 0.5, p1 * 0.25]
    want = oaff.sum_rank_partials([p.numpy() for p in four])
    assert torch.equal(distributed.sum_rank_partials(four).float(), torch.from_numpy(want))


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        local = torch.randn((5, 33), generator=g) * 3
        summed = distributed.gather_rank_partials(local)
        torch.save((local, summed), f"{out}/r{rank}.pt")
    finally:
        dist.destroy_process_group()


def _head_worker(rank, world, port, out):
    from tensorfold_b200.cuda.comm import Comm
    from tensorfold_b200.families.qwen3_5.cuda import decode_tp

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        comm = Comm()
        g = torch.Generator().manual_seed(9)
        logits = torch.randn((5, 64 * world), generator=g)      # every rank draws the same full logits, keeps its columns
        logits[1, 3] = logits[1, 64 * world - 2] = 7.0          # a tie between the first and the last rank
        mine = logits[:, 64 * rank:64 * (rank + 1)]
        values, ids = decode_tp.gather_candidates(*decode_tp.split_candidates(mine, None, 64 * rank), comm)
        pick = decode_tp.greedy_merged(values, ids)
        s = decode_tp.Sampling(top_k=5)
        cv, ci = decode_tp.gather_candidates(*decode_tp.split_candidates(mine, s, 64 * rank), comm)
        comm.barrier()
        torch.save((logits, pick, cv, ci), f"{out}/h{rank}.pt")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_gather_head_candidates(tmp_path, world):
    port = 29650 + world + os.getpid() % 200
    mp.spawn(_head_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        logits, pick, cv, ci = torch.load(tmp_path / f"h{r}.pt")
        assert torch.equal(pick, logits.argmax(dim=-1)) and int(pick[1]) == 3
        assert cv.shape == (5, world * (5 + 8)) and torch.equal(logits.gather(1, ci), cv)
        want = torch.topk(logits, 5, dim=-1).indices
        assert all(set(want[i].tolist()) <= set(ci[i].tolist()) for i in range(5))


@pytest.mark.parametrize("world", [2, 4])
def test_gloo_ranks_agree_bit_for_bit_and_sum_in_rank_order(tmp_path, world):
    port = 29600 + world + os.getpid() % 200
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    got = [torch.load(tmp_path / f"r{r}.pt") for r in range(world)]
    want = oaff.sum_rank_partials([g[0].numpy() for g in got])
    for local, summed in got:
        assert torch.equal(summed.float(), torch.from_numpy(want))


def test_default_split_is_shape_only_and_fills_the_lanes_once():
    """(128-column block, slice) units fill the persistent kernel's 592 lanes once, never with slices shorter than six
    groups; projections launched as a set (gate and up) split by the set's blocks, so the SET fills the lanes once."""

    from tensorfold_b200.cuda.kernels import qmm

    assert qmm.default_split(17408, 5120) == 4 and qmm.default_split(17408, 5120, share=2) == 2
    assert qmm.default_split(5120, 17408) == 14 and qmm.default_split(5120, 6144) == 14
    assert qmm.default_split(248320, 5120) == 1 and qmm.default_split(128, 128) == 1
    for n, k in ((1024, 5120), (5120, 17408), (17408, 5120), (256, 512), (4096, 4096), (14336, 4096)):
        for share in (1, 2, 3, 4):
            sk = qmm.default_split(n, k, share=share)
            assert 1 <= sk <= qmm.default_split(n, k)
            assert sk == 1 or (k // 64) // sk >= 6
            assert -(-n // 128) * sk * share <= qmm.LANES or sk == 1


def test_decode_items_and_reduction_forms_follow_sizes_only():
    """Load-time choices that never change a bit: pairs an item of the decode plan holds, and the form a reduction takes."""

    from tensorfold_b200.cuda import experts, tp

    assert experts.decode_tile(96, 128) == 8 and experts.decode_tile(16 * 9, 161) == 8      # few pairs an expert
    assert experts.decode_tile(128 * 7, 128) == 16 and experts.decode_tile(513, 128) == 16
    assert experts.max_items(96, 128, 8) == 96 + 12 and experts.max_items(2048 * 7, 129, 128) == 129 + 112
    red = object.__new__(tp.PeerReducer)                       # the rule needs no buffers
    red.force, red.flagged_up_to = None, 1 << 19
    for world, n, itemsize, want in ((2, 16 * 6144, 4, tp.PeerReducer.FLAGGED), (8, 6144, 2, tp.PeerReducer.FLAGGED),
                                     (8, 16 * 6144, 4, tp.PeerReducer.HOPS), (4, 16 * 5120, 2, tp.PeerReducer.HOPS),
                                     (8, 2048 * 6144, 2, tp.PeerReducer.SHARES), (2, 256 * 6144, 2, tp.PeerReducer.SHARES),
                                     (8, 16 * 6144 + 8, 4, tp.PeerReducer.FLAGGED), (8, 2048 * 6144 + 8, 2, tp.PeerReducer.ALL)):
        red.world = world
        assert red.form(n, itemsize) == want, (world, n, itemsize)
