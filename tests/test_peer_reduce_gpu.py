"""The one-launch reduction over peer memory (tf_peer_reduce).  On one GPU the ranks' buffers all live on this device and
their flags are set beforehand as if every other rank had long arrived, so each rank's launch runs alone and in turn:
that checks the arithmetic and the addressing of both forms against ``sum_rank_partials``.  The flags' protocol between
processes runs in ``peer_worker.py`` on two or more GPUs (skipped on a box with one)."""

import json
import os
import subprocess
import sys

import pytest
import torch

from tensorfold_b200 import _lib
from tensorfold_b200.cuda import tp
from tensorfold_b200.families.qwen3_5.cuda import distributed

from gpu_util import DEV

pytestmark = pytest.mark.gpu
R = tp.PeerReducer


def local_ranks(world, elements):
    """``world`` reducers over buffers of this one device; every flag another rank would raise is already far ahead."""

    _lib.check(_lib.lib().tf_init(torch.cuda.current_device()), "init")
    bufs = [tp.PeerReducer.alloc(tp.PeerReducer.layout(elements, world)[-1]) for _ in range(world)]
    ranks = [tp.PeerReducer(elements, bufs=bufs, rank=r, device=DEV) for r in range(world)]
    for red in ranks:
        flags = red._mine[:red.flags].view(torch.int32).view(-1, 32)
        flags[:16, 0] = 1 << 20                                  # ready[0..7], done[0..7]
    torch.cuda.synchronize()
    return ranks, bufs


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("part_dtype", [torch.float32, torch.bfloat16])
def test_both_forms_give_the_rank_ordered_sum(world, part_dtype):
    shape = (24, 1024)
    ranks, bufs = local_ranks(world, shape[0] * shape[1])
    try:
        g = torch.Generator().manual_seed(world)
        parts = [(torch.randn(shape, generator=g) * 3).to(part_dtype).to(DEV) for _ in range(world)]
        for out_dtype in (torch.bfloat16, torch.float32):
            want = distributed.sum_rank_partials(parts, out_dtype)
            forms = (R.ALL, R.SHARES, R.FLAGGED) + ((R.HOPS,) if world >= 4 else ())
            for form in forms:             # every rank sums all; a rank sums its share for all; flagged words in one hop, in two
                outs = []
                for r, red in enumerate(ranks):
                    red.partial(shape, part_dtype).copy_(parts[r])
                    red._view(red.out_off, shape, out_dtype).zero_()
                torch.cuda.synchronize()
                halves = {R.FLAGGED: (R.FLAGGED_PUSH, R.FLAGGED_PULL), R.HOPS: (R.HOPS_SEND, R.HOPS_MIDDLE, R.HOPS_COLLECT)}.get(form, (form,))
                for half in halves:                              # all ranks store their words before any rank collects
                    for red in ranks:
                        red.force = half
                        out = red.reduce(red.partial(shape, part_dtype), out_dtype, grid_cap=3 if form == R.ALL else 0)
                        if half == halves[-1]:
                            outs.append(out)
                torch.cuda.synchronize()
                for r, o in enumerate(outs):
                    assert torch.equal(o, want), (world, part_dtype, out_dtype, form, r)
        assert _lib.device_error(parts[0]) == 0
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            _lib.lib().tf_peer_free(b)


def test_bulk_copies_and_plain_loads_give_the_same_sums():
    """The share form brings the partials in with bulk copies where a share splits into 4 KB pieces; with the tuning
    switch it uses plain loads.  Same additions in the same order: same bits."""

    world, shape = 4, (64, 1024)
    ranks, bufs = local_ranks(world, shape[0] * shape[1])
    try:
        g = torch.Generator().manual_seed(9)
        for part_dtype in (torch.bfloat16, torch.float32):
            parts = [(torch.randn(shape, generator=g) * 3).to(part_dtype).to(DEV) for _ in range(world)]
            got = {}
            for plain in (0, 1):
                _lib.check(_lib.lib().tf_tune(b"peer_plain", plain), "tune")
                for r, red in enumerate(ranks):
                    red.force = R.SHARES
                    red.partial(shape, part_dtype).copy_(parts[r])
                torch.cuda.synchronize()
                outs = [red.reduce(red.partial(shape, part_dtype), torch.bfloat16) for red in ranks]
                torch.cuda.synchronize()
                got[plain] = outs[0].clone()
                assert all(torch.equal(o, outs[0]) for o in outs)
            assert torch.equal(got[0], got[1])
            assert torch.equal(got[0], distributed.sum_rank_partials(parts))
        assert _lib.device_error(parts[0]) == 0
    finally:
        _lib.lib().tf_tune(b"peer_plain", 0)
        torch.cuda.synchronize()
        for b in bufs:
            _lib.lib().tf_peer_free(b)


def test_a_missing_peer_ends_the_wait_with_an_error():
    """Rank 1 never calls: rank 0's launch gives up after its poll limit, reports error 4 and leaves the context usable."""

    _lib.check(_lib.lib().tf_init(torch.cuda.current_device()), "init")
    n = 4096
    bufs = [tp.PeerReducer.alloc(tp.PeerReducer.layout(n, 2)[-1]) for _ in range(2)]
    try:
        red = tp.PeerReducer(n, bufs=bufs, rank=0, device=DEV)
        red.partial((n,), torch.float32).fill_(1.0)
        for form in (R.SHARES, R.FLAGGED):                       # a barrier that no one joins; words that never come
            red.force = form
            red.reduce(red.partial((n,), torch.float32), polls=2000)
            torch.cuda.synchronize()
            assert _lib.device_error(red._mine) == 4, form
        x = torch.ones((8,), device=DEV)
        assert float((x + x).sum()) == 16.0                      # the context still works
        assert _lib.device_error(red._mine) == 0                 # read and cleared
    finally:
        for b in bufs:
            _lib.lib().tf_peer_free(b)


def refused(**kw):
    import ctypes
    bufs = [tp.PeerReducer.alloc(1 << 20) for _ in range(2)]
    try:
        args = dict(rank=0, world=2, part_off=4096, out_off=4096 + (1 << 18), total=4096, parts_bf16=0, out_f32=0, mode=0,
                    ll_off=1 << 19, ll_slot=1 << 15)
        args.update(kw)
        table = (ctypes.c_void_p * 2)(*bufs)
        return _lib.lib().tf_peer_reduce(table, args["rank"], args["world"], args["part_off"], args["out_off"], args["total"],
                                         args["parts_bf16"], args["out_f32"], args["mode"], args["ll_off"], args["ll_slot"], 10, 0,
                                         None)
    finally:
        for b in bufs:
            _lib.lib().tf_peer_free(b)


def test_bad_arguments_launch_nothing():
    _lib.check(_lib.lib().tf_init(torch.cuda.current_device()), "init")
    assert refused(world=3) < 0 and refused(rank=2) < 0 and refused(total=4) < 0 and refused(total=4100) < 0
    assert refused(part_off=0) < 0 and refused(part_off=4104) < 0
    assert refused(out_off=4096 + 1024) < 0                       # the result would overlap the partial
    assert refused(total=4104, mode=1) < 0                        # does not split into pieces of eight a rank
    assert refused(mode=9) < 0 and refused(mode=2, ll_slot=1 << 14) < 0 and refused(mode=2, ll_off=4096) < 0
    assert refused(mode=5) < 0                                    # two hops need four ranks
    torch.cuda.synchronize()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_ranks_in_their_own_processes_agree_with_the_collectives():
    world = min(8, 1 << (torch.cuda.device_count().bit_length() - 1))
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    done = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(here, "peer_worker.py")],
                          capture_output=True, text=True, timeout=600, env=env)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    line = [l for l in done.stdout.splitlines() if l.startswith("{")][-1]
    report = json.loads(line)
    assert report["equal"] and report["errors"] == 0, report
