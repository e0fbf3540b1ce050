"""The plan entry point that brings its own scratch (``tf_moe_plan_static``) against the one that takes caller scratch.

Some hosts cannot allocate when they call the library: all device memory already belongs to their pools, or they may
only touch the tensors they were handed.  For them the plan can run on a small array built into the library.  This test
calls it through the C ABI twice in a row (the array keeps the first call's contents, which must not leak into the
second) and wants exactly the members, items and counts of ``tf_moe_plan``.  It is collected last on purpose."""

import pytest
import torch

from tensorfold_b200 import _lib
from tensorfold_b200.cuda import experts

pytestmark = pytest.mark.gpu
DEV = "cuda"


def plans(picks, e, tile, static):
    rows, slots = picks.shape
    pairs = rows * slots
    lib = _lib.lib()
    stream = _lib.stream_of(picks)
    members = torch.full((pairs,), -7, dtype=torch.int32, device=DEV)
    cap = experts.max_items(pairs, e, tile)
    items = torch.full((cap, 3), -7, dtype=torch.int32, device=DEV)
    counts = torch.full((2,), -7, dtype=torch.int32, device=DEV)
    if static:
        rc = lib.tf_moe_plan_static(picks.data_ptr(), pairs, e, tile, members.data_ptr(), items.data_ptr(), counts.data_ptr(),
                                    cap, stream)
    else:
        rank = torch.zeros((pairs,), dtype=torch.int32, device=DEV)
        hist = torch.zeros((lib.tf_moe_plan_blocks(pairs) * e,), dtype=torch.int32, device=DEV)
        rc = lib.tf_moe_plan(picks.data_ptr(), pairs, e, tile, members.data_ptr(), items.data_ptr(), counts.data_ptr(),
                             rank.data_ptr(), hist.data_ptr(), cap, stream)
    _lib.check(rc, "plan")
    torch.cuda.synchronize()
    n = int(counts[0])
    return members.cpu(), items[:n].cpu(), counts.cpu()


def test_static_scratch_plan_equals_the_caller_scratch_plan_twice_in_a_row():
    g = torch.Generator().manual_seed(77)
    cases = [(300, 7, 50, 16), (23, 7, 50, 64), (1500, 9, 129, 64)]          # the second is smaller than the first: stale
    for rows, slots, e, tile in cases:                                        # scratch from the larger call must not matter
        picks = torch.stack([torch.randperm(e, generator=g)[:slots] for _ in range(rows)]).to(torch.int32).to(DEV)
        want = plans(picks, e, tile, static=False)
        for _ in range(2):
            got = plans(picks, e, tile, static=True)
            assert all(torch.equal(a, b) for a, b in zip(got, want)), (rows, slots, e, tile)


def test_sizes_beyond_the_built_in_scratch_are_refused():
    lib = _lib.lib()
    picks = torch.zeros((16385,), dtype=torch.int32, device=DEV)
    out = torch.zeros((16385 * 3,), dtype=torch.int32, device=DEV)
    rc = lib.tf_moe_plan_static(picks.data_ptr(), 16385, 8, 16, out.data_ptr(), out.data_ptr(), out.data_ptr(), 100,
                                _lib.stream_of(picks))
    assert rc < 0 and b"exceed the built-in scratch" in lib.tf_last_error()
    rc = lib.tf_moe_plan_static(picks.data_ptr(), 16384, 4097, 16, out.data_ptr(), out.data_ptr(), out.data_ptr(), 100,
                                _lib.stream_of(picks))
    assert rc < 0
