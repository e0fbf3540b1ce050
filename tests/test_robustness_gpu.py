"""What a caller sees when something goes wrong on the device, without faulting or hanging anything: a wait that
nothing satisfies runs out, the kernel returns and the error word names it; a plan item that names an expert outside
the table is skipped and reported; in both cases the context stays usable and the next call is correct."""

import pytest
import torch

from tensorfold_b200 import _lib, synthetic
from tensorfold_b200.cuda import experts
from tensorfold_b200.cuda.kernels import qmm

from gpu_util import DEV, to_dev

pytestmark = pytest.mark.gpu


def test_a_lost_wait_comes_back_as_an_error_code():
    x = torch.zeros(1, device=DEV)
    assert _lib.device_error(x) == 0
    lib = _lib.lib()
    _lib.check(lib.tf_selftest_lost_wait(8, _lib.stream_of(x)), "self-test")
    assert _lib.device_error(x) == 1                         # a stage never arrived
    assert _lib.device_error(x) == 0                         # reading clears the word
    assert lib.tf_selftest_lost_wait(0, _lib.stream_of(x)) < 0
    # the context is intact: a matmul right after it is still exact
    q = qmm.pack(*to_dev(*synthetic.raw_weight(256, 512, 4, 64, 3)), 64)
    a = synthetic.activations(5, 512, 1).to(DEV)
    assert torch.equal(qmm.matmul(a, q), torch.cat([qmm.matmul(a[r:r + 1], q) for r in range(5)]))
    assert _lib.device_error(x) == 0


def test_a_plan_item_outside_the_table_is_skipped_and_reported():
    d, ni, e, gs = 256, 128, 4, 64
    mats = lambda n, k, s: tuple(torch.stack(ts) for ts in zip(*[synthetic.raw_weight(n, k, 4, gs, s + i) for i in range(e)]))
    ex = experts.make([to_dev(*mats(ni, d, 1)), to_dev(*mats(ni, d, 20))], to_dev(*mats(d, ni, 40)), gs)
    rows, slots = 6, 2
    plan = experts.Plan(rows, slots, e, DEV)
    picks = torch.tensor([[0, 1], [2, 3], [1, 0], [3, 2], [0, 2], [1, 3]], dtype=torch.int32, device=DEV)
    experts.route(picks, plan)
    x = synthetic.activations(rows, d, 2).to(DEV)
    good = torch.zeros((rows * slots, ni), dtype=torch.bfloat16, device=DEV)
    experts.gate_up(x, ex, plan, good, rows)
    assert _lib.device_error(x) == 0
    # the same plan against a table of two experts, through the C ABI (the Python wrapper refuses this before launching)
    small = ex.up[:2].contiguous()
    out = torch.full_like(good, 7.0)
    rc = _lib.lib().tf_moe_experts(x.data_ptr(), x.stride(0), slots, small.data_ptr(), small.stride(0), 2, 2 * ni, d, gs,
                                   plan.items.data_ptr(), plan.counts.data_ptr(), plan.members.data_ptr(), plan.items.shape[0],
                                   plan.tile, out.data_ptr(), out.stride(0), 0, 2, 0.0, _lib.stream_of(x))
    _lib.check(rc, "experts")
    assert _lib.device_error(x) == 5                         # reported, not read
    pairs = picks.reshape(-1)
    inside = pairs < 2
    assert torch.equal(out[inside], good[inside])            # the items of experts 0 and 1 ran as before
    assert bool((out[~inside] == 7.0).all())                 # the others were left alone
    with pytest.raises(ValueError):
        experts.gate_up(x, experts.Experts(small, ex.down[:2].contiguous(), ex.gs, ex.width, ex.dims), plan, out, rows)
