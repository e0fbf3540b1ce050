"""The tcgen05 decode kernel (tf_qmm_set) on a B200, through the C ABI: a row's bits must not depend on the row count, on
the launch geometry (lanes a block, blocks an SM), on whether its projection ran alone or in a set, or on the scratch
area's history; results stay within the reference's bf16 tolerance of the float64 oracle for every format; K slices
returned to the caller add up, in slice order, to the reduced result."""

import ctypes

import pytest
import torch

from tensorfold_b200 import _lib, synthetic
from tensorfold_b200.cuda.kernels import qmm

from gpu_util import DEV, assert_close_bf16, oracle_f64, to_dev

pytestmark = pytest.mark.gpu

FORMATS = [(b, g) for b in qmm.BITS if b != 8 for g in qmm.GROUPS]


def packed(n, k, gs, seed, bits=4):
    w = to_dev(*synthetic.raw_weight(n, k, bits, gs, seed))
    return qmm.pack(*w, gs, bits=bits)


def tune(**knobs):
    for key, value in knobs.items():
        _lib.check(_lib.lib().tf_tune(key.encode(), value), "tune")


@pytest.fixture(autouse=True)
def default_knobs():
    yield
    tune(stream_lanes=0, stream_blocks=0)


@pytest.mark.parametrize("n,k,gs,sk", [(48, 5120, 64, 8), (1024, 5120, 64, 8), (1024, 5120, 64, 1), (5120, 6144, 64, 8),
                                       (200, 1024, 32, 2), (1536, 2048, 32, 4), (256, 2048, 128, 2), (640, 64 * 34, 64, 2),
                                       (384, 64 * 51, 64, 3), (300, 32 * 21, 32, 3), (2048, 64 * 20, 64, 20)])
def test_rows_do_not_depend_on_rows_lanes_or_blocks(n, k, gs, sk):
    q = packed(n, k, gs, n + 3 * k)
    x = synthetic.activations(40, k, 4).to(DEV)
    alone = torch.cat([qmm.matmul(x[r:r + 1], q, sk=sk) for r in range(40)])
    alone32 = torch.cat([qmm.matmul(x[r:r + 1], q, sk=sk, f32=True) for r in range(20)])
    for lanes, blocks in ((0, 0), (1, 0), (2, 0), (4, 0), (2, 1), (1, 1)):
        tune(stream_lanes=lanes, stream_blocks=blocks)
        for m in (1, 2, 5, 8, 9, 13, 16, 17, 33, 40):
            assert torch.equal(qmm.matmul(x[:m], q, sk=sk), alone[:m]), f"{n}x{k} sk={sk} lanes={lanes} blocks={blocks}: M={m}"
        assert torch.equal(qmm.matmul(x[:20], q, sk=sk, f32=True), alone32)
    perm = torch.randperm(40, generator=torch.Generator().manual_seed(3)).to(DEV)
    assert torch.equal(qmm.matmul(x[perm], q, sk=sk), alone[perm])
    assert _lib.device_error(x) == 0


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_every_format_is_accurate_and_geometry_free(bits, gs):
    n, k = 328, gs * 24
    words, scales, biases = synthetic.affine_weight(n, k, bits, gs, seed=31 * bits + gs)
    q = qmm.pack(*to_dev(words, scales, biases), gs, bits=bits)
    x = synthetic.activations(16, k, 9)
    ref = oracle_f64(x, words, scales, biases, gs, bits)
    xd = x.to(DEV)
    for sk in (1, 3, 4):
        want = qmm.matmul(xd, q, sk=sk)
        assert_close_bf16(want, ref, f"{bits}b/g{gs} sk={sk}")
        for lanes in (1, 2, 4):
            tune(stream_lanes=lanes)
            for m in (1, 7, 16):
                assert torch.equal(qmm.matmul(xd[:m], q, sk=sk), want[:m]), (bits, gs, sk, lanes, m)
        tune(stream_lanes=0)
    assert _lib.device_error(xd) == 0


def test_a_set_gives_the_bits_of_separate_calls():
    """q/k/v of the dense-27B layer in one launch, then gate/up; each output equals its own single-projection call."""

    k = 5120
    x = synthetic.activations(16, k, 1).to(DEV)
    for shapes in ([6144, 1024, 1024], [17408, 17408], [1024, 6144, 48, 200]):
        qs = [packed(n, k, 64, 7 + i) for i, n in enumerate(shapes)]
        sks = [qmm.default_split(n, k, 64) for n in shapes]
        want = [qmm.matmul(x, q, sk=sk) for q, sk in zip(qs, sks)]
        for m in (1, 16):
            for blocks in (0, 1):                           # all resident blocks, and one an SM (several items a block)
                tune(stream_blocks=blocks)
                got = qmm.matmul_set(x[:m], qs, sks=sks)
                for g, w, n in zip(got, want, shapes):
                    assert torch.equal(g, w[:m]), (shapes, n, m, blocks)
    assert _lib.device_error(x) == 0


def test_scratch_counters_return_to_zero_and_calls_repeat():
    k = 2048
    qs = [packed(n, k, 64, 40 + n) for n in (512, 384)]
    x = synthetic.activations(12, k, 2).to(DEV)
    first = qmm.matmul_set(x, qs, sks=[4, 8])
    stream = torch.cuda.current_stream().cuda_stream
    scratch = qmm._set_scratch[(x.device.index, stream)]
    counters = 64 * 1024                                     # the counter area at the head of the scratch
    torch.cuda.synchronize()
    assert int(scratch[:counters].max()) == 0
    for _ in range(3):
        again = qmm.matmul_set(x, qs, sks=[4, 8])
        assert all(torch.equal(a, b) for a, b in zip(first, again))
    assert int(scratch[:counters].max()) == 0


def test_a_wide_call_after_a_narrow_one_on_the_same_scratch():
    """The counter area has a fixed place: slices of an earlier, narrower call must not sit where a later call counts."""

    k = 1024
    x = synthetic.activations(16, k, 6).to(DEV)
    narrow, wide = packed(256, k, 64, 1), packed(128 * 70, k, 64, 2)
    fresh = qmm.matmul(x, wide, sk=2)
    qmm.matmul(x, narrow, sk=8)
    assert torch.equal(qmm.matmul(x, wide, sk=2), fresh)
    assert torch.equal(qmm.matmul(x[3:4], wide, sk=2), fresh[3:4])
    assert _lib.device_error(x) == 0


def test_given_group_sums_and_strided_outputs():
    n, k = 640, 3072
    q = packed(n, k, 64, 5)
    x = synthetic.activations(16, k, 3).to(DEV)
    xs = qmm.group_sums(x)
    want = qmm.matmul(x, q, sk=4)
    assert torch.equal(qmm.matmul(x, q, xs, sk=4), want)       # tf_group_sums gives the kernel's own sums
    wide = torch.zeros((16, 2 * n + 8), dtype=torch.bfloat16, device=DEV)
    qmm.matmul(x, q, sk=4, out=wide[:, 8:8 + n])
    assert torch.equal(wide[:, 8:8 + n], want) and float(wide[:, :8].abs().max()) == 0 and float(wide[:, 8 + n:].abs().max()) == 0


def test_slices_add_up_in_slice_order():
    n, k = 520, 4096
    q = packed(n, k, 64, 8)
    x = synthetic.activations(21, k, 3).to(DEV)
    for sk in (2, 8, 16):
        parts = qmm.matmul(x, q, sk=sk, reduce=False)
        assert parts.shape == (sk, 21, n) and parts.dtype == torch.float32
        total = parts[0].clone()
        for s in range(1, sk):
            total = total + parts[s]
        assert torch.equal(total, qmm.matmul(x, q, sk=sk, f32=True))
        assert torch.equal(total.bfloat16(), qmm.matmul(x, q, sk=sk))


def test_accuracy_at_the_layer_shapes():
    n, k, gs = 1024, 5120, 64
    w = synthetic.affine_weight(n, k, 4, gs, seed=77)
    q = qmm.pack(*to_dev(*w), gs)
    x = synthetic.activations(16, k, 5)
    assert_close_bf16(qmm.matmul(x.to(DEV), q), oracle_f64(x, *w, gs, 4), "tcgen05 kernel")


def test_the_tiled_kernel_behind_tf_qmm_keeps_its_own_contract():
    """tf_qmm (mma.sync chains, clusters) still serves 8-bit weights, the expert tables and C callers: its rows are
    stable over row counts too, and within tolerance of the same oracle."""

    n, k = 640, 2048
    w = synthetic.affine_weight(n, k, 4, 64, seed=12)
    q = qmm.pack(*to_dev(*w), 64)
    x = synthetic.activations(40, k, 7)
    xd = x.to(DEV)
    qmm.STREAM = False
    try:
        alone = torch.cat([qmm.matmul(xd[r:r + 1], q) for r in range(40)])
        for m in (1, 16, 17, 40):
            assert torch.equal(qmm.matmul(xd[:m], q), alone[:m])
    finally:
        qmm.STREAM = True
    assert_close_bf16(alone, oracle_f64(x, *w, 64, 4), "tiled kernel")


def test_c_abi_refuses_bad_sets():
    lib = _lib.lib()
    q = packed(256, 1024, 64, 1)
    x = synthetic.activations(4, 1024, 1).to(DEV)
    out = torch.empty((4, 256), dtype=torch.bfloat16, device=DEV)
    scratch = torch.zeros((1 << 20,), dtype=torch.uint8, device=DEV)
    one_i, one_l, one_p = ctypes.c_int * 1, ctypes.c_int64 * 1, ctypes.c_void_p * 1
    stream = torch.cuda.current_stream().cuda_stream

    def call(m=4, sk=2, bits=4, scratch_ptr=scratch.data_ptr(), scratch_bytes=scratch.numel(), out_ptr=out.data_ptr(), nproj=1):
        return lib.tf_qmm_set(x.data_ptr(), 1024, m, None, 1024, bits, 64, nproj, one_p(q.weight.data_ptr()), one_l(0), one_i(256),
                              one_i(sk), one_p(out_ptr), one_l(256), 0, 0, scratch_ptr, scratch_bytes, 0, stream)

    assert call() == 0
    assert call(m=0) < 0
    assert call(sk=3) < 0                                    # 16 groups do not split three ways
    assert call(bits=8) < 0 and call(bits=7) < 0
    assert call(scratch_ptr=None) < 0 and call(scratch_bytes=64) < 0
    assert call(out_ptr=None) < 0
    assert call(nproj=5) < 0
    torch.cuda.synchronize()
    assert _lib.device_error(x) == 0
