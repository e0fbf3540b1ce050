"""The persistent decode kernel (tf_qmm_set) on a B200: every output row must carry the bits of the tiled kernel behind
tf_qmm for the same projection and slice count (the exact-decoding contract does not care which launch form ran), for
single projections and for sets that share their input, at every lane count and for every format."""

import ctypes

import pytest
import torch

from tensorfold_b200 import _lib, synthetic
from tensorfold_b200.cuda.kernels import qmm

from gpu_util import DEV, assert_close_bf16, oracle_f64, to_dev

pytestmark = pytest.mark.gpu

FORMATS = [(b, g) for b in qmm.BITS for g in qmm.GROUPS]


def packed(n, k, gs, seed, bits=4):
    w = to_dev(*synthetic.raw_weight(n, k, bits, gs, seed))
    return qmm.pack(*w, gs, bits=bits)


def tiled_kernel(x, q, **kw):
    """The same call through tf_qmm (the tiled kernel with clusters)."""

    qmm.STREAM = False
    try:
        return qmm.matmul(x, q, **kw)
    finally:
        qmm.STREAM = True


@pytest.fixture(autouse=True)
def default_knobs():
    yield
    _lib.lib().tf_tune(b"stream_lanes", 0)
    _lib.lib().tf_tune(b"stream_blocks", 0)


@pytest.mark.parametrize("n,k,gs,sk", [(48, 5120, 64, 8), (1024, 5120, 64, 8), (1024, 5120, 64, 1), (5120, 6144, 64, 8),
                                       (200, 1024, 32, 2), (1536, 2048, 32, 4), (256, 2048, 128, 2), (640, 64 * 34, 64, 2),
                                       (384, 64 * 51, 64, 3), (300, 32 * 21, 32, 3), (2048, 64 * 20, 64, 20),
                                       (640, 64 * 34, 64, 5), (512, 6144, 64, 14), (256, 32 * 21, 32, 4)])
def test_rows_carry_the_tiled_kernels_bits(n, k, gs, sk):
    q = packed(n, k, gs, n + 3 * k)
    x = synthetic.activations(16, k, 4).to(DEV)
    want = tiled_kernel(x, q, sk=sk) if sk <= 8 else tiled_kernel(x, q, sk=sk, part=torch.empty((sk, 16, n), device=DEV))
    for m in (1, 2, 5, 8, 9, 13, 16):
        got = qmm.matmul(x[:m], q, sk=sk)
        assert torch.equal(got, want[:m]), f"{n}x{k} sk={sk}: rows differ at M={m}"
    assert torch.equal(qmm.matmul(x, q, sk=sk, f32=True), tiled_kernel(x, q, sk=sk, f32=True) if sk <= 8 else
                       tiled_kernel(x, q, sk=sk, f32=True, part=torch.empty((sk, 16, n), device=DEV)))
    assert _lib.device_error(x) == 0


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_every_format_and_lane_count(bits, gs):
    n, k = 328, gs * 24
    q = packed(n, k, gs, 31 * bits + gs, bits)
    x = synthetic.activations(16, k, 9).to(DEV)
    for sk in (1, 3, 4):
        want = tiled_kernel(x, q, sk=sk)
        for lanes in (1, 2, 4):
            _lib.check(_lib.lib().tf_tune(b"stream_lanes", lanes), "tune")
            for m in (1, 7, 16):
                assert torch.equal(qmm.matmul(x[:m], q, sk=sk), want[:m]), (bits, gs, sk, lanes, m)
    assert _lib.device_error(x) == 0


def test_a_set_gives_the_bits_of_separate_calls():
    """q/k/v of the dense-27B layer in one launch, then gate/up; each output equals its own tf_qmm call."""

    k = 5120
    x = synthetic.activations(16, k, 1).to(DEV)
    for shapes in ([6144, 1024, 1024], [17408, 17408], [1024, 6144, 48, 200]):
        qs = [packed(n, k, 64, 7 + i) for i, n in enumerate(shapes)]
        sks = [qmm.default_split(n, k, 64) for n in shapes]
        want = [tiled_kernel(x, q, sk=sk) for q, sk in zip(qs, sks)]
        for m in (1, 16):
            for blocks in (0, 1):                           # all resident blocks, and one an SM (several items a block)
                _lib.check(_lib.lib().tf_tune(b"stream_blocks", blocks), "tune")
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
    qmm.matmul(x, narrow, sk=8)
    assert torch.equal(qmm.matmul(x, wide, sk=2), tiled_kernel(x, wide, sk=2))
    assert torch.equal(qmm.matmul(x, narrow, sk=8), tiled_kernel(x, narrow, sk=8))
    assert _lib.device_error(x) == 0


def test_given_group_sums_and_strided_outputs():
    n, k = 640, 3072
    q = packed(n, k, 64, 5)
    x = synthetic.activations(16, k, 3).to(DEV)
    xs = qmm.group_sums(x)
    want = tiled_kernel(x, q, sk=4)
    assert torch.equal(qmm.matmul(x, q, xs, sk=4), want)
    wide = torch.zeros((16, 2 * n + 8), dtype=torch.bfloat16, device=DEV)
    qmm.matmul(x, q, sk=4, out=wide[:, 8:8 + n])
    assert torch.equal(wide[:, 8:8 + n], want) and float(wide[:, :8].abs().max()) == 0 and float(wide[:, 8 + n:].abs().max()) == 0


def test_accuracy_against_the_oracle():
    n, k, gs = 1024, 5120, 64
    w = synthetic.affine_weight(n, k, 4, gs, seed=77)
    q = qmm.pack(*to_dev(*w), gs)
    x = synthetic.activations(16, k, 5)
    assert_close_bf16(qmm.matmul(x.to(DEV), q), oracle_f64(x, *w, gs, 4), "stream kernel")


def test_c_abi_refuses_bad_sets():
    lib = _lib.lib()
    q = packed(256, 1024, 64, 1)
    x = synthetic.activations(4, 1024, 1).to(DEV)
    out = torch.empty((4, 256), dtype=torch.bfloat16, device=DEV)
    scratch = torch.zeros((1 << 20,), dtype=torch.uint8, device=DEV)
    one_i, one_l, one_p = ctypes.c_int * 1, ctypes.c_int64 * 1, ctypes.c_void_p * 1
    stream = torch.cuda.current_stream().cuda_stream

    def call(m=4, sk=2, scratch_ptr=scratch.data_ptr(), scratch_bytes=scratch.numel(), out_ptr=out.data_ptr(), nproj=1):
        return lib.tf_qmm_set(x.data_ptr(), 1024, m, None, 1024, 4, 64, nproj, one_p(q.weight.data_ptr()), one_l(0), one_i(256),
                              one_i(sk), one_p(out_ptr), one_l(256), 0, scratch_ptr, scratch_bytes, 0, stream)

    assert call() == 0
    assert call(m=17) < 0 and call(m=0) < 0
    assert call(sk=3) == 0                                   # slices need not divide the 16 groups evenly
    assert call(sk=17) < 0                                   # but each holds one group at least
    assert call(scratch_ptr=None) < 0 and call(scratch_bytes=64) < 0
    assert call(out_ptr=None) < 0
    assert call(nproj=5) < 0
    torch.cuda.synchronize()
    assert _lib.device_error(x) == 0
