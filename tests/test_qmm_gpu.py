"""The tiled affine matmul on a B200 against the CPU oracle, through the C ABI: pack round trips, bit-exact rows at every
row count, accuracy within the reference's bf16 tolerance, exact-integer cases bit-for-bit.  Mirrors the reference's
tests/cuda/test_qmm.py and tests/test_cuda_affine.py:109-131."""

import numpy as np
import pytest
import torch

from oracle import affine as oracle
from tensorfold_b200 import _lib, synthetic
from tensorfold_b200.cuda.kernels import qmm

from gpu_util import DEV, assert_close_bf16, oracle_f64, to_dev

pytestmark = pytest.mark.gpu

ROWS = [1, 2, 7, 8, 9, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 127, 128, 129, 200, 256, 384, 512, 700, 1024, 1500, 2048]
FORMATS = [(b, g) for b in qmm.BITS for g in qmm.GROUPS]


def packed(n, k, gs, seed, bits=4):
    w = to_dev(*synthetic.raw_weight(n, k, bits, gs, seed))
    return qmm.pack(*w, gs, bits=bits), w


@pytest.mark.parametrize("n,k,gs", [(48, 5120, 64), (1024, 5120, 64), (5120, 6144, 64), (200, 1024, 32), (1536, 2048, 32),
                                    (300, 1024, 128)])
def test_pack_round_trip(n, k, gs):
    q, w = packed(n, k, gs, n + k)
    back = qmm.unpack(q)
    assert all(torch.equal(a, b) for a, b in zip(back, w))


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_pack_round_trip_every_format(bits, gs):
    q, w = packed(130, gs * 6, gs, 17 * bits + gs, bits)
    back = qmm.unpack(q)
    assert all(torch.equal(a, b) for a, b in zip(back, w))


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_exact_integer_case_is_bit_exact(bits, gs):
    """scale 0.25, bias -0.5, x in {-1, -.5, 0, .5, 1}: every product and sum is exact, so the output must be too."""

    rng = np.random.default_rng(93)
    k, n, m = gs * 2, 35, 19
    values = rng.integers(0, 1 << bits, size=(n, k), dtype=np.uint32)
    words = torch.from_numpy(oracle.pack_codes(values, bits).view(np.int32))
    scales = torch.full((n, 2), 0.25).bfloat16()
    biases = torch.full((n, 2), -0.5).bfloat16()
    xf = rng.integers(-2, 3, size=(m, k)).astype(np.float32) * 0.5
    want = np.sum(xf[:, None, :] * (values.astype(np.float32) * 0.25 - 0.5)[None, :, :], axis=2)
    q = qmm.pack(*to_dev(words, scales, biases), gs, bits=bits)
    x = torch.from_numpy(xf).bfloat16().to(DEV)
    got = qmm.matmul(x, q, f32=True).cpu().numpy()
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(qmm.matmul(x[17:18], q, f32=True).cpu().numpy(), want[17:18])


@pytest.mark.parametrize("n,k,gs", [(48, 5120, 64), (1024, 5120, 64), (5120, 17408, 64), (200, 1024, 32), (1536, 2048, 32),
                                    (256, 2048, 128)])
def test_rows_do_not_depend_on_row_count(n, k, gs):
    q, _ = packed(n, k, gs, 3 * n + k)
    top = max(ROWS)
    x = synthetic.activations(top, k, 7).to(DEV)
    alone = torch.cat([qmm.matmul(x[r:r + 1], q) for r in range(top)])
    for m in ROWS:
        assert torch.equal(qmm.matmul(x[:m], q), alone[:m]), f"{n}x{k}: rows differ at M={m}"
    perm = torch.randperm(top, generator=torch.Generator().manual_seed(3)).to(DEV)
    assert torch.equal(qmm.matmul(x[perm], q), alone[perm])
    f32 = qmm.matmul(x[:40], q, f32=True)
    assert torch.equal(torch.cat([qmm.matmul(x[r:r + 1], q, f32=True) for r in range(40)]), f32)


@pytest.mark.parametrize("bits,gs", [(2, 64), (3, 32), (3, 64), (5, 128), (6, 64), (8, 32), (8, 128)])
def test_rows_do_not_depend_on_row_count_other_widths(bits, gs):
    n, k = 200, gs * 24
    q, _ = packed(n, k, gs, bits * 100 + gs, bits)
    x = synthetic.activations(130, k, 11).to(DEV)
    alone = torch.cat([qmm.matmul(x[r:r + 1], q) for r in range(130)])
    for m in (1, 5, 8, 9, 16, 17, 32, 33, 64, 65, 130):
        assert torch.equal(qmm.matmul(x[:m], q), alone[:m]), (bits, gs, m)


@pytest.mark.parametrize("n,k,gs", [(1024, 5120, 64), (512, 2048, 32), (384, 2048, 128)])
def test_accuracy_matches_oracle(n, k, gs):
    q, w = packed(n, k, gs, 11 * n + k)
    x = synthetic.activations(16, k, 5)
    y = qmm.matmul(x.to(DEV), q)
    assert_close_bf16(y, oracle_f64(x, *[t.cpu() for t in w], gs, 4), f"{n}x{k}")


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_accuracy_every_format(bits, gs):
    n, k = 264, gs * 16
    words, scales, biases = synthetic.affine_weight(n, k, bits, gs, seed=bits * 7 + gs)
    q = qmm.pack(*to_dev(words, scales, biases), gs, bits=bits)
    x = synthetic.activations(16, k, 2)
    ref = oracle_f64(x, words, scales, biases, gs, bits)
    for m in (1, 16):
        assert_close_bf16(qmm.matmul(x[:m].to(DEV), q), ref[:m], f"{bits}b/g{gs} M={m}")
    for sk in (1, 2, 4, 16):
        assert_close_bf16(qmm.matmul(x.to(DEV), q, sk=sk), ref, f"{bits}b/g{gs} sk={sk}")


def test_config0_single_matmul():
    """4-bit / group 64, x [4, 4096], W [4096, 4096], seed 0: the CPU-runnable reference configuration."""

    words, scales, biases = synthetic.affine_weight(4096, 4096, 4, 64, seed=0)
    x = synthetic.activations(4, 4096, 0)
    q = qmm.pack(*to_dev(words, scales, biases), 64)
    y = qmm.matmul(x.to(DEV), q)
    assert y.shape == (4, 4096) and y.dtype == torch.bfloat16
    assert_close_bf16(y, oracle_f64(x, words, scales, biases, 64, 4), "config 0")


def test_split_depends_only_on_shape():
    for n, k in [(48, 5120), (1024, 5120), (5120, 6144), (17408, 5120), (5120, 17408), (248320, 5120)]:
        sk = qmm.default_split(n, k)
        assert sk == qmm.default_split(n, k) and 1 <= sk <= (k // 64)


def test_strided_rows_buffers_and_unreduced_slices():
    n, k, gs = 5120, 17408, 64
    q, _ = packed(n, k, gs, 17)
    wide = synthetic.activations(24, k + 64, 3).to(DEV)
    x = wide[:, :k]                                   # rows 16-byte aligned, stride k + 64
    want = qmm.matmul(x.contiguous(), q)
    assert torch.equal(qmm.matmul(x, q), want)
    out = torch.empty_like(want)
    assert qmm.matmul(x, q, out=out) is out and torch.equal(out, want)
    sk = qmm.default_split(n, k)
    assert sk > 1
    slices = qmm.matmul(x, q, reduce=False, f32=True)
    assert slices.shape == (sk, 24, n)
    total = slices[0]
    for s in range(1, sk):
        total = total + slices[s]
    assert torch.equal(total, qmm.matmul(x, q, f32=True))
    assert torch.equal(qmm.matmul(x, q, sk=16), qmm.matmul(x, q, sk=16, part=torch.empty((16, 24, n), device=DEV)))
    odd = wide[:, 1:k + 1]                            # misaligned rows are copied, not refused
    assert torch.equal(qmm.matmul(odd, q), qmm.matmul(odd.contiguous(), q))


def test_group_sums_are_the_kernels_own():
    k, gs = 5120, 64
    q, _ = packed(1024, k, gs, 23)
    x = synthetic.activations(37, k, 9).to(DEV)
    xs = qmm.group_sums(x, gs)
    ref = x.float().view(37, k // gs, gs).double().sum(-1)
    assert (xs.double() - ref).abs().max() <= 1e-4
    assert torch.equal(qmm.matmul(x, q, xs), qmm.matmul(x, q))
    assert torch.equal(qmm.group_sums(x[5:6], gs), xs[5:6])
    for g in (32, 128):
        assert (qmm.group_sums(x, g).double() - x.float().view(37, k // g, g).double().sum(-1)).abs().max() <= 2e-4


def test_super_block_views_give_the_same_columns():
    """Rows [a, b) of a tiled weight on 128-column boundaries are a view (families/qwen3_5/cuda/qmm_fast.py:28-46)."""

    n, k, gs = 1024, 2048, 64
    q, _ = packed(n, k, gs, 29)
    x = synthetic.activations(9, k, 4).to(DEV)
    sk = qmm.default_split(n, k, gs)
    full = qmm.matmul(x, q, sk=sk)
    part = qmm.Q4(q.weight[2:5], None, None, 384, k, gs)
    assert torch.equal(qmm.matmul(x, part, sk=sk), full[:, 256:640])


def test_lane_mapping_never_changes_bits():
    """How K slices map to blocks and lanes is a tuning knob; every setting gives the same bits."""

    n, k, gs = 1024, 4096, 64
    q, _ = packed(n, k, gs, 41)
    x = synthetic.activations(33, k, 6).to(DEV)
    lib = _lib.lib()
    want = {m: qmm.matmul(x[:m], q, sk=8, f32=True) for m in (1, 16, 33)}
    try:
        for lanes in (1, 2, 4):
            _lib.check(lib.tf_tune(b"qmm_lanes", lanes), "tune")
            for m in (1, 16, 33):
                assert torch.equal(qmm.matmul(x[:m], q, sk=8, f32=True), want[m]), (lanes, m)
            sl = qmm.matmul(x[:16], q, sk=8, f32=True, reduce=False)
            total = sl[0]
            for s in range(1, 8):
                total = total + sl[s]
            assert torch.equal(total, want[16])
    finally:
        lib.tf_tune(b"qmm_lanes", 0)


def test_fork_join_runs_independent_projections_side_by_side():
    """q/k/v-style projections of the same rows launched through fork_join give the bits of one-after-another launches,
    eagerly and from a captured CUDA graph."""

    shapes = [(1024, 1024), (256, 1024), (256, 1024)]
    qs = [qmm.pack(*to_dev(*synthetic.affine_weight(n, k, 4, 64, seed=40 + i)), 64) for i, (n, k) in enumerate(shapes)]
    x = synthetic.activations(9, 1024, 5).to(DEV)
    want = [qmm.matmul(x, q) for q in qs]
    outs = [torch.zeros_like(w) for w in want]
    thunks = [(lambda q=q, o=o: qmm.matmul(x, q, out=o)) for q, o in zip(qs, outs)]
    qmm.fork_join(thunks)
    torch.cuda.synchronize()
    for o, w in zip(outs, want):
        assert torch.equal(o, w)
    for o in outs:
        o.zero_()
    stream, graph = torch.cuda.Stream(), torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            qmm.fork_join(thunks)
            y = qmm.matmul(outs[0], qs[1])                             # a dependent launch after the join
        graph.replay()
    torch.cuda.synchronize()
    for o, w in zip(outs, want):
        assert torch.equal(o, w)
    assert torch.equal(y, qmm.matmul(want[0], qs[1]))


def test_no_wait_gave_up():
    x = torch.zeros(1, device=DEV)
    assert _lib.device_error(x) == 0
