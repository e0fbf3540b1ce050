"""The CPU oracle against the golden vectors made from the reference's own Python, and against the reference's
``code_at`` expression compiled as C++ (where it was built)."""

import numpy as np
import pytest

from oracle import affine, moe, native

FORMATS = [(b, g) for b in affine.BITS for g in affine.GROUPS]


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_dequantize_matches_reference_bits(golden, bits, gs):
    tag = f"deq_b{bits}_g{gs}"
    s = affine.bf16_from_bits(golden[tag + "_scales"])
    b = affine.bf16_from_bits(golden[tag + "_biases"])
    got = affine.dequantize(golden[tag + "_words"], s, b, bits, gs, dtype=np.float32)
    np.testing.assert_array_equal(got, golden[tag + "_w"])                 # float32 q*s+b: bit-for-bit


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_pack_and_codes_are_inverses(bits, gs):
    rng = np.random.default_rng(811)
    values = rng.integers(0, 1 << bits, size=(5, gs * 4), dtype=np.uint32)
    words = affine.pack_codes(values, bits)
    assert affine.packed_shape(words.shape, (5, 4), (5, 4), bits, gs) == values.shape
    np.testing.assert_array_equal(affine.codes(words, bits), values)
    stream = [sum(int(v) << (i * bits) for i, v in enumerate(row)) for row in values]
    want = np.array([[(s >> sh) & 0xFFFFFFFF for sh in range(0, gs * 4 * bits, 32)] for s in stream], dtype=np.uint32)
    np.testing.assert_array_equal(words, want)


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_codes_match_the_reference_expression_compiled_as_cpp(bits, gs):
    decode = native.code_at()
    if decode is None:
        pytest.skip("oracle/_ref/code_at.so is built only where a reference checkout is present")
    import ctypes

    values = [(i * 29 + i // 7) % (1 << bits) for i in range(gs * 3)]
    words = affine.pack_codes(np.array([values]), bits)
    buf = (ctypes.c_uint32 * words.shape[1])(*words[0].tolist())
    assert [decode(buf, i, bits) for i in range(len(values))] == values
    np.testing.assert_array_equal(affine.codes(words, bits)[0], values)


def test_shape_only_planning_matches_reference(golden):
    shapes = golden["split_k_shapes"]
    assert [affine.split_k(int(n), int(k), 64) for n, k in shapes] == golden["split_k_g64"].tolist()
    assert [affine.split_k(int(n), int(k), 32) for n, k in shapes] == golden["split_k_g32"].tolist()
    assert [affine.split_k(int(n), int(k), 64, 296) for n, k in shapes] == golden["split_k_g64_t296"].tolist()
    assert [affine.bucket(int(m)) for m in golden["bucket_m"]] == golden["bucket"].tolist()
    assert [moe.max_items(*map(int, c)) for c in golden["max_items_cases"]] == golden["max_items"].tolist()


def test_input_slices_and_partition_map_match_reference(golden):
    for bits, gs, rank, a, b, g0, g1 in golden["input_slice"].tolist():
        assert affine.input_slice(gs * 4, bits, gs, rank) == ((a, b), (g0, g1))
    np.testing.assert_array_equal(affine.output_rows(16, 0), golden["rows_plain_r0"])
    np.testing.assert_array_equal(affine.output_rows(16, 1), golden["rows_plain_r1"])
    np.testing.assert_array_equal(affine.output_rows(40, 0, segments=(8, 8, 24)), golden["rows_seg_r0"])
    np.testing.assert_array_equal(affine.output_rows(40, 1, segments=(8, 8, 24)), golden["rows_seg_r1"])
    np.testing.assert_array_equal(affine.output_rows(32, 1, block=8), golden["rows_block_r1"])
    with pytest.raises(ValueError):
        affine.input_slice(384, 5, 128, 0)                       # tests/test_cuda_affine.py:140-142


def test_rank_sum_matches_reference_bits(golden):
    got = affine.bf16_bits(affine.sum_rank_partials([golden["rank_p0"], golden["rank_p1"]]))
    np.testing.assert_array_equal(got, golden["rank_sum_bf16"])


@pytest.mark.parametrize("bits,gs", FORMATS)
def test_exact_integer_case_is_exact(bits, gs):
    """scale 0.25, bias -0.5, x in {-1, -.5, 0, .5, 1}: every model must give the exact value
    (tests/test_cuda_affine.py:109-131)."""

    rng = np.random.default_rng(93)
    k, n, m = gs * 2, 35, 19
    values = rng.integers(0, 1 << bits, size=(n, k), dtype=np.uint32)
    words = affine.pack_codes(values, bits)
    scales = np.full((n, 2), 0.25, dtype=np.float32)
    biases = np.full((n, 2), -0.5, dtype=np.float32)
    x = rng.integers(-2, 3, size=(m, k)).astype(np.float32) * 0.5
    want = np.sum(x[:, None, :] * (values.astype(np.float32) * 0.25 - 0.5)[None, :, :], axis=2)
    np.testing.assert_array_equal(affine.quantized_matmul(x, words, scales, biases, gs, bits), want)
    np.testing.assert_array_equal(affine.lane_matmul(x, words, scales, biases, gs, bits, sk=1, f32=True), want)
    got = native.qmm_f64(affine.bf16_bits(x), words, affine.bf16_bits(scales), affine.bf16_bits(biases), gs, bits)
    np.testing.assert_array_equal(got, want)


def test_lane_model_tracks_the_definition():
    rng = np.random.default_rng(5)
    n, k, gs = 96, 1024, 64
    words = rng.integers(0, 2 ** 32, size=(n, k // 8), dtype=np.uint64).astype(np.uint32)
    s = affine.bf16_round(rng.random((n, k // gs), dtype=np.float32) * 0.02 + 0.001)
    b = affine.bf16_round(rng.standard_normal((n, k // gs), dtype=np.float32) * 0.05)
    x = affine.bf16_round(rng.standard_normal((7, k), dtype=np.float32))
    ref = affine.quantized_matmul(x, words, s, b, gs, 4)
    for sk in (1, 2):
        y = affine.lane_matmul(x, words, s, b, gs, 4, sk=sk)
        assert np.abs(y - ref).max() <= np.abs(ref).max() * 2 ** -7
    np.testing.assert_allclose(native.qmm_f64(affine.bf16_bits(x), words, affine.bf16_bits(s), affine.bf16_bits(b), gs, 4),
                               ref, rtol=1e-12, atol=1e-12)


def test_plan_and_selection_rules():
    picks = np.array([[3, 1, 4], [3, 0, 4], [3, 2, 4]], dtype=np.int32)
    items, members, distinct = moe.plan(picks, 5, 2)
    assert distinct == 5
    assert items.tolist() == [[0, 0, 1], [1, 1, 1], [2, 2, 1], [3, 3, 2], [3, 5, 1], [4, 6, 2], [4, 8, 1]]
    assert members.tolist() == [4, 1, 7, 0, 3, 6, 2, 5, 8]
    logits = np.array([[0.5, 2.0, 2.0, -1.0, 0.25]], dtype=np.float32)           # tie 1 vs 2 -> lower id first
    pk, w = moe.select_rows(logits, 2, 4, shared=True)
    assert pk.tolist() == [[1, 2, 4]]
    assert w[0, 0] == w[0, 1] == 0.5
    assert w[0, 2] == affine.bf16_round(np.float32(1 / (1 + np.exp(-0.25))))


def test_bf16_rounding_is_nearest_even():
    import torch

    v = torch.randn(4096, generator=torch.Generator().manual_seed(1)) * 37
    want = v.to(torch.bfloat16).float().numpy()
    np.testing.assert_array_equal(affine.bf16_round(v.numpy()), want)
    np.testing.assert_array_equal(affine.bf16_from_bits(affine.bf16_bits(v.numpy())), want)


def test_plan_equals_the_references_expected_plan(golden):
    """``oracle.moe.plan`` against the plans the reference's own test expects (``want_plan``, taken from the reference's
    test file by the golden generator): items, members and the count of distinct experts."""

    for tag in "abc":
        rows, slots, e, tile, distinct = map(int, golden[f"plan_{tag}_case"])
        picks = golden[f"plan_{tag}_picks"]
        assert picks.shape == (rows, slots)
        items, members, seen = moe.plan(picks, e, tile)
        assert items.tolist() == golden[f"plan_{tag}_items"].tolist()
        assert members.tolist() == golden[f"plan_{tag}_members"].tolist()
        assert seen == distinct


def test_top_k_rule_matches_the_references_kernel_body(golden):
    """``select_rows`` against the reference's ``_topk_rows`` body run over NumPy (tests/golden/make_golden.py): the
    chosen experts, their order under ties, the renormalised bf16 weights and the sigmoid-gated shared slot, bit for bit."""

    from oracle import moe as omoe

    rows, ne, top_k = map(int, golden["topk_case"])
    picks, wts = omoe.select_rows(golden["topk_logits"], top_k, ne, shared=True)
    assert picks.tolist() == golden["topk_picks"].tolist()
    assert picks[0, :2].tolist() == [3, 7] and picks[2, :top_k].tolist() == list(range(top_k))
    assert np.array_equal(wts, golden["topk_wts"])


def test_combine_and_swiglu_match_the_references_statements(golden):
    from oracle import moe as omoe

    assert np.array_equal(omoe.combine(golden["combine_y"], golden["combine_w"]), golden["combine_out"])
    assert np.array_equal(omoe.silu_mul(golden["swiglu_g"], golden["swiglu_u"]), golden["swiglu_out"])
    assert np.array_equal(omoe.silu_mul(golden["swiglu_g"], golden["swiglu_u"], 2.5), golden["swiglu_out_limit"])
