"""Helpers shared by the GPU parity tests: the oracle as checker, inputs from the seeded generators."""

import numpy as np
import torch

from oracle import native
from tensorfold_b200 import synthetic

DEV = "cuda"


def oracle_f64(x, words, scales, biases, gs, bits):
    """float64 x @ dequant(w).T from the C oracle (bf16 inputs as bit patterns)."""

    return native.qmm_f64(synthetic.bf16_bits(x), words.cpu().numpy(), synthetic.bf16_bits(scales),
                          synthetic.bf16_bits(biases), gs, bits)


def to_dev(*ts):
    return tuple(t.to(DEV) for t in ts)


def assert_close_bf16(y, ref, what=""):
    """The reference's tolerance for bf16 outputs with fp32 accumulation: |y - ref|max <= 2^-7 |ref|max
    (tests/cuda/test_qmm.py:64-70), plus a relative bound on the large elements."""

    y = y.detach().float().cpu().numpy().astype(np.float64)
    err = np.abs(y - ref).max()
    top = np.abs(ref).max()
    assert err <= top * 2 ** -7, f"{what}: max abs error {err} exceeds 2^-7 * {top}"
    big = np.abs(ref) > top * 2 ** -4
    if big.any():
        rel = (np.abs(y - ref)[big] / np.abs(ref)[big]).max()
        assert rel <= 2 ** -6, f"{what}: max relative error {rel} on large elements"
