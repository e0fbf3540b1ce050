"""The C-ABI library loads and exports every symbol the header declares; host-only helpers agree with the oracle.
No compute call is made: these run without a GPU."""

import re
from pathlib import Path

import pytest

from oracle import affine
from tensorfold_b200 import _lib
from tensorfold_b200.cuda.kernels import qmm

ROOT = Path(__file__).resolve().parents[1]


def declared():
    text = (ROOT / "include" / "tensorfold_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tf_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = _lib.lib()
    names = declared()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_lib.SIGNATURES) <= set(names)
    assert lib.tf_arch() == b"sm_100a" and lib.tf_version() >= 100


def test_host_helpers_match_the_oracle(golden):
    lib = _lib.lib()
    for (n, k), want in zip(golden["split_k_shapes"].tolist(), golden["split_k_g64"].tolist()):
        assert lib.tf_split_k(n, k, 64, 192) == want == qmm.split_k(n, k) == affine.split_k(n, k)
    for (n, k), want in zip(golden["split_k_shapes"].tolist(), golden["split_k_g32"].tolist()):
        assert lib.tf_split_k(n, k, 32, 192) == want == qmm.split_k(n, k, 32)
    for m, want in zip(golden["bucket_m"].tolist(), golden["bucket"].tolist()):
        assert lib.tf_bucket(m) == want == qmm.bucket(m)
    assert lib.tf_bucket(0) < 0
    with pytest.raises(ValueError):
        qmm.bucket(0)
    assert lib.tf_unit_words(4, 64) == 4 * 32 * 8 + 128
    assert lib.tf_tiled_words(4096, 4096, 4, 64) == 32 * 64 * 1152
    assert lib.tf_tiled_words(48, 5120, 4, 64) == 1 * 80 * 1152          # padded to one super-block
    assert lib.tf_unit_words(7, 64) < 0 and lib.tf_tiled_words(64, 96, 4, 64) < 0


def test_refused_arguments_raise_before_any_launch():
    import torch

    x = torch.zeros((2, 128), dtype=torch.bfloat16)
    q = qmm.Q4(torch.zeros((1, 2, 1152), dtype=torch.int32), None, None, 64, 128, 64)
    with pytest.raises(ValueError):
        qmm.matmul(x.float(), q)                         # not bf16
    with pytest.raises(ValueError):
        qmm.matmul(x[:, :64], q)                         # wrong K
    with pytest.raises(ValueError):
        qmm.matmul(x, q)                                 # CPU tensors: no CPU implementation
    with pytest.raises(ValueError):
        qmm.pack(torch.zeros((4, 16), dtype=torch.int32), torch.zeros((4, 2)), torch.zeros((4, 2)), 64)


def test_c_abi_refuses_null_and_short_buffers_without_launching():
    """tf_qmm is called with made-up (non-null, aligned) addresses and must refuse before touching any of them: out missing
    when the sum is written to it, part missing when the slices leave the kernel, out rows shorter than n."""

    lib = _lib.lib()
    x, w, out, part = 0x10000, 0x20000, 0x30000, 0x40000

    def call(**kw):
        a = dict(x=x, ldx=128, m=4, xs=None, tiled=w, sb=0, n=64, k=128, bits=4, gs=64, sk=1, out=out, ldo=64, f32=0, part=None,
                 reduce=1, pdl=0)
        a.update(kw)
        return lib.tf_qmm(a["x"], a["ldx"], a["m"], a["xs"], a["tiled"], a["sb"], a["n"], a["k"], a["bits"], a["gs"], a["sk"],
                          a["out"], a["ldo"], a["f32"], a["part"], a["reduce"], a["pdl"], None)

    assert call(out=None) < 0                                    # one slice: the result goes to out
    assert call(sk=2, out=None) < 0                              # slices summed on chip: out again
    assert call(sk=2, reduce=0, part=None) < 0                   # slices leave the kernel: part
    assert call(k=64 * 32, ldx=64 * 32, sk=16, part=None) < 0    # more slices than a cluster holds: part
    assert call(ldo=32) < 0 and call(sb=-1) < 0
    assert call(x=None) < 0 and call(tiled=None) < 0 and call(x=x + 2) < 0
    assert call(sk=3) < 0                                        # two groups do not make three slices
    assert b"tf_qmm" in lib.tf_last_error()
    # with everything in place the next refusal is the missing per-device set-up (no GPU here): still no launch
    assert call() != 0
