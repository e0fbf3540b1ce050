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


def test_peer_reduction_layout_and_refusals():
    """The buffers of the one-launch reduction: flags first, then partial, result and the slots of flagged words, all
    16-byte aligned and disjoint; the form follows the partial's size; bad arguments are refused before any launch."""

    import ctypes

    from tensorfold_b200.cuda import tp

    lib = _lib.lib()
    flags = lib.tf_peer_flag_bytes()
    assert flags >= 18 * 128 and flags % 256 == 0
    for world in (2, 4, 8):
        for elements in (6144, 16 * 6144, 2048 * 6144):
            f, part, out, ll, slot, total = tp.PeerReducer.layout(elements, world)
            assert f == flags == part and out >= part + elements * 4 and ll >= out + elements * 4
            assert all(v % 16 == 0 for v in (part, out, ll, slot)) and total == ll + 2 * world * slot
            assert slot >= 2 * min(elements * 4, 1 << 19)          # a slot holds twice the largest flagged partial
    table = (ctypes.c_void_p * 2)(4096, 8192)                      # never dereferenced: every call below is refused
    call = lambda **kw: lib.tf_peer_reduce(table, kw.get("rank", 0), kw.get("world", 2), kw.get("part", 4096),
                                           kw.get("out", 1 << 20), kw.get("total", 4096), 0, 0, kw.get("mode", 0),
                                           kw.get("ll", 1 << 21), kw.get("slot", 1 << 16), 0, 0, None)
    assert call(world=3) < 0 and call(rank=2) < 0 and call(total=7) < 0 and call(total=4100) < 0
    assert call(part=64) < 0 and call(part=4100) < 0 and call(out=4096 + 64) < 0
    assert call(mode=9) < 0 and call(mode=1, total=4104) < 0 and call(mode=5) < 0
    assert call(mode=2, ll=4096) < 0 and call(mode=2, slot=1 << 10) < 0
    assert lib.tf_peer_reduce(None, 0, 2, 4096, 1 << 20, 4096, 0, 0, 0, 0, 0, 0, 0, None) < 0
    assert lib.tf_peer_alloc(16, None) < 0 and lib.tf_peer_export(None, None) < 0 and lib.tf_peer_open(None, None) < 0
