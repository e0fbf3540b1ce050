"""ctypes binding of ``libtensorfold_b200.so``.  Loading fails loudly: there is no other implementation to fall back to."""

from __future__ import annotations

import ctypes
from functools import lru_cache
from pathlib import Path

import os

LIB_PATH = Path(os.environ.get("TENSORFOLD_B200_LIB") or Path(__file__).resolve().parent / "libtensorfold_b200.so")

_vp, _i32, _i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64

# name -> (restype, argtypes); mirrors include/tensorfold_b200.h
SIGNATURES = {
    "tf_version": (_i32, ()),
    "tf_arch": (ctypes.c_char_p, ()),
    "tf_last_error": (ctypes.c_char_p, ()),
    "tf_init": (_i32, (_i32,)),
    "tf_device_error": (_i32, (_i32, _vp, ctypes.POINTER(_i32))),
    "tf_tune": (_i32, (ctypes.c_char_p, _i32)),
    "tf_split_k": (_i32, (_i32, _i32, _i32, _i32)),
    "tf_bucket": (_i32, (_i32,)),
    "tf_tiled_words": (_i64, (_i32, _i32, _i32, _i32)),
    "tf_unit_words": (_i32, (_i32, _i32)),
    "tf_pack": (_i32, (_vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp)),
    "tf_unpack": (_i32, (_vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp)),
    "tf_group_sums": (_i32, (_vp, _i64, _i32, _i32, _i32, _vp, _vp)),
    "tf_qmm": (_i32, (_vp, _i64, _i32, _vp, _vp, _i64, _i32, _i32, _i32, _i32, _i32, _vp, _i64, _i32, _vp, _i32, _i32,
                      _vp)),
    "tf_qmm_set_scratch_bytes": (_i64, (_i32, _vp, _vp)),
    "tf_qmm_set_geometry": (_i32, (_i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp)),
    "tf_qmm_set": (_i32, (_vp, _i64, _i32, _vp, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _i64, _i32,
                          _vp)),
    "tf_pack_pair": (_i32, (_vp, _vp, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _vp, _vp)),
    "tf_qmm_act": (_i32, (_vp, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _i64, _i32, ctypes.c_float, _i32, _vp)),
    "tf_moe_plan_blocks": (_i32, (_i32,)),
    "tf_moe_plan": (_i32, (_vp, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _i32, _vp)),
    "tf_moe_plan_static": (_i32, (_vp, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _vp)),
    "tf_moe_experts": (_i32, (_vp, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _i32, _vp, _i64, _i32, _i32,
                              ctypes.c_float, _vp)),
    "tf_moe_experts_prefill": (_i32, (_vp, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp, _i32, _i32, _vp, _vp, _i64,
                                      _i32, _i32, ctypes.c_float, _vp)),
    "tf_selftest_lost_wait": (_i32, (_i32, _vp)),
    "tf_moe_router": (_i32, (_vp, _i64, _i32, _i32, _vp, _i32, _vp, _i64, _vp)),
    "tf_moe_router_tiles": (_i32, (_vp, _i64, _i32, _i32, _vp, _i32, _vp, _i64, _vp)),
    "tf_moe_topk": (_i32, (_vp, _i64, _i32, _i32, _i32, _i32, _vp, _vp, _vp)),
    "tf_peer_flag_bytes": (ctypes.c_size_t, ()),
    "tf_peer_alloc": (_i32, (ctypes.c_size_t, _vp)),
    "tf_peer_free": (_i32, (_vp,)),
    "tf_peer_export": (_i32, (_vp, _vp)),
    "tf_peer_open": (_i32, (_vp, _vp)),
    "tf_peer_close": (_i32, (_vp,)),
    "tf_peer_reduce": (_i32, (_vp, _i32, _i32, ctypes.c_size_t, ctypes.c_size_t, _i64, _i32, _i32, _i32, ctypes.c_size_t,
                              ctypes.c_size_t, ctypes.c_uint, _i32, _vp)),
    "tf_moe_topk_local": (_i32, (_vp, _i64, _i32, _i32, _i32, _i32, _i32, _i32, _vp, _vp, _vp)),
    "tf_moe_combine": (_i32, (_vp, _i32, _vp, _i32, _i32, _i32, _vp, _vp)),
    "tf_affine_rows": (_i32, (_vp, _i32, _i32, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _vp, _i32, _vp)),
    "tf_add_rmsnorm": (_i32, (_vp, _vp, _vp, _i32, _i32, ctypes.c_float, _vp, _vp, _vp, _i32, _vp)),
    "tf_swiglu": (_i32, (_vp, _vp, _i32, _i32, _vp, _vp, _i32, _vp)),
    "tf_sum_ranks": (_i32, (_vp, _i32, _i64, _i32, _vp, _i32, _vp)),
    "tf_qmm_prefill": (_i32, (_vp, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _vp, _i64, _i32, _vp)),
    "tf_qmm_prefill_act": (_i32, (_vp, _i64, _i32, _vp, _i64, _i32, _i32, _i32, _vp, _i64, _i32, _i32, ctypes.c_float, _vp)),
    "tf_reduce_slices": (_i32, (_vp, _i32, _i64, _vp, _i32, _vp)),
}


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    if not LIB_PATH.exists():
        raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m tensorfold_b200.build` "
                           "(there is no fallback path)")
    handle = ctypes.CDLL(str(LIB_PATH))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)          # AttributeError here means the library and the header disagree
        fn.restype, fn.argtypes = res, list(args)
    return handle


def check(code: int, what: str) -> None:
    """Raise like the reference does: ValueError for refused arguments, RuntimeError for launch failures."""

    if code == 0:
        return
    text = lib().tf_last_error().decode(errors="replace")
    if code < 0:
        raise ValueError(f"{what}: {text}")
    raise RuntimeError(f"{what}: CUDA error {code}: {text}")


_ready: set[int] = set()


def ensure_device(index: int) -> None:
    """Per-device set-up (kernel attributes, error word); the first call must come before any CUDA-graph capture."""

    if index not in _ready:
        check(lib().tf_init(index), "tf_init")
        _ready.add(index)


def stream_of(t) -> int:
    import torch

    if not t.is_cuda:
        raise ValueError("operands must live on a CUDA device: this path has no CPU implementation")
    ensure_device(t.device.index)
    if t.device.index != torch.cuda.current_device():
        # the entry points take per-device state (error word, SM count, built-in scratch) from the CURRENT device
        raise ValueError(f"operands live on cuda:{t.device.index} but cuda:{torch.cuda.current_device()} is current: "
                         "call under torch.cuda.device(tensor.device)")
    return torch.cuda.current_stream(t.device).cuda_stream


def device_error(t) -> int:
    """Read and clear the error word kernels set when a bounded wait gave up (0: none).  Synchronises the stream."""

    import torch

    code = _i32(0)
    check(lib().tf_device_error(t.device.index, torch.cuda.current_stream(t.device).cuda_stream, ctypes.byref(code)),
          "tf_device_error")
    return code.value
