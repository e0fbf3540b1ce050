"""ctypes access to the oracle's native helpers (``oracle/_ref``).  Test infrastructure only."""

from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

_REF = Path(__file__).parent / "_ref"


def _load(name: str):
    path = _REF / name
    if not path.exists():
        from .build_ref import build

        build()
    return ctypes.CDLL(str(path)) if path.exists() else None


def code_at():
    """The reference's ``code_at`` expression compiled as C++ (None where it was never built)."""

    lib = _load("code_at.so")
    if lib is None:
        return None
    lib.decode.argtypes = (ctypes.POINTER(ctypes.c_uint32), ctypes.c_int, ctypes.c_int)
    lib.decode.restype = ctypes.c_uint32
    return lib.decode


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def port():
    lib = _load("liboracle.so")
    if lib is None:
        raise RuntimeError("oracle/_ref/liboracle.so could not be built")
    i64, i32, vp = ctypes.c_int64, ctypes.c_int, ctypes.c_void_p
    lib.oracle_dequantize.argtypes = (vp, vp, vp, i64, i64, i32, i32, vp)
    lib.oracle_qmm_f64.argtypes = (vp, i64, vp, vp, vp, i64, i64, i32, i32, vp)
    lib.oracle_qmm_f32.argtypes = (vp, i64, vp, vp, vp, i64, i64, i32, i32, vp)
    lib.oracle_threads.restype = i32
    lib.oracle_set_threads.argtypes = (i32,)
    lib.oracle_set_threads.restype = None
    return lib


def qmm_f64(x_bits, words, s_bits, b_bits, gs: int, bits: int) -> np.ndarray:
    """float64 ``x @ dequant(w).T`` with bf16 inputs given as uint16 bit patterns."""

    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    words = np.ascontiguousarray(words).view(np.uint32)
    s_bits = np.ascontiguousarray(s_bits, dtype=np.uint16)
    b_bits = np.ascontiguousarray(b_bits, dtype=np.uint16)
    m, k = x_bits.shape
    n = words.shape[0]
    out = np.empty((m, n), dtype=np.float64)
    port().oracle_qmm_f64(_ptr(x_bits), m, _ptr(words), _ptr(s_bits), _ptr(b_bits), n, k, bits, gs, _ptr(out))
    return out


def qmm_f32(x_bits, words, s_bits, b_bits, gs: int, bits: int) -> np.ndarray:
    x_bits = np.ascontiguousarray(x_bits, dtype=np.uint16)
    words = np.ascontiguousarray(words).view(np.uint32)
    s_bits = np.ascontiguousarray(s_bits, dtype=np.uint16)
    b_bits = np.ascontiguousarray(b_bits, dtype=np.uint16)
    m, k = x_bits.shape
    n = words.shape[0]
    out = np.empty((m, n), dtype=np.float32)
    port().oracle_qmm_f32(_ptr(x_bits), m, _ptr(words), _ptr(s_bits), _ptr(b_bits), n, k, bits, gs, _ptr(out))
    return out


def threads() -> int:
    return int(port().oracle_threads())


def set_threads(n: int) -> None:
    """Use ``n`` OpenMP threads from now on, whatever OMP_NUM_THREADS said when the process started."""

    port().oracle_set_threads(int(n))
