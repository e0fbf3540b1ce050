"""4-bit lane matmul: rows run the same groups and K slices at any row count, so no row affects another.

Host-side mirror of the reference module ``tensorfold.cuda.kernels.qmm`` (cuda/kernels/qmm.py:24-171): same names,
argument meaning and errors; the arithmetic runs in ``libtensorfold_b200.so``.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import dataclass

import torch

from ... import _lib

BITS = (2, 3, 4, 5, 6, 8)
GROUPS = (32, 64, 128)


@dataclass
class Q4:
    """A packed (n, k) weight in the tiled layout: int32 units [ceil(n / 128), k / gs, unit words], each unit the codes
    of 128 output columns for one group followed by their 128 (scale, bias) bf16 pairs.  ``scales`` and ``biases`` stay
    None: the pairs live inside ``weight`` (``unpack`` returns them).  Field order follows cuda/kernels/qmm.py:24-35."""

    weight: torch.Tensor
    scales: torch.Tensor | None
    biases: torch.Tensor | None
    n: int
    k: int
    gs: int
    bits: int = 4

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()


def pack(weight: torch.Tensor, scales: torch.Tensor, biases: torch.Tensor, gs: int, chunk: int = 4096,
         bits: int = 4) -> Q4:
    """MLX (n, k * bits / 32) words, (n, k / gs) bf16 scales and biases -> ``Q4``.  ``chunk`` is accepted for
    signature parity (cuda/kernels/qmm.py:55) and unused: the repack is one kernel."""

    if bits not in BITS or gs not in GROUPS:
        raise ValueError("affine weights require 2/3/4/5/6/8 bits and groups of 32/64/128")
    if weight.dim() != 2 or weight.dtype not in (torch.int32, torch.uint32):
        raise ValueError("pack: weight must be 2-D int32/uint32 MLX words")
    if scales.dtype != torch.bfloat16 or biases.dtype != torch.bfloat16 or scales.shape != biases.shape:
        raise ValueError("pack: scales and biases must be matching bf16 tensors")
    n, words = weight.shape
    k = words * 32 // bits
    if scales.shape != (n, k // gs) or k % gs or (k * bits) % 32:
        raise ValueError(f"pack: words {tuple(weight.shape)} do not match scales {tuple(scales.shape)} at {bits} bits")
    stream = _lib.stream_of(weight)
    weight, scales, biases = weight.contiguous(), scales.contiguous(), biases.contiguous()
    lib = _lib.lib()
    unit = lib.tf_unit_words(bits, gs)
    out = torch.empty((-(-n // 128), k // gs, unit), dtype=torch.int32, device=weight.device)
    _lib.check(lib.tf_pack(weight.data_ptr(), scales.data_ptr(), biases.data_ptr(), n, k, bits, gs, out.data_ptr(),
                           stream), "pack")
    return Q4(out, None, None, n, k, gs, bits)


def unpack(q: Q4, chunk: int = 64) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """The stored MLX layout again: (n, k * bits / 32) int32 words, (n, k / gs) bf16 scales and biases."""

    stream = _lib.stream_of(q.weight)
    dev = q.weight.device
    words = torch.empty((q.n, q.k * q.bits // 32), dtype=torch.int32, device=dev)
    scales = torch.empty((q.n, q.k // q.gs), dtype=torch.bfloat16, device=dev)
    biases = torch.empty_like(scales)
    tiled = q.weight if q.weight.is_contiguous() else q.weight.contiguous()
    _lib.check(_lib.lib().tf_unpack(tiled.data_ptr(), q.n, q.k, q.bits, q.gs, words.data_ptr(), scales.data_ptr(),
                                    biases.data_ptr(), stream), "unpack")
    return words, scales, biases


def split_k(n: int, k: int, gs: int = 64, target: int = 192) -> int:
    """K slices for an (n, k) weight: a function of the shape only (never of the row count)."""

    tiles, groups, sk = -(-n // 64), k // gs, 1
    while sk < 8 and tiles * sk < target and groups % (sk * 2) == 0 and groups // (sk * 2) >= 8:
        sk *= 2
    return sk


LANES = 592            # 128-column lanes the persistent decode kernel streams side by side on a B200: 148 SMs x 4
MIN_GROUPS = 6         # groups a K slice should hold at least (three pipeline stages of 128 inputs at groups of 64)


def default_split(n: int, k: int, gs: int = 64, share: float = 1.0) -> int:
    """The K slices ``matmul`` uses when it is given none: a function of the shape only (never of the row count), chosen
    so that the projection's (128-column block, slice) units fill the machine's lanes once: LANES / blocks, at least
    MIN_GROUPS groups a slice.  Slices need not divide the groups evenly (slice s covers groups
    [s G / sk, (s + 1) G / sk)).  ``share`` is for projections an engine always launches as a set (q/k/v, gate/up):
    the set's 128-column blocks over this projection's, so that the SET fills the lanes once (2 for gate or up)."""

    blocks, groups = -(-n // 128), k // gs
    sk = int(LANES // max(1.0, blocks * share))
    return max(1, min(sk, groups // MIN_GROUPS if groups >= MIN_GROUPS else 1))


def set_splits(shapes, gs: int = 64) -> list[int]:
    """K slices for projections an engine always launches together (``matmul_set``): [(n, k), ...] -> one slice count
    each, so that the set's units fill the lanes once.  A load-time decision, like stacking: a projection's bits depend
    on its slice count, so it must use the same count wherever it runs."""

    blocks = [-(-n // 128) for n, _ in shapes]
    return [default_split(n, k, gs, share=sum(blocks) / b) for (n, k), b in zip(shapes, blocks)]


def bucket(m: int) -> int:
    """The reference's row tile (16, 32, else 64); kept for callers that size buffers by it.  Tiles never change bits."""

    if m < 1:
        raise ValueError("the lane matmul takes at least one row")
    return 16 if m <= 16 else 32 if m <= 32 else 64


def group_sums(x: torch.Tensor, gs: int = 64) -> torch.Tensor:
    """(M, K) bf16 (rows may be strided) -> (M, K/gs) fp32 sums of each group's inputs, with the matmul's own bits."""

    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] % gs:
        raise ValueError("group_sums: x must be (M, K) bf16 with K a multiple of the group")
    if x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) % 2) or x.data_ptr() % 4:
        x = x.clone(memory_format=torch.contiguous_format)
    stream = _lib.stream_of(x)
    m, k = x.shape
    xs = torch.empty((m, k // gs), dtype=torch.float32, device=x.device)
    _lib.check(_lib.lib().tf_group_sums(x.data_ptr(), x.stride(0), m, k, gs, xs.data_ptr(), stream), "group_sums")
    return xs


def _rows(x: torch.Tensor, k: int, who: str) -> torch.Tensor:
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != k:
        raise ValueError(f"{who}: x must be (M, {k}) bf16")
    if x.shape[0] < 1:
        raise ValueError(f"{who}: x needs at least one row")
    if x.stride(1) != 1 or (x.shape[0] > 1 and x.stride(0) % 8) or x.data_ptr() % 16:
        x = x.clone(memory_format=torch.contiguous_format)     # bulk copies read rows in 16-byte pieces
    return x


def matmul(x: torch.Tensor, q: Q4, xs: torch.Tensor | None = None, *, sk: int | None = None, f32: bool = False,
           out: torch.Tensor | None = None, part: torch.Tensor | None = None, reduce: bool = True,
           pdl: bool = False) -> torch.Tensor:
    """x @ q.T as (M, n) bf16, or unrounded fp32 with ``f32``; ``reduce=False`` returns K slices to add in order.

    ``pdl`` (not in the reference) launches with programmatic stream serialisation so the weight prefetch of this call
    overlaps the end of the previous kernel in the stream."""

    x = _rows(x, q.k, "matmul")
    m = x.shape[0]
    stream = _lib.stream_of(x)
    if q.weight.device != x.device:
        raise ValueError("matmul: x and the weight must share a CUDA device")
    kg = q.k // q.gs
    if xs is not None and (xs.dtype != torch.float32 or xs.shape != (m, kg) or not xs.is_contiguous()):
        raise ValueError(f"matmul: xs must be contiguous ({m}, {kg}) fp32")
    sk = sk or default_split(q.n, q.k, q.gs)
    if sk < 1 or sk > kg:
        raise ValueError("matmul: 1 to K / gs slices (a slice holds one group at least)")
    slices = sk > 1 and not reduce
    if out is None:
        if not slices:
            out = torch.empty((m, q.n), dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
    elif out.shape != (m, q.n) or out.dtype != (torch.float32 if f32 else torch.bfloat16) or out.stride(1) != 1:
        raise ValueError("matmul: out must be (M, n) of the requested dtype with unit-stride rows")
    if sk > 1 and (not reduce or sk > 8):
        if part is None:
            part = torch.empty((sk, m, q.n), dtype=torch.float32, device=x.device)
        elif part.dtype != torch.float32 or not part.is_contiguous() or part.numel() < sk * m * q.n:
            raise ValueError("matmul: part must hold (SK, M, n) fp32")
    if q.weight.dim() != 3 or q.weight.stride(2) != 1 or q.weight.stride(1) != q.weight.shape[2]:
        raise ValueError("matmul: the tiled weight may be sliced by super-blocks of 128 columns only")
    if STREAM and m <= STREAM_ROWS and part is None and (reduce or sk == 1):
        return matmul_set(x, [q], xs, sks=[sk], f32=f32, outs=[out], pdl=pdl)[0]     # same bits, persistent launch
    _lib.check(_lib.lib().tf_qmm(
        x.data_ptr(), x.stride(0), m, xs.data_ptr() if xs is not None else None, q.weight.data_ptr(),
        q.weight.stride(0), q.n, q.k, q.bits, q.gs, sk, out.data_ptr() if out is not None else None,
        out.stride(0) if out is not None else 0, int(f32), part.data_ptr() if part is not None else None,
        int(reduce), int(pdl), stream), "matmul")
    if sk == 1 or reduce:
        return out
    return part.reshape(-1)[:sk * m * q.n].view(sk, m, q.n)


STREAM = os.environ.get("TENSORFOLD_B200_STREAM", "1") != "0"      # decode windows run the persistent kernel (same bits)
STREAM_ROWS = 16
SET_MAX = 4
SCRATCH_BYTES = 16 << 20          # one scratch area: room for a gate/up set of 17408 rows each in 4 K slices
SCRATCH_AREAS = 4                 # areas made on a device's first call: the calling stream's and three side streams'
_set_scratch: dict = {}           # (device index, stream) -> the stream's scratch area
_free_areas: dict = {}            # device index -> areas not yet handed to a stream


def _scratch_for(device: torch.device, stream: int, need: int) -> torch.Tensor:
    """The scratch area of (device, stream) where the K slices of a set meet: zeroed once, left zero by every call.

    Areas are made eagerly (four on a device's first call, more when a fifth stream shows up or a set needs more room)
    and only handed out during a stream capture: a graph must not own memory that later calls use, so a capture that
    would need a new allocation is refused with a message saying which eager call to make first."""

    key = (device.index, stream)
    buf = _set_scratch.get(key)
    if buf is not None and buf.numel() >= need:
        return buf
    capturing = torch.cuda.is_current_stream_capturing()
    free = _free_areas.setdefault(device.index, [])
    if not free and not capturing and not any(k[0] == device.index for k in _set_scratch):
        free.extend(torch.zeros((SCRATCH_BYTES,), dtype=torch.uint8, device=device) for _ in range(SCRATCH_AREAS))
    fits = [i for i, area in enumerate(free) if area.numel() >= need]
    if buf is None and fits:
        buf = free.pop(fits[0])
    elif capturing:
        raise RuntimeError("matmul_set: this call needs a new scratch area, which cannot be made while the stream is "
                           "capturing; run it once eagerly (any stream of this device) before the capture")
    else:
        buf = torch.zeros((max(need, SCRATCH_BYTES),), dtype=torch.uint8, device=device)
    _set_scratch[key] = buf
    return buf


def reset_scratch() -> None:
    """Forget every scratch area (after ``device_error`` reported a lost wait their counters may be non-zero)."""

    _set_scratch.clear()
    _free_areas.clear()


def matmul_set(x: torch.Tensor, qs, xs: torch.Tensor | None = None, *, sks=None, f32: bool = False, outs=None,
               pdl: bool = False) -> list:
    """Several projections of the SAME rows (q/k/v, gate/up) in one persistent launch: [x @ q.T for q in qs], each with
    the bits ``matmul(x, q, sk=sk)`` gives.  1 to 16 rows, up to 4 weights of one format and K.  Not in the reference,
    whose engines issue these as separate calls (families/qwen3_5/cuda/qmm_fast.py:49-64)."""

    qs = list(qs)
    if not 1 <= len(qs) <= SET_MAX:
        raise ValueError(f"matmul_set: 1 to {SET_MAX} weights a set")
    q0 = qs[0]
    if any((q.k, q.gs, q.bits) != (q0.k, q0.gs, q0.bits) for q in qs):
        raise ValueError("matmul_set: the weights of a set share K, group and bit width")
    x = _rows(x, q0.k, "matmul_set")
    m = x.shape[0]
    if m > STREAM_ROWS:
        raise ValueError(f"matmul_set: at most {STREAM_ROWS} rows (use matmul for larger windows)")
    stream = _lib.stream_of(x)
    kg = q0.k // q0.gs
    if xs is not None and (xs.dtype != torch.float32 or xs.shape != (m, kg) or not xs.is_contiguous()):
        raise ValueError(f"matmul_set: xs must be contiguous ({m}, {kg}) fp32")
    sks = [sk or default_split(q.n, q.k, q.gs) for q, sk in zip(qs, sks or [None] * len(qs))]
    outs = list(outs) if outs is not None else [None] * len(qs)
    dtype = torch.float32 if f32 else torch.bfloat16
    for i, q in enumerate(qs):
        if q.weight.device != x.device:
            raise ValueError("matmul_set: x and the weights must share a CUDA device")
        if sks[i] < 1 or sks[i] > kg:
            raise ValueError("matmul_set: 1 to K / gs slices (a slice holds one group at least)")
        if q.weight.dim() != 3 or q.weight.stride(2) != 1 or q.weight.stride(1) != q.weight.shape[2]:
            raise ValueError("matmul_set: the tiled weight may be sliced by super-blocks of 128 columns only")
        if outs[i] is None:
            outs[i] = torch.empty((m, q.n), dtype=dtype, device=x.device)
        elif outs[i].shape != (m, q.n) or outs[i].dtype != dtype or outs[i].stride(1) != 1:
            raise ValueError("matmul_set: out must be (M, n) of the requested dtype with unit-stride rows")
    count = len(qs)
    ints, longs, ptrs = ctypes.c_int * count, ctypes.c_int64 * count, ctypes.c_void_p * count
    n_arr, sk_arr = ints(*[q.n for q in qs]), ints(*sks)
    lib = _lib.lib()
    need = lib.tf_qmm_set_scratch_bytes(count, n_arr, sk_arr)
    if need < 0:
        raise ValueError("matmul_set: bad shapes")
    scratch = _scratch_for(x.device, stream, need)
    _lib.check(lib.tf_qmm_set(
        x.data_ptr(), x.stride(0), m, xs.data_ptr() if xs is not None else None, q0.k, q0.bits, q0.gs, count,
        ptrs(*[q.weight.data_ptr() for q in qs]), longs(*[q.weight.stride(0) for q in qs]), n_arr, sk_arr,
        ptrs(*[o.data_ptr() for o in outs]), longs(*[o.stride(0) for o in outs]), int(f32), scratch.data_ptr(),
        scratch.numel(), int(pdl), stream), "matmul_set")
    return outs


def prefill_matmul(x: torch.Tensor, q: Q4, *, f32: bool = False, tile: int = 0,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """Prefill: weights rounded once to bf16, one fp32 chain over K on the tcgen05 tensor cores; any chunking gives the
    same bits, not decode's.  ``tile`` is accepted for signature parity (cuda/kernels/qmm.py:160) and unused.  Formats
    the tcgen05 kernel does not take (other widths, groups of 128, K not a multiple of 64) run through ``matmul``."""

    x = _rows(x, q.k, "prefill_matmul")
    if q.bits != 4 or q.gs not in (32, 64) or q.k % 64:
        return matmul(x, q, f32=f32, out=out)
    m = x.shape[0]
    stream = _lib.stream_of(x)
    if out is None:
        out = torch.empty((m, q.n), dtype=torch.float32 if f32 else torch.bfloat16, device=x.device)
    elif out.shape != (m, q.n) or out.dtype != (torch.float32 if f32 else torch.bfloat16) or out.stride(1) != 1:
        raise ValueError("prefill_matmul: out must be (M, n) of the requested dtype with unit-stride rows")
    _lib.check(_lib.lib().tf_qmm_prefill(x.data_ptr(), x.stride(0), m, q.weight.data_ptr(), q.weight.stride(0), q.n, q.k, q.gs,
                                         out.data_ptr(), out.stride(0), int(f32), stream), "prefill_matmul")
    return out


_side_streams: dict = {}


def fork_join(calls) -> None:
    """Runs independent launches side by side: ``calls`` are thunks that launch on the current stream (projections that
    read the same input, like q/k/v or gate/up).  The first runs on the current stream, the others on side streams that
    wait for everything already queued on it; the current stream then waits for all of them.  Works eagerly and under
    CUDA-graph capture (the waits become graph edges).  A decode-sized projection cannot fill the GPU on its own (its
    launch, first-byte latency and slice reduction are fixed costs), so independent ones overlap nearly for free.

    Tensors a thunk allocates belong to its side stream's pool: give the thunks preallocated outputs (``out=``) for
    anything the main stream reads after the join, or call ``record_stream(main)`` on what they return; a tensor made
    and consumed inside one thunk needs neither."""

    calls = list(calls)
    if len(calls) < 2:
        for fn in calls:
            fn()
        return
    main = torch.cuda.current_stream()
    pool = _side_streams.setdefault(main.device, [])
    while len(pool) < len(calls) - 1:
        pool.append(torch.cuda.Stream(device=main.device))
    fork = torch.cuda.Event()
    fork.record(main)
    calls[0]()
    for fn, side in zip(calls[1:], pool):
        side.wait_event(fork)
        with torch.cuda.stream(side):
            fn()
        done = torch.cuda.Event()
        done.record(side)
        main.wait_event(done)


def pack_pair(gate: tuple, up: tuple, gs: int, bits: int = 4) -> Q4:
    """Gate and up projections (each MLX words, scales, biases of n rows) as ONE weight of 2 n rows that interleaves 16
    gate rows with 16 up rows, so a matmul tile pair holds both halves of every SwiGLU output (see ``matmul_act``)."""

    (wg, sg, bg), (wu, su, bu) = gate, up
    if wg.shape != wu.shape or sg.shape != su.shape or wg.dim() != 2:
        raise ValueError("pack_pair: gate and up must have the same 2-D shapes")
    n, words = wg.shape
    k = words * 32 // bits
    if n % 16 or k % gs or any(t.dtype != torch.bfloat16 for t in (sg, bg, su, bu)):
        raise ValueError("pack_pair: rows in whole 16-row tiles, bf16 scales and biases")
    stream = _lib.stream_of(wg)
    ts = [t.contiguous() for t in (wg, sg, bg, wu, su, bu)]
    lib = _lib.lib()
    out = torch.empty((-(-2 * n // 128), k // gs, lib.tf_unit_words(bits, gs)), dtype=torch.int32, device=wg.device)
    _lib.check(lib.tf_pack_pair(*[t.data_ptr() for t in ts], n, k, bits, gs, out.data_ptr(), stream), "pack_pair")
    return Q4(out, None, None, 2 * n, k, gs, bits)


def matmul_act(x: torch.Tensor, q: Q4, *, act: str = "swiglu", limit: float = 0.0, out: torch.Tensor | None = None,
               pdl: bool = False, prefill: bool = False) -> torch.Tensor:
    """Projection with the experts' activation epilogue, dense form: ``act="swiglu"`` on a ``pack_pair`` weight gives
    bf16(bf16(silu(bf16 gate)) * bf16 up) as (M, n / 2); ``act="relu2"`` gives bf16(relu(bf16 v)^2) as (M, n)."""

    x = _rows(x, q.k, "matmul_act")
    if act not in ("swiglu", "relu2"):
        raise ValueError("matmul_act: act is 'swiglu' or 'relu2'")
    m = x.shape[0]
    stream = _lib.stream_of(x)
    ncols = q.n // 2 if act == "swiglu" else q.n
    if out is None:
        out = torch.empty((m, ncols), dtype=torch.bfloat16, device=x.device)
    elif out.shape != (m, ncols) or out.dtype != torch.bfloat16 or out.stride(1) != 1:
        raise ValueError("matmul_act: out must be (M, columns) bf16 with unit-stride rows")
    if prefill and q.bits == 4 and q.gs in (32, 64):          # the prefill arithmetic (weights rounded once to bf16)
        _lib.check(_lib.lib().tf_qmm_prefill_act(x.data_ptr(), x.stride(0), m, q.weight.data_ptr(), q.weight.stride(0), q.n, q.k,
                                                 q.gs, out.data_ptr(), out.stride(0), 0, 2 if act == "swiglu" else 1,
                                                 float(limit), stream), "matmul_act (prefill)")
        return out
    _lib.check(_lib.lib().tf_qmm_act(x.data_ptr(), x.stride(0), m, q.weight.data_ptr(), q.weight.stride(0), q.n, q.k, q.bits,
                                     q.gs, out.data_ptr(), out.stride(0), 2 if act == "swiglu" else 1, float(limit), int(pdl),
                                     stream), "matmul_act")
    return out
