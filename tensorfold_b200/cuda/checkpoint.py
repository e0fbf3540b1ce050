"""Checkpoint -> device load path for quantized projections: safetensors files read by byte range, a rank reading only
the bytes it owns, the result handed to the tiling kernel.

Mirrors what the reference spreads over ``cuda/direct_read.py:26-176`` (O_DIRECT span reader, safetensors index),
``families/qwen3_5/cuda/weights.py:280-303`` (per-tensor repack) and ``families/glm5_next/cuda/split.py:74-229``
(rank-aware byte ranges): a column-parallel projection's shard is a run of whole rows of ``weight``, ``scales`` and
``biases``, so each rank reads three contiguous ranges per segment and nothing else; a row-parallel shard is a run of
whole words and groups inside every row, which is read with the rows and cut on the device.  Values are never touched:
the shards are bit-for-bit what ``distributed.split_output`` / ``split_input`` cut from the whole tensors.
"""

from __future__ import annotations

import errno
import json
import os
import struct
from dataclasses import dataclass
from pathlib import Path
from typing import Sequence

import torch

from ..families.qwen3_5.cuda.weights import QLinear
from .kernels import affine

ALIGN = 4096              # O_DIRECT wants file offsets, lengths and buffer addresses on this grid
PIECE = 32 << 20          # bytes a direct read fills at a time (and a page-locked piece holds on the way to a GPU)

DTYPES = {"BOOL": torch.bool, "U8": torch.uint8, "I8": torch.int8, "U16": torch.uint16, "I16": torch.int16,
          "U32": torch.uint32, "I32": torch.int32, "U64": torch.uint64, "I64": torch.int64, "F16": torch.float16,
          "BF16": torch.bfloat16, "F32": torch.float32, "F64": torch.float64}


def _grid_up(v: int) -> int:
    return -(-v // ALIGN) * ALIGN


class Spans:
    """Byte ranges of files as uint8 tensors.  Reads go around the page cache (O_DIRECT) while the file system accepts
    that, through it otherwise (``direct`` turns False on the first refusal); ``bytes_read`` counts what was asked for."""

    def __init__(self, direct: bool = True) -> None:
        self.direct = direct and hasattr(os, "O_DIRECT")
        self.bytes_read = 0

    # ------------------------------------------------------------------ host
    def read(self, path: str | Path, offset: int, n: int, *, pinned: bool = False) -> torch.Tensor:
        """Bytes [offset, offset + n) of ``path`` on the host (page-locked when ``pinned`` and CUDA is present)."""

        if offset < 0 or n < 0:
            raise ValueError("negative byte range")
        self.bytes_read += n
        size = os.path.getsize(path)
        if offset + n > size:
            raise IOError(f"{path}: bytes {offset}-{offset + n} lie past its end ({size})")
        pinned = pinned and torch.cuda.is_available()
        if n and self.direct:
            try:
                return self._direct(path, offset, n, size, pinned)
            except OSError as exc:
                if exc.errno != errno.EINVAL:
                    raise
                self.direct = False               # refused on open or on a read: the page cache from now on
        out = torch.empty((n,), dtype=torch.uint8, pin_memory=pinned)
        view = memoryview(out.numpy())
        with open(path, "rb", buffering=0) as f:
            f.seek(offset)
            at = 0
            while at < n:
                got = f.readinto(view[at:at + PIECE])
                if not got:
                    raise IOError(f"{path}: short read at {offset + at}")
                at += got
        return out

    def _direct(self, path, offset: int, n: int, size: int, pinned: bool) -> torch.Tensor:
        lo = offset // ALIGN * ALIGN
        hi = min(_grid_up(offset + n), _grid_up(size))
        block = torch.empty((hi - lo + 2 * ALIGN,), dtype=torch.uint8, pin_memory=pinned)
        lead = -block.data_ptr() % ALIGN          # the allocation need not sit on the grid: the span inside it does
        span = memoryview(block.numpy())[lead:lead + hi - lo]
        fd = os.open(path, os.O_RDONLY | os.O_DIRECT)
        try:
            self._fill(fd, span, lo, offset - lo + n, path)
        finally:
            os.close(fd)
        out = block[lead + offset - lo:lead + offset - lo + n]
        return out if pinned or out.data_ptr() % 16 == 0 else out.clone()     # typed views want an aligned start

    @staticmethod
    def _fill(fd: int, span: memoryview, lo: int, need: int, path) -> None:
        """Aligned reads of at most PIECE bytes into ``span`` (which starts at file offset ``lo``) until ``need`` bytes
        are there; the last read may run past the end of the file and comes back short."""

        at = 0
        while at < need:
            got = os.preadv(fd, [span[at:at + PIECE]], lo + at)
            if got <= 0:
                raise IOError(f"{path}: short read at {lo + at}")
            at += got

    # ------------------------------------------------------------------ device
    def upload(self, path: str | Path, offset: int, n: int, device: torch.device | str) -> torch.Tensor:
        """The same bytes as a new uint8 tensor on ``device``: for a CUDA device, page-locked pieces of at most PIECE
        bytes are read and copied one after another (host memory stays bounded whatever the tensor's size)."""

        device = torch.device(device)
        if device.type != "cuda":
            return self.read(path, offset, n)
        out = torch.empty((n,), dtype=torch.uint8, device=device)
        for at in range(0, n, PIECE):
            take = min(PIECE, n - at)
            out[at:at + take].copy_(self.read(path, offset + at, take, pinned=True))
        return out

    def close(self) -> None:
        """Nothing is held between calls; kept so callers can treat the reader like the reference's."""


def read_header(path: str | Path) -> tuple[int, dict]:
    """(file offset where the tensor data starts, the JSON header) of a safetensors file."""

    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) != 8:
            raise IOError(f"{path}: not a safetensors file (no header length)")
        n = struct.unpack("<Q", head)[0]
        raw = f.read(n)
        if len(raw) != n:
            raise IOError(f"{path}: header of {n} bytes is cut short")
    return 8 + n, json.loads(raw)


@dataclass(frozen=True)
class Entry:
    path: Path
    begin: int                # file offset of the tensor's first byte
    nbytes: int
    dtype: torch.dtype
    shape: tuple[int, ...]

    @property
    def row_bytes(self) -> int:
        return self.nbytes // self.shape[0] if self.shape and self.shape[0] else 0


class Checkpoint:
    """Tensors of a set of safetensors files by name (a later file's name wins), whole, by row range, or as the
    quantized projection a rank owns."""

    def __init__(self, files: Sequence[str | Path], spans: Spans | None = None) -> None:
        self.spans = spans or Spans()
        self.index: dict[str, Entry] = {}
        for path in files:
            base, header = read_header(path)
            size = os.path.getsize(path)
            for name, e in header.items():
                if name == "__metadata__":
                    continue
                if e["dtype"] not in DTYPES:
                    raise ValueError(f"{name}: safetensors dtype {e['dtype']} is not supported")
                begin, end = e["data_offsets"]
                dtype, shape = DTYPES[e["dtype"]], tuple(int(v) for v in e["shape"])
                count = 1
                for v in shape:
                    count *= v
                if end - begin != count * torch.empty((), dtype=dtype).element_size() or base + end > size:
                    raise ValueError(f"{name}: byte range {begin}-{end} does not hold {shape} of {e['dtype']} inside {path}")
                self.index[name] = Entry(Path(path), base + begin, end - begin, dtype, shape)

    def keys(self) -> list[str]:
        return list(self.index)

    def __contains__(self, name: str) -> bool:
        return name in self.index

    def close(self) -> None:
        self.spans.close()

    def _typed(self, raw: torch.Tensor, e: Entry, shape) -> torch.Tensor:
        return raw.view(e.dtype).reshape(shape)

    def tensor(self, name: str, device: torch.device | str = "cpu") -> torch.Tensor:
        e = self.index[name]
        return self._typed(self.spans.upload(e.path, e.begin, e.nbytes, device), e, e.shape)

    def rows(self, name: str, lo: int, hi: int, device: torch.device | str = "cpu") -> torch.Tensor:
        """Rows [lo, hi) of a tensor with at least one dimension: one contiguous byte range of the file."""

        e = self.index[name]
        if not e.shape or not 0 <= lo <= hi <= e.shape[0]:
            raise ValueError(f"{name}: rows {lo}-{hi} outside {e.shape}")
        raw = self.spans.upload(e.path, e.begin + lo * e.row_bytes, (hi - lo) * e.row_bytes, device)
        return self._typed(raw, e, (hi - lo,) + e.shape[1:])

    def linear(self, prefix: str, *, bits: int = 4, gs: int = 64, device: torch.device | str = "cpu", rank: int = 0,
               world: int = 1, parallel: str | None = None, segments: Sequence[int] | None = None,
               block: int = 1) -> QLinear:
        """``prefix``.weight / .scales / .biases as the QLinear rank ``rank`` of ``world`` owns: ``parallel`` "column"
        (whole output rows; ``segments`` and ``block`` as in ``distributed.output_rows``), "row" (whole words and
        groups of every row) or None (the whole projection)."""

        names = [f"{prefix}.weight", f"{prefix}.scales", f"{prefix}.biases"]
        for name in names:
            if name not in self.index:
                raise KeyError(name)
        w, s, b = (self.index[name] for name in names)
        if len(w.shape) != 2 or s.shape != b.shape or len(s.shape) != 2 or s.shape[0] != w.shape[0]:
            raise ValueError(f"{prefix}: weight {w.shape}, scales {s.shape}, biases {b.shape} are not one projection")
        n, k = affine.packed_shape(w.shape, s.shape, b.shape, bits, gs)     # raises when the shapes are not this format
        if parallel is None or world == 1:
            parts = [self.tensor(name, device) for name in names]
        elif parallel == "column":
            lengths = tuple(segments) if segments is not None else (n,)
            if sum(lengths) != n or any(v <= 0 or v % (world * block) for v in lengths):
                raise ValueError(f"output segments {lengths} do not split into {world} blocks of {block}")
            if not 0 <= rank < world:
                raise ValueError("rank outside the world")
            parts = []
            for name in names:
                runs, base = [], 0
                for length in lengths:
                    share = length // world
                    runs.append(self.rows(name, base + rank * share, base + (rank + 1) * share, device))
                    base += length
                parts.append(runs[0] if len(runs) == 1 else torch.cat(runs))
        elif parallel == "row":
            (w0, w1), (g0, g1) = affine.input_slice(k, bits, gs, rank, world)
            whole = [self.tensor(name, device) for name in names]
            parts = [whole[0][:, w0:w1].contiguous(), whole[1][:, g0:g1].contiguous(), whole[2][:, g0:g1].contiguous()]
        else:
            raise ValueError("parallel is None, 'column' or 'row'")
        weight = parts[0].view(torch.int32) if parts[0].dtype == torch.uint32 else parts[0]
        return QLinear(weight, parts[1], parts[2], gs=gs, bits=bits)


def expert_tables(ckpt: Checkpoint, prefix: str, projections: Sequence[str] = ("gate_proj", "up_proj", "down_proj"), *,
                  device: torch.device | str = "cpu", rank: int = 0, world: int = 1):
    """A routed layer's expert tables ``prefix.<projection>.weight / .scales / .biases`` of shape [E, ...] as the
    experts rank ``rank`` of ``world`` owns, [rank E / world, (rank + 1) E / world): the experts are the tensors' first
    dimension, so a rank's share is one contiguous byte range per tensor and only that is read.  Returns
    ({projection: (words, scales, biases)}, first): what ``tp.shard_experts`` cuts from the whole tables
    (reference: families/qwen3_5_moe/cuda/weights.py:32-46 reads them whole)."""

    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank outside the world")
    tables, first = {}, 0
    for proj in projections:
        names = [f"{prefix}.{proj}.{part}" for part in ("weight", "scales", "biases")]
        for name in names:
            if name not in ckpt:
                raise KeyError(name)
        e = ckpt.index[names[0]].shape[0]
        if any(ckpt.index[name].shape[0] != e for name in names) or e % world:
            raise ValueError(f"{prefix}.{proj}: {e} experts do not divide across {world} ranks")
        first = rank * e // world
        parts = [ckpt.rows(name, first, (rank + 1) * e // world, device) for name in names]
        words = parts[0].view(torch.int32) if parts[0].dtype == torch.uint32 else parts[0]
        tables[proj] = (words, parts[1], parts[2])
    return tables, first


def load_experts(ckpt: Checkpoint, prefix: str, device: torch.device | str, gs: int = 64, *, rank: int = 0, world: int = 1,
                 limit: float = 0.0):
    """The rank's experts of a SwiGLU layer, uploaded and tiled for the grouped kernels: (``experts.Experts``, first)."""

    from . import experts

    tables, first = expert_tables(ckpt, prefix, device=device, rank=rank, world=world)
    return experts.make([tables["gate_proj"], tables["up_proj"]], tables["down_proj"], gs, limit=limit), first


def load_packed(ckpt: Checkpoint, prefix: str, device: torch.device | str, **kw):
    """The rank's shard of a projection, uploaded and tiled for the kernels (``kernels.qmm.pack``)."""

    from .kernels import qmm

    q = ckpt.linear(prefix, device=device, **kw)
    return qmm.pack(q.weight, q.scales, q.biases, q.gs, bits=q.bits)


__all__ = ["ALIGN", "PIECE", "Spans", "read_header", "Entry", "Checkpoint", "expert_tables", "load_experts", "load_packed"]
