"""Tensor- and expert-parallel layers over the GPUs of one NVLink/NVSwitch box (1, 2, 4 or 8 ranks, one process each).

Column-parallel projections own whole output rows, row-parallel ones whole quantization groups of the inputs
(families/qwen3_5/cuda/distributed.py of the reference, two ranks there); every partial sum is reduced in rank order
((p0 + p1) + p2 ...) in fp32 and rounded once, so all ranks hold the same bits and a row's bits do not depend on the row
count.  The routed MoE block is expert-parallel without an all-to-all: activations are replicated, every rank routes all
rows, keeps the pairs whose expert it owns, and contributes a partial [M, D] (the reference splits every expert's width
across its two ranks instead, families/nemotron_h/cuda/tp.py:38-51)."""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _lib
from . import experts as grouped
from . import moe
from .kernels import qmm
from ..families.qwen3_5.cuda import distributed
from ..families.qwen3_5.cuda.weights import QLinear

GATHER_LIMIT = 1 << 20          # partials up to this many bytes take one all-gather; larger ones exchange shares first


def ordered_all_reduce(local: torch.Tensor, group=None, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """Sum of every rank's ``local`` [M, N] (fp32 or bf16) in rank order, fp32 adds, one rounding to ``dtype``.

    Small partials: one all-gather, then each rank adds all of them.  Large ones: every rank receives one share of each
    partial (all-to-all), adds its shares in rank order, and the finished shares are all-gathered: the bytes of a ring
    all-reduce with a fixed summation order.  Both give the same bits."""

    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return local.to(dtype)
    local = local.contiguous()
    total = local.numel()
    if total * local.element_size() <= GATHER_LIMIT or total % world:
        return distributed.gather_rank_partials(local, group, dtype)
    share = total // world
    recv = torch.empty((world, share), dtype=local.dtype, device=local.device)
    dist.all_to_all_single(recv.view(-1), local.view(-1), group=group)
    mine = distributed._ordered_sum(recv, dtype)
    out = torch.empty((total,), dtype=dtype, device=local.device)
    dist.all_gather_into_tensor(out, mine.view(-1), group=group)
    return out.view(local.shape)


class _Raw:
    """A device address as an object torch can wrap (no copy, no ownership)."""

    def __init__(self, ptr: int, nbytes: int) -> None:
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerReducer:
    """The rank-ordered all-reduce in one launch over peer memory (``tf_peer_reduce``): every rank owns one buffer that the
    other processes of the box map, producers write their partial straight into it (``partial``), and ``reduce`` returns
    the sum, the bits ``ordered_all_reduce`` gives.  Buffers: [flags | partial | result | slots].  Partials of up to
    ``flagged_up_to`` bytes travel as flagged words (no barrier; whole partials to every rank, or shares in two hops on
    four and eight ranks); larger ones in shares between two barriers (a rank sums 1/world and stores it to every rank).

    The result tensor is a view of the buffer: it is overwritten by the next ``reduce``, and so is the partial."""

    ALL, SHARES, FLAGGED, FLAGGED_PUSH, FLAGGED_PULL, HOPS, HOPS_SEND, HOPS_MIDDLE, HOPS_COLLECT = range(9)
    HOPS_FROM = 64 << 10        # partial bytes from which four or eight ranks exchange shares in two hops of flagged words

    def __init__(self, elements: int, group=None, *, device=None, flagged_up_to: int = 1 << 19, bufs: list[int] | None = None,
                 rank: int | None = None) -> None:
        lib = _lib.lib()
        self.group, self.elements, self.flagged_up_to = group, elements, flagged_up_to
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.world = len(bufs) if bufs is not None else dist.get_world_size(group)
        self.flags, self.part_off, self.out_off, self.ll_off, self.ll_slot, self.nbytes = self.layout(elements, self.world, flagged_up_to)
        self.force: int | None = None                          # a form for every call (tests)
        self._opened: list[int] = []
        self._owned = 0
        if bufs is not None:                                   # buffers made by the caller (one process driving them all)
            self.rank, self.bufs = rank, list(bufs)
        else:
            self.rank = dist.get_rank(group)
            with torch.cuda.device(self.device):
                self._owned = self.alloc(self.nbytes)
                handle = ctypes.create_string_buffer(64)
                _lib.check(lib.tf_peer_export(self._owned, handle), "peer export")
                handles = [None] * self.world
                dist.all_gather_object(handles, handle.raw, group=group)
                self.bufs = []
                for r, h in enumerate(handles):
                    if r == self.rank:
                        self.bufs.append(self._owned)
                        continue
                    ptr = ctypes.c_void_p()
                    _lib.check(lib.tf_peer_open(h, ctypes.byref(ptr)), f"peer open (rank {r})")
                    self._opened.append(ptr.value)
                    self.bufs.append(ptr.value)
                dist.barrier(group)                            # every buffer is mapped before anyone signals
        self._table = (ctypes.c_void_p * self.world)(*self.bufs)
        self._mine = torch.as_tensor(_Raw(self.bufs[self.rank], self.nbytes), device=self.device)
        self._views: dict[tuple, torch.Tensor] = {}

    @staticmethod
    def layout(elements: int, world: int, flagged_up_to: int = 1 << 19) -> tuple[int, int, int, int, int, int]:
        """Bytes of the flags, offsets of the partial and of the result, offset and size of the slots of flagged words,
        bytes of a whole buffer, for partials of up to ``elements`` fp32 values."""

        flags = int(_lib.lib().tf_peer_flag_bytes())
        room = (-(-elements * 4 // 256)) * 256
        slot = 2 * min(room, (-(-flagged_up_to // 256)) * 256)        # (a multiple of 512: splits into 16-byte pieces a rank)
        ll_off = flags + 2 * room
        return flags, flags, flags + room, ll_off, slot, ll_off + 2 * world * slot

    @staticmethod
    def alloc(nbytes: int) -> int:
        ptr = ctypes.c_void_p()
        _lib.check(_lib.lib().tf_peer_alloc(nbytes, ctypes.byref(ptr)), "peer alloc")
        return ptr.value

    def _view(self, off: int, shape, dtype: torch.dtype) -> torch.Tensor:
        key = (off, tuple(shape), dtype)
        view = self._views.get(key)
        if view is None:
            n = int(torch.Size(shape).numel())
            if n > self.elements or dtype not in (torch.float32, torch.bfloat16):
                raise ValueError("PeerReducer: fp32 or bf16, no more elements than the reducer was made for")
            view = self._views[key] = self._mine[off:off + n * dtype.itemsize].view(dtype).view(shape)
        return view

    def partial(self, shape, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """Where this rank's partial goes: a view of its buffer for the producer to write into."""

        return self._view(self.part_off, shape, dtype)

    def form(self, n: int, itemsize: int) -> int:
        if self.force is not None:
            return self.force
        if n * itemsize <= self.flagged_up_to:
            two_hops = self.world >= 4 and n * itemsize >= self.HOPS_FROM and n % (8 * self.world) == 0
            return self.HOPS if two_hops else self.FLAGGED
        return self.SHARES if n % (8 * self.world) == 0 else self.ALL

    def reduce(self, part: torch.Tensor, dtype: torch.dtype = torch.bfloat16, *, polls: int = 0, grid_cap: int = 0) -> torch.Tensor:
        """Sum of every rank's ``part`` (a tensor from ``partial``; anything else is copied in first)."""

        n = part.numel()
        home = self.partial(part.shape, part.dtype)
        if part.data_ptr() != home.data_ptr() or not part.is_contiguous():
            home.copy_(part)
        _lib.check(_lib.lib().tf_peer_reduce(self._table, self.rank, self.world, self.part_off, self.out_off, n,
                                             int(part.dtype == torch.bfloat16), int(dtype == torch.float32),
                                             self.form(n, part.element_size()), self.ll_off, self.ll_slot, polls, grid_cap,
                                             _lib.stream_of(home)), "peer reduce")
        return self._view(self.out_off, part.shape, dtype)

    def close(self) -> None:
        lib = _lib.lib()
        torch.cuda.synchronize(self.device)
        if self._owned and dist.is_initialized():
            dist.barrier(self.group)                           # no rank unmaps while another may still read
        for ptr in self._opened:
            lib.tf_peer_close(ptr)
        self._opened = []
        if self._owned:
            if dist.is_initialized():
                dist.barrier(self.group)
            lib.tf_peer_free(self._owned)
            self._owned = 0


def shard_experts(raw_up: list[tuple], raw_down: tuple, rank: int, world: int) -> tuple[list[tuple], tuple, int]:
    """Rank's share of the expert tables: experts [rank * E / world, (rank + 1) * E / world)."""

    e = raw_down[0].shape[0]
    if e % world:
        raise ValueError("experts must divide across the ranks")
    a, b = rank * e // world, (rank + 1) * e // world
    cut = lambda m: tuple(t[a:b] for t in m)
    return [cut(m) for m in raw_up], cut(raw_down), a


@dataclass
class ExpertParallelMoE:
    """One rank's share of a routed layer: the full router, the local experts and their first global id."""

    router: torch.Tensor            # [E (+1), D] bf16: every rank routes every row
    experts: grouped.Experts        # local experts only
    top_k: int
    first: int                      # global id of local expert 0
    total: int                      # experts in the whole layer
    has_shared_row: bool = False    # router carries a shared-expert gate row after the experts' (not read here)

    def buffers(self, rows: int, device, *, prefill: bool = False) -> moe.MoEBuffers:
        class _Cfg:
            num_experts_per_tok, num_experts = self.top_k, self.total
            moe_intermediate_size, hidden_size = self.experts.width, self.experts.dims
        return moe.MoEBuffers(rows, _Cfg, device, prefill=prefill, table_experts=self.experts.count)

    def partial(self, x: torch.Tensor, buf: moe.MoEBuffers, out: torch.Tensor | None = None) -> torch.Tensor:
        """This rank's contribution [R, D] bf16: its experts' slots combined, the others weighted zero."""

        rows = x.shape[0]
        logits = buf.logits[:rows]
        form = buf.plan.prefill                                # prompt passes take the tensor-core router, as moe.moe does
        moe.router(x, self.router[:self.total], logits[:, :self.total], prefill=form)
        moe.select_local_rows(logits, buf, self.top_k, self.total, self.first, self.experts.count)
        wts = buf.wts[:rows]
        grouped.route(buf.pick[:rows], buf.plan)
        grouped.gate_up(x, self.experts, buf.plan, buf.act.view(-1, self.experts.width), rows)
        grouped.down(buf.act.view(-1, self.experts.width), self.experts, buf.plan, buf.y.view(-1, self.experts.dims), rows)
        return moe.combine(buf.y[:rows], wts, out)

    def run(self, x: torch.Tensor, buf: moe.MoEBuffers, group=None, reducer: PeerReducer | None = None) -> torch.Tensor:
        if reducer is None:
            return ordered_all_reduce(self.partial(x, buf), group)
        part = reducer.partial((x.shape[0], self.experts.dims))
        return reducer.reduce(self.partial(x, buf, out=part))


@dataclass
class RowParallelLinear:
    """A projection whose inputs are split across ranks in whole groups; ``forward`` reduces the partials."""

    q: qmm.Q4

    @staticmethod
    def shard(q: QLinear, rank: int, world: int) -> "RowParallelLinear":
        part = distributed.split_input(q, rank, world)
        return RowParallelLinear(qmm.pack(part.weight, part.scales, part.biases, part.gs, bits=part.bits))

    def partial(self, x_local: torch.Tensor, *, f32: bool = True) -> torch.Tensor:
        """This rank's share of the sums: fp32, unrounded (``f32=False`` rounds the share to bf16 first: half the
        bytes on the wire, two roundings instead of one, not what the reference does)."""

        return qmm.matmul(x_local, self.q, f32=f32)

    def forward(self, x_local: torch.Tensor, group=None, *, f32: bool = True) -> torch.Tensor:
        """fp32 partials summed in rank order and rounded once (families/qwen3_5/cuda/distributed.py:249-284)."""

        return ordered_all_reduce(self.partial(x_local, f32=f32), group)


@dataclass
class ColumnParallelLinear:
    """A projection whose output rows are split across ranks; no reduction."""

    q: qmm.Q4

    @staticmethod
    def shard(q: QLinear, rank: int, world: int, segments=None, block: int = 1) -> "ColumnParallelLinear":
        part = distributed.split_output(q, rank, world, segments, block)
        return ColumnParallelLinear(qmm.pack(part.weight, part.scales, part.biases, part.gs, bits=part.bits))

    def forward(self, x: torch.Tensor, **kw) -> torch.Tensor:
        return qmm.matmul(x, self.q, **kw)
