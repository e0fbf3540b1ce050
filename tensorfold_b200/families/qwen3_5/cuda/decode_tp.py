"""The head of a tensor-parallel decode step when the vocabulary rows are split across ranks: every rank holds whole
dot products of its rows (so logits keep their bits) and hands over just enough local candidates for rank 0 to choose
exactly as one GPU would.  Mirrors ``split_candidates`` of families/qwen3_5/cuda/decode_tp.py:72-80 of the reference;
the sampling rules that consume the candidates stay in the engine."""

from __future__ import annotations

from dataclasses import dataclass

import torch

MARGIN = 8     # candidates beyond top_k a rank hands over, so that tied values still resolve by id (engine/exact_sampling.py:13)


@dataclass(frozen=True)
class Sampling:
    """The fields of the engine's sampling record that decide how many candidates are needed."""

    seed: int = 0
    temperature: float = 1.0
    top_k: int = 20
    top_p: float = 0.95
    min_p: float = 0.0


def split_candidates(logits: torch.Tensor, sampling, offset: int) -> tuple[torch.Tensor, torch.Tensor]:
    """This rank's candidates for rows of ``logits`` [R, V_local] whose first column is vocabulary id ``offset``: the
    first local maximum when greedy (``sampling`` None or temperature <= 0), otherwise top_k + MARGIN local values
    (all of them without a top_k): enough to contain the global top-k.  Returns (values fp32, global ids)."""

    if sampling is None or sampling.temperature <= 0:
        values, ids = logits.float().max(dim=-1)
        return values[:, None].contiguous(), (ids + offset)[:, None].contiguous()
    count = min(logits.shape[1], int(sampling.top_k) + MARGIN) if sampling.top_k else logits.shape[1]
    values, ids = torch.topk(logits.float(), count, dim=-1, sorted=False)
    return values.contiguous(), (ids + offset).contiguous()


def head_logits(x: torch.Tensor, head, rank: int, world_size: int):
    """Logits of this rank's vocabulary rows and the id of its first row: ``head`` is the rank's share of the
    quantised head (``distributed.split_weights(..., split_head=True)``), run as one matmul."""

    from . import qmm_fast

    return qmm_fast.matmul(x, head), rank * head.n


def gather_candidates(values: torch.Tensor, ids: torch.Tensor, comm) -> tuple[torch.Tensor, torch.Tensor]:
    """Every rank's candidates side by side, rank 0's first: ([R, world * C] values, ids).  ``comm`` is a
    ``tensorfold_b200.cuda.comm.Comm``; the reference gathers its two ranks the same way
    (families/qwen3_5/cuda/decode_tp.py:96-104)."""

    rows, count = values.shape
    ids = ids.to(torch.int64)
    all_values = torch.empty((comm.world, rows, count), dtype=values.dtype, device=values.device)
    all_ids = torch.empty((comm.world, rows, count), dtype=ids.dtype, device=ids.device)
    comm.all_gather(values.contiguous(), all_values)
    comm.all_gather(ids.contiguous(), all_ids)
    side_by_side = lambda t: t.permute(1, 0, 2).reshape(rows, comm.world * count)
    return side_by_side(all_values), side_by_side(all_ids)


def greedy_merged(values: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """The whole vocabulary's first maximum from the ranks' local maxima (one candidate a rank, rank order = id order):
    the earliest rank that holds the largest value wins, as ``argmax`` over the unsplit logits would choose."""

    best = values.argmax(dim=1, keepdim=True)               # torch returns the first of equal maxima
    return ids.gather(1, best)[:, 0]
