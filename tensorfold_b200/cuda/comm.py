"""All-gather on the current stream; a rank-order sum after it keeps every rank bit-equal.

Mirror of the reference's ``tensorfold.cuda.comm`` (cuda/comm.py:35-79), which binds ``ncclAllGather`` through ctypes for
two machines.  Here the ranks are the GPUs of one NVLink/NVSwitch box and the communicator is a ``torch.distributed``
process group (NCCL on GPUs, gloo in CPU tests); the collective still runs on the caller's current stream."""

from __future__ import annotations

import torch
import torch.distributed as dist


class Comm:
    def __init__(self, group=None) -> None:
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed must be initialised (one process per GPU)")
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)

    def all_gather(self, send: torch.Tensor, recv: torch.Tensor) -> None:
        """recv [world * n] <- every rank's send [n], in rank order (contiguous tensors, same dtype)."""

        if recv.numel() != send.numel() * self.world or send.dtype != recv.dtype:
            raise ValueError("all_gather: recv must hold world x send of the same dtype")
        if not send.is_contiguous() or not recv.is_contiguous():
            raise ValueError("all_gather: tensors must be contiguous")
        dist.all_gather_into_tensor(recv.view(-1), send.view(-1), group=self.group)

    def barrier(self) -> None:
        dist.barrier(group=self.group)
