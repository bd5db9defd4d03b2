"""Tensor collectives on the world communicator (reference: pyrannc/tensor_coll.py:1-17, main.cpp:78-136)."""
from __future__ import annotations

import torch

from .parallel import comm


def _allreduce_sum(t: torch.Tensor) -> None:
    comm.allreduce(t, "sum")


def _allreduce_min(t: torch.Tensor) -> None:
    comm.allreduce(t, "min")


def allreduce_tensor(t: torch.Tensor, sum: bool = True) -> None:  # noqa: A002
    comm.allreduce(t, "sum" if sum else "min")


def bcast(t: torch.Tensor, root: int = 0) -> torch.Tensor:
    comm.bcast(t, root)
    return t


def bcast_tensor(t: torch.Tensor, root: int = 0) -> torch.Tensor:
    """The reference's name for :func:`bcast` (main.cpp:96-119)."""
    return bcast(t, root)


def all_gather(t: torch.Tensor, buf: torch.Tensor = None) -> torch.Tensor:
    """Concatenation of every rank's ``t`` along a new leading dimension (flattened into ``buf`` when given)."""
    n = comm.get_world_size()
    if buf is None:
        buf = torch.empty((n,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    comm.allgather_into(buf.view(-1), t.contiguous().view(-1))
    return buf
