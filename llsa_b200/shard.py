"""Host logic for running the LLSA operators on several GPUs of one box.

Every (batch, head) slice of llsa_l1 / llsa_l2 is independent in all stages
(the reference's grids are all `(…, B*H)`, e.g. sparse_attention_res_2.py:179),
so the work shards over ranks along the flattened B*H axis with no collective
on the data path; a collective is needed only to hand a caller the full output
when it asks for it (`gather_slices`).
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple

import torch
import torch.distributed as dist

__all__ = ["slice_range", "take_slices", "gather_slices", "sharded_call"]


def slice_range(n_slices: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) range of the flattened (b,h) axis owned by `rank`;
    sizes differ by at most one and the ranges tile [0, n_slices) in rank order."""
    if not (0 <= rank < world):
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, rem = divmod(n_slices, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def take_slices(x: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """The rank's (b,h) slices of a [B,H,N,D] tensor as [1, n_local, N, D] (a view when B*H is flattenable)."""
    B, H, N, D = x.shape
    begin, end = slice_range(B * H, world, rank)
    return x.reshape(1, B * H, N, D)[:, begin:end]


def gather_slices(local: torch.Tensor, B: int, H: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gathers per-rank [1, n_local, N, D] results back into [B,H,N,D] on every rank."""
    world = dist.get_world_size(group)
    N, D = local.shape[2], local.shape[3]
    sizes = [e - b for b, e in (slice_range(B * H, world, r) for r in range(world))]
    widest = max(sizes)
    if local.shape[1] < widest:      # all_gather wants equal shapes: pad the short ranks, trim afterwards
        local = torch.cat([local, local.new_zeros((1, widest - local.shape[1], N, D))], 1)
    parts: List[torch.Tensor] = [local.new_empty((1, widest, N, D)) for _ in sizes]
    dist.all_gather(parts, local.contiguous(), group=group)
    return torch.cat([p[:, :n] for p, n in zip(parts, sizes)], 1).reshape(B, H, N, D)


def sharded_call(fn: Callable[..., torch.Tensor], q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *args,
                 group: Optional[dist.ProcessGroup] = None, gather: bool = True, **kwargs) -> torch.Tensor:
    """Runs `fn(q, k, v, *args)` (llsa_l1 / llsa_l2 or any per-slice attention) on this rank's
    (b,h) slices of replicated inputs; returns the full output when `gather`, else the local part."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    B, H = q.shape[:2]
    o = fn(take_slices(q, world, rank), take_slices(k, world, rank), take_slices(v, world, rank), *args, **kwargs)
    return gather_slices(o, B, H, group) if gather else o
