"""(batch x head) partition across the GPUs of one box.

Every stage of the path (m/l, block lists, sparse attention) is independent per (batch, head)
unit, so ranks own contiguous unit ranges and never exchange data on the hot path.  The only
collective is the optional all-gather of per-rank outputs when a caller wants the whole tensor.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from .synth import shard_heads


def local_units(total_units: int, group: Optional[dist.ProcessGroup] = None) -> range:
    """Units [start, stop) of this rank under the contiguous split."""
    return shard_heads(total_units, dist.get_world_size(group), dist.get_rank(group))


def all_gather_units(local: torch.Tensor, total_units: int, group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Gather per-rank tensors [n_local_units, ...] into [total_units, ...] on every rank.

    Equal splits use one all_gather_into_tensor (NCCL on GPUs); uneven splits pad each shard to the
    largest one first.  Not part of any timed kernel path."""
    world = dist.get_world_size(group)
    sizes = [len(shard_heads(total_units, world, r)) for r in range(world)]
    assert local.shape[0] == sizes[dist.get_rank(group)], "local shard does not match the contiguous split"
    biggest = max(sizes)
    if min(sizes) == biggest:
        out = torch.empty((total_units,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    pad = torch.zeros((biggest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([p[:n] for p, n in zip(parts, sizes)], dim=0)
