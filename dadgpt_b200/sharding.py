"""Sharding of the (batch x head) axis across ranks.

Every (batch, head) unit of causal attention is independent (the reference's kernels index them
with blockIdx.y, cuda/attention.cu:23,100,165), so ranks never exchange data inside the path.
A rank owns a contiguous range of units; `unit0` (the global index of its first unit) is what
the kernels need to draw the same dropout mask as an unsharded run. The only collective is an
all-gather of results *after* the computation, used by verification.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass(frozen=True)
class UnitShard:
    unit0: int   # global index of the first unit owned by this rank
    count: int   # number of units owned

    @property
    def units(self) -> slice:
        return slice(self.unit0, self.unit0 + self.count)


def shard_units(total_units: int, world: int, rank: int) -> UnitShard:
    """Contiguous, balanced split: the first (total % world) ranks get one extra unit."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    if total_units < 0:
        raise ValueError("negative unit count")
    base, extra = divmod(total_units, world)
    count = base + (1 if rank < extra else 0)
    unit0 = rank * base + min(rank, extra)
    return UnitShard(unit0, count)


def all_gather_units(local: torch.Tensor, total_units: int, group=None) -> torch.Tensor:
    """Gathers per-rank [count, ...] slices into the full [total_units, ...] tensor on every rank
    (NCCL over NVLink for CUDA tensors, gloo for CPU tensors). Ragged splits are padded to the
    largest shard for the collective and trimmed afterwards."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    shards = [shard_units(total_units, world, r) for r in range(world)]
    if local.shape[0] != shards[rank].count:
        raise ValueError(f"rank {rank} holds {local.shape[0]} units, expected {shards[rank].count}")
    biggest = max(s.count for s in shards)
    padded = local
    if local.shape[0] < biggest:
        pad = torch.zeros((biggest - local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype,
                          device=local.device)
        padded = torch.cat([local, pad])
    buf = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(buf, padded.contiguous(), group=group)
    return torch.cat([b[:s.count] for b, s in zip(buf, shards)])
