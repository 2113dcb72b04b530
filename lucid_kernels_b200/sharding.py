"""Sharding of the independent (batch, head) systems across ranks.

Every (batch, head) pair is its own triangular system, so the path needs no exchange: rank r of W owns
a contiguous slice of the flattened index hb = b*H + h and runs the single-GPU kernels on it.  A
collective (all-gather) is used only to reassemble outputs for validation.
"""
from __future__ import annotations

from typing import List, Tuple

import torch


def shard_range(num_systems: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Half-open range of systems owned by `rank`; the first (num_systems % world_size) ranks own one more."""
    assert 0 <= rank < world_size and num_systems >= 0
    base, extra = divmod(num_systems, world_size)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def all_ranges(num_systems: int, world_size: int) -> List[Tuple[int, int]]:
    return [shard_range(num_systems, world_size, r) for r in range(world_size)]


def to_systems(x: torch.Tensor) -> torch.Tensor:
    """(B, N, H, D) -> (1, N, B*H, D) view-or-copy with systems ordered hb = b*H + h."""
    B, N, H, D = x.shape
    return x.permute(1, 0, 2, 3).reshape(1, N, B * H, D)


def from_systems(x: torch.Tensor, B: int, H: int) -> torch.Tensor:
    """Inverse of `to_systems`."""
    _, N, BH, D = x.shape
    assert BH == B * H
    return x.reshape(N, B, H, D).permute(1, 0, 2, 3)


def take_shard(x: torch.Tensor, world_size: int, rank: int) -> torch.Tensor:
    """The (1, N, n_local, D) shard of a (B, N, H, D) tensor owned by `rank`."""
    sys = to_systems(x)
    lo, hi = shard_range(sys.shape[2], world_size, rank)
    return sys[:, :, lo:hi].contiguous()


def gather_shards(local: torch.Tensor, B: int, H: int, group=None) -> torch.Tensor:
    """All-gather (1, N, n_local, D) shards into the full (B, N, H, D) tensor (validation only).
    Shards may differ in size; each is padded to the largest for the collective."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    ranges = all_ranges(B * H, world)
    width = max(hi - lo for lo, hi in ranges)
    _, N, n_local, D = local.shape
    padded = local.new_zeros(1, N, width, D)
    padded[:, :, :n_local] = local
    bufs = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(bufs, padded.contiguous(), group=group)
    parts = [bufs[r][:, :, : hi - lo] for r, (lo, hi) in enumerate(ranges)]
    return from_systems(torch.cat(parts, dim=2), B, H)
