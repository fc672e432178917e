"""Batch partition for multi-GPU runs.  The DDF op is independent per sample in
the forward and in all three gradients (the filters are per-sample), so N GPUs
each take a contiguous slice of the batch and no collective is needed on the
data path.  The only communication is an all-gather of results for checking."""
from __future__ import annotations

import torch
import torch.distributed as dist


def batch_slice(batch: int, rank: int, world: int) -> tuple[int, int]:
    """Samples [lo, hi) owned by `rank`: lo = rank*batch//world (balanced to +-1)."""
    if not (0 <= rank < world):
        raise ValueError(f"rank {rank} outside world of {world}")
    return rank * batch // world, (rank + 1) * batch // world


def gather_batch(local: torch.Tensor, batch: int) -> torch.Tensor:
    """All-gathers per-rank slices (dim 0) back into batch order on every rank.
    Slices may differ in length by one; they are padded for the collective."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    sizes = [batch_slice(batch, r, world) for r in range(world)]
    longest = max(hi - lo for lo, hi in sizes)
    pad = local.new_zeros((longest,) + tuple(local.shape[1:]))
    pad[: local.shape[0]] = local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad)
    return torch.cat([p[: hi - lo] for p, (lo, hi) in zip(parts, sizes)], dim=0)
