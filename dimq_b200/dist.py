"""Batch sharding across the GPUs of one box: every rank holds a full replica of the packed
weights (a few tens of MB) and its slice of the batch; the only collective is an all-gather of
the logits.  Works with any ``torch.distributed`` backend (NCCL on GPUs, gloo in CPU tests)."""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(total: int, rank: int, world: int) -> tuple[int, int]:
    """``[begin, end)`` of rank ``rank``'s contiguous slice of ``total`` items (sizes differ by at most one)."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"bad rank/world {rank}/{world}")
    base, extra = divmod(int(total), world)
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def gather_logits(local: torch.Tensor, total: int | None = None) -> torch.Tensor:
    """All-gather per-rank logits ``[b_r, C]`` into ``[sum b_r, C]`` in rank order on every rank.

    Equal shards use one ``all_gather_into_tensor``; ragged shards are padded to the largest shard and
    trimmed after the gather.
    """
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    if total is None:
        sizes = [local.shape[0]] * world
    else:
        sizes = [shard_bounds(total, r, world)[1] - shard_bounds(total, r, world)[0] for r in range(world)]
    biggest = max(sizes)
    if all(s == biggest for s in sizes):
        out = local.new_empty((world * biggest, *local.shape[1:]))
        if dist.get_backend() == "gloo":
            chunks = list(out.chunk(world))
            dist.all_gather(chunks, local.contiguous())
        else:
            dist.all_gather_into_tensor(out, local.contiguous())
        return out
    padded = local.new_zeros((biggest, *local.shape[1:]))
    padded[: local.shape[0]] = local
    chunks = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(chunks, padded)
    return torch.cat([c[:s] for c, s in zip(chunks, sizes)], dim=0)
