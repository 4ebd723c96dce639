"""Batch sharding across GPUs: the denoising step shards by image (and CFG branch) with replicated
weights and no collective on the data path; only timings and final latents cross ranks, on the host side.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(total: int, world: int, rank: int) -> tuple[int, int]:
    """[start, stop) of the images rank `rank` owns when `total` images are split as evenly as possible."""
    if world <= 0 or not 0 <= rank < world or total < 0:
        raise ValueError("bad shard request")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def max_over_ranks(value: float, device=None) -> float:
    """Largest `value` over all ranks (identity without an initialised process group)."""
    if not (dist.is_available() and dist.is_initialized()):
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


def gather_latents(local: torch.Tensor, total: int) -> torch.Tensor | None:
    """Collects the per-rank latents [b_r, ...] on rank 0 in image order (host side, end of generation)."""
    if not (dist.is_available() and dist.is_initialized()):
        return local
    world, rank = dist.get_world_size(), dist.get_rank()
    parts = [None] * world
    dist.all_gather_object(parts, local.cpu())
    if rank != 0:
        return None
    out = torch.cat(parts, dim=0)
    assert out.shape[0] == total
    return out
