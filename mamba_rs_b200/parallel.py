"""Multi-GPU plumbing of the path: batch sharding and the one optional collective.

The selective scan shards by whole sequences (every (sequence, channel)
recurrence is independent), so ranks never exchange data on the scan itself,
forward or backward.  The only collective a trainer needs is the sum of the
flat f32 parameter-gradient arena between backward and the optimiser step
(the reference has no multi-GPU at all; its grad arena is
src/mamba_ssm/gpu/weights.rs:487-560).  One process per GPU, torch.distributed
for the plumbing: NCCL over NVLink on GPUs, gloo on CPU for tests.
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist

__all__ = ["shard_batch", "allreduce_grads", "init_from_env"]


def shard_batch(global_batch: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous range [lo, hi) of whole sequences owned by `rank`.

    The first `global_batch % world` ranks take one extra sequence, so shard
    sizes differ by at most one and every sequence has exactly one owner."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of world {world}")
    if global_batch < 0:
        raise ValueError("negative batch")
    base, extra = divmod(global_batch, world)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo, hi


def init_from_env(backend: str | None = None):
    """Join the process group described by RANK / WORLD_SIZE / MASTER_* (torchrun).
    Returns (rank, world, local_rank); a single process needs no group."""
    import os
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        dist.init_process_group(backend)
    return rank, world, local


def allreduce_grads(flat_grads: torch.Tensor, group=None, bucket_bytes: int = 64 << 20,
                    average: bool = False) -> torch.Tensor:
    """Sum the flat f32 gradient arena over ranks, in place, in buckets.

    Buckets are sized for launch latency and overlap, not for link count: with
    NVSwitch every peer is at full bandwidth.  `average` divides by the world
    size afterwards (the reference's AdamW expects a sum over its own batch, so
    a data-parallel run averages)."""
    if flat_grads.dtype != torch.float32 or not flat_grads.is_contiguous():
        raise TypeError("the gradient arena is one contiguous float32 tensor")
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return flat_grads
    n = flat_grads.numel()
    step = max(1, bucket_bytes // 4)
    works = []
    for lo in range(0, n, step):
        works.append(dist.all_reduce(flat_grads[lo:lo + step], op=dist.ReduceOp.SUM, group=group,
                                     async_op=True))
    for w in works:
        w.wait()
    if average:
        flat_grads.div_(dist.get_world_size(group))
    return flat_grads
