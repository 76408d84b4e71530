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

__all__ = ["shard_batch", "allreduce_grads", "init_from_env", "BucketedGradReducer"]


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


class BucketedGradReducer:
    """All-reduce of the flat f32 gradient arena, one bucket per layer, overlapped
    with the rest of the backward.

    The backward walks the layers last to first; as soon as a layer's parameter
    gradients are complete the caller names its bucket with ``bucket_ready(i)``:
    the sum over ranks of that slice is issued on a side stream (NCCL over
    NVLink on GPUs), ordered after the work already queued on the caller's stream,
    and runs under the backward kernels of the layers still to come.
    ``finish()`` joins the side stream (and divides by the world size when
    averaging).  With a CPU tensor (gloo) the same calls run without streams.
    The reference keeps this arena as ``GpuMambaGrads.flat``
    (src/mamba_ssm/gpu/weights.rs:487-560) and has no collective of its own; the
    place it would sit is between backward and optimiser,
    src/mamba_ssm/gpu/trainer.rs:1476-1481."""

    def __init__(self, flat_grads: torch.Tensor, bounds, group=None, average: bool = False):
        if flat_grads.dtype != torch.float32 or not flat_grads.is_contiguous() or flat_grads.dim() != 1:
            raise TypeError("the gradient arena is one contiguous 1-D float32 tensor")
        self.flat, self.group, self.average = flat_grads, group, average
        self.bounds = [(int(lo), int(hi)) for lo, hi in bounds]
        for lo, hi in self.bounds:
            if not (0 <= lo <= hi <= flat_grads.numel()):
                raise ValueError(f"bucket [{lo}, {hi}) outside the arena of {flat_grads.numel()} elements")
        self.active = dist.is_initialized() and dist.get_world_size(group) > 1
        self.cuda = flat_grads.is_cuda
        self.side = torch.cuda.Stream(device=flat_grads.device) if (self.cuda and self.active) else None
        self.works = []
        self.done = set()

    def bucket_ready(self, i: int):
        if i in self.done:
            raise ValueError(f"bucket {i} was already reduced")
        self.done.add(i)
        if not self.active:
            return
        lo, hi = self.bounds[i]
        view = self.flat[lo:hi]
        if self.side is not None:
            self.side.wait_stream(torch.cuda.current_stream(self.flat.device))
            with torch.cuda.stream(self.side):
                self.works.append(dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        else:
            self.works.append(dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def finish(self) -> torch.Tensor:
        for w in self.works:
            w.wait()
        self.works = []
        if self.side is not None:
            torch.cuda.current_stream(self.flat.device).wait_stream(self.side)
        if self.active and self.average:
            n = dist.get_world_size(self.group)
            for i in self.done:
                lo, hi = self.bounds[i]
                self.flat[lo:hi].div_(n)
        return self.flat
