"""World-size-2 (and 3) tests of the multi-GPU host logic on CPU with gloo:
sharding covers every sequence once, and parameter gradients computed per shard
and all-reduced equal the single-process gradients over the whole batch."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from helpers import quantised_inputs, rel_err
from mamba_rs_b200.parallel import BucketedGradReducer, allreduce_grads, shard_batch


def test_shard_batch_partitions_every_sequence_once():
    for B in (0, 1, 7, 8, 16, 63, 64):
        for world in (1, 2, 3, 4, 8):
            owned = []
            sizes = []
            for r in range(world):
                lo, hi = shard_batch(B, r, world)
                owned += list(range(lo, hi))
                sizes.append(hi - lo)
            assert owned == list(range(B))
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_batch(8, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, B, T, D, N, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q = quantised_inputs(B, T, D, N, 0, "f32", seed=3)
        dg = np.random.default_rng(4).standard_normal((B, T, D)).astype(np.float32)
        lo, hi = shard_batch(B, rank, world)
        sl = slice(lo, hi)
        if hi > lo:
            g = oracle.m1_fused_bwd(q["x"][sl], q["delta_raw"][sl], q["Bm"][sl], q["Cm"][sl], q["z"][sl],
                                    q["a_neg"], q["Dp"], dg[sl])
            flat = np.concatenate([g["dA_log"].ravel(), g["dD"].ravel()])
            per_seq = g["dB"]
        else:  # a rank may own nothing when B < world: it still joins the collective
            flat = np.zeros(D * N + D, np.float32)
            per_seq = np.zeros((0, T, N), np.float32)
        arena = torch.from_numpy(flat.copy())
        allreduce_grads(arena, bucket_bytes=256)  # several buckets
        np.save(os.path.join(out_dir, f"arena{rank}.npy"), arena.numpy())
        # the per-layer reducer: buckets named last to first, as a backward pass finishes them
        arena2 = torch.from_numpy(flat.copy())
        cut = D * N
        red = BucketedGradReducer(arena2, [(0, cut), (cut, cut + D)])
        red.bucket_ready(1)
        red.bucket_ready(0)
        red.finish()
        np.save(os.path.join(out_dir, f"arena_b{rank}.npy"), arena2.numpy())
        np.save(os.path.join(out_dir, f"dB{rank}.npy"), per_seq)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,B", [(2, 4), (2, 3), (3, 2)])
def test_sharded_gradients_allreduce_to_the_whole_batch(tmp_path, world, B):
    T, D, N = 24, 8, 16
    port = _free_port()
    mp.spawn(_worker, args=(world, port, B, T, D, N, str(tmp_path)), nprocs=world, join=True)
    q = quantised_inputs(B, T, D, N, 0, "f32", seed=3)
    dg = np.random.default_rng(4).standard_normal((B, T, D)).astype(np.float32)
    whole = oracle.m1_fused_bwd(q["x"], q["delta_raw"], q["Bm"], q["Cm"], q["z"], q["a_neg"], q["Dp"], dg)
    ref = np.concatenate([whole["dA_log"].ravel(), whole["dD"].ravel()])
    arenas = [np.load(tmp_path / f"arena{r}.npy") for r in range(world)]
    for a in arenas[1:]:
        np.testing.assert_array_equal(a, arenas[0])  # every rank holds the same sum
    assert rel_err(arenas[0], ref) <= 1e-5  # only the summation order over samples differs
    for r in range(world):  # the bucketed reducer gives the same sums as the flat all-reduce
        np.testing.assert_array_equal(np.load(tmp_path / f"arena_b{r}.npy"), arenas[0])
    # per-sequence outputs need no exchange: the shards concatenate to the whole
    dB = np.concatenate([np.load(tmp_path / f"dB{r}.npy") for r in range(world)], axis=0)
    np.testing.assert_array_equal(dB, whole["dB"])
