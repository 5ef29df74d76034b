"""Host logic of the batch scheduler, including the world_size-2 exchange over gloo on CPU ranks."""
import os
import socket

import numpy as np
import pytest

from chromofold_b200.scheduler import gather_head_outputs, gather_sequence_outputs, imbalance, shard_kv_heads, shard_sequences


def test_sequence_sharding_is_a_balanced_partition():
    rng = np.random.default_rng(3)
    ctx = rng.integers(2048, 32769, 64) // 16 * 16
    for world in (1, 2, 4, 8):
        shards = shard_sequences(ctx, world)
        flat = sorted(i for s in shards for i in s)
        assert flat == list(range(64))                       # every sequence exactly once
        assert imbalance(ctx, shards) < 1.03                 # LPT on 64 items is near perfect
        assert shards == shard_sequences(ctx, world)         # deterministic
    assert shard_sequences([], 4) == [[], [], [], []]
    assert shard_sequences([5, 5, 5], 2) == [[0, 2], [1]]    # ties: lower index first, then lower rank
    with pytest.raises(ValueError):
        shard_sequences([1], 0)


def test_kv_head_sharding_covers_heads_in_contiguous_blocks():
    assert shard_kv_heads(8, 1) == [(0, 8)]
    assert shard_kv_heads(8, 4) == [(0, 2), (2, 2), (4, 2), (6, 2)]
    assert shard_kv_heads(8, 8) == [(i, 1) for i in range(8)]
    assert shard_kv_heads(8, 3) == [(0, 3), (3, 3), (6, 2)]
    assert shard_kv_heads(2, 4) == [(0, 1), (1, 1), (0, 0), (0, 0)]   # more ranks than heads: the rest idle


def _worker(rank, world, port, ret):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ctx = (np.arange(11) * 37 % 23 + 1) * 16
    shards = shard_sequences(ctx, world)
    # each rank "computes" rows that encode (sequence index, head): what the attention launch would return
    local = torch.tensor([[float(100 * s + h) for h in range(8)] for s in shards[rank]]).reshape(-1, 8, 1)
    full = gather_sequence_outputs(local, shards, rank, world, dist)
    heads = shard_kv_heads(4, world)
    mine = torch.zeros(3, 8, 1)
    b, n = heads[rank]
    mine[:, b * 2:(b + n) * 2] = torch.arange(8.0).reshape(1, 8, 1)[:, b * 2:(b + n) * 2] + 10 * rank
    merged = gather_head_outputs(mine, heads, 2, rank, world, dist)
    if rank == 0:
        ret["seq"] = full.squeeze(-1).numpy().tolist()
        ret["head"] = merged.squeeze(-1).numpy().tolist()
    dist.barrier()
    dist.destroy_process_group()


def test_output_gather_world_size_2_gloo():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
    assert ret["seq"] == [[float(100 * s + h) for h in range(8)] for s in range(11)]
    assert ret["head"] == [[0.0, 1.0, 2.0, 3.0, 14.0, 15.0, 16.0, 17.0]] * 3
