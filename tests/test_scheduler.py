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


def test_c_planners_follow_the_same_rules(native):
    """cf_b200_mg_plan_sequences / _plan_kv_heads (the one-process scheduler's placement, host arithmetic only) give the
    placements of shard_sequences / shard_kv_heads; arguments are checked before anything else."""
    import ctypes as C
    lib = native.lib()
    rng = np.random.default_rng(5)
    for n, world in ((64, 8), (64, 3), (11, 2), (5, 8), (0, 4)):
        ctx = (rng.integers(2048, 32769, n) // 16 * 16).astype(np.uint64)
        out = np.full(n, 99, np.uint32)
        assert lib.cf_b200_mg_plan_sequences(None, ctx.ctypes.data_as(C.c_void_p), n, world, out.ctypes.data_as(C.c_void_p)) == 0
        assert [np.nonzero(out == d)[0].tolist() for d in range(world)] == shard_sequences(ctx, world)
    for heads, world in ((8, 1), (8, 4), (8, 8), (8, 3), (2, 4)):
        begin, span = np.zeros(world, np.uint32), np.zeros(world, np.uint32)
        assert lib.cf_b200_mg_plan_kv_heads(None, heads, world, begin.ctypes.data_as(C.c_void_p), span.ctypes.data_as(C.c_void_p)) == 0
        assert list(zip(begin.tolist(), span.tolist())) == shard_kv_heads(heads, world)
    one = np.ones(1, np.uint64)
    assert lib.cf_b200_mg_plan_sequences(None, one.ctypes.data_as(C.c_void_p), 1, 0, one.ctypes.data_as(C.c_void_p)) == native.CF_ERR_INVALID_ARGUMENT
    assert lib.cf_b200_mg_plan_sequences(None, None, 1, 2, one.ctypes.data_as(C.c_void_p)) == native.CF_ERR_INVALID_ARGUMENT
    assert lib.cf_b200_mg_plan_kv_heads(None, 0, 2, one.ctypes.data_as(C.c_void_p), one.ctypes.data_as(C.c_void_p)) == native.CF_ERR_INVALID_ARGUMENT
    assert lib.cf_b200_mg_create(None) is None
    assert lib.cf_b200_mg_execute_async(None, None, 0, None, None, 0, 1, None) == native.CF_ERR_INVALID_ARGUMENT
    assert C.sizeof(native.MgShard) == C.sizeof(native.SealedAttentionDesc) + 8 and C.sizeof(native.MgConfig) == 40
