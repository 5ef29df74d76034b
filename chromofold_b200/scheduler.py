"""Batch scheduler: how one decode step is split over the GPUs of a box.

Attention of one (sequence, kv head) depends on nothing else, so the path shards without a collective:

  * sequences over ranks   — longest-processing-time bin packing on context length (deterministic: ties go to the
    lower sequence index, then to the lower rank). The reference's only placement rule is a seeded hash that ignores
    load (src/distributed_runtime.cpp:37-43,73-74); its multi-GPU runtime validates shards and counts, it moves no data
    and launches nothing (src/cuda/multigpu_cuda_runtime.cu:92-193).
  * kv heads over ranks     — contiguous blocks of kv heads; query heads follow their kv head
    (query head h reads kv head h / group), so the per-rank outputs are disjoint column blocks: a gather, not a
    reduction. This is the shape of the reference's cf_multigpu_attention_shard (query_head_begin / query_head_count,
    include/chromofold/multigpu_cuda_runtime.h:53-66).

The only exchange is the optional gather of outputs to rank 0 (torch.distributed: NCCL on GPUs, gloo on CPU ranks).
"""
import numpy as np


def shard_sequences(context_lengths, world_size):
    """-> list (per rank) of sequence indices, each list in ascending order."""
    lengths = np.asarray(context_lengths, np.int64)
    if world_size < 1:
        raise ValueError("world_size must be >= 1")
    order = sorted(range(len(lengths)), key=lambda i: (-int(lengths[i]), i))
    load = [0] * world_size
    shards = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda x: (load[x], x))
        shards[r].append(i)
        load[r] += int(lengths[i])
    return [sorted(s) for s in shards]


def shard_kv_heads(kv_heads, world_size):
    """-> list (per rank) of (kv_head_begin, kv_head_span); ranks beyond the head count get (0, 0)."""
    if world_size < 1 or kv_heads < 1:
        raise ValueError("kv_heads and world_size must be >= 1")
    active = min(world_size, kv_heads)
    base, extra = divmod(kv_heads, active)
    out, begin = [], 0
    for r in range(world_size):
        span = (base + (1 if r < extra else 0)) if r < active else 0
        out.append((begin if span else 0, span))
        begin += span
    return out


def imbalance(context_lengths, shards):
    """max rank load / mean rank load (1.0 = perfect)."""
    lengths = np.asarray(context_lengths, np.int64)
    loads = np.array([int(lengths[s].sum()) if len(s) else 0 for s in shards], np.float64)
    return float(loads.max() / loads.mean()) if loads.mean() > 0 else 1.0


def gather_sequence_outputs(local_out, shards, rank, world_size, dist=None):
    """Sequence sharding: rank r holds rows for shards[r]; rank 0 gets [n_sequences, ...] in original order."""
    import torch
    if world_size == 1:
        return local_out
    n = sum(len(s) for s in shards)
    longest = max(len(s) for s in shards)
    pad = torch.zeros((longest,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    pad[:local_out.shape[0]] = local_out
    bucket = [torch.zeros_like(pad) for _ in range(world_size)] if rank == 0 else None
    dist.gather(pad, bucket, dst=0)
    if rank != 0:
        return None
    full = torch.zeros((n,) + tuple(local_out.shape[1:]), dtype=local_out.dtype, device=local_out.device)
    for r, s in enumerate(shards):
        if s:
            full[torch.as_tensor(s, device=full.device)] = bucket[r][:len(s)]
    return full


def gather_head_outputs(local_out, head_shards, group, rank, world_size, dist=None):
    """KV-head sharding: every rank holds [n, Hq, D] with only its own query-head block filled; rank 0 gets the union."""
    import torch
    if world_size == 1:
        return local_out
    bucket = [torch.zeros_like(local_out) for _ in range(world_size)] if rank == 0 else None
    dist.gather(local_out.contiguous(), bucket, dst=0)
    if rank != 0:
        return None
    full = torch.zeros_like(local_out)
    for r, (begin, span) in enumerate(head_shards):
        if span:
            full[:, begin * group:(begin + span) * group] = bucket[r][:, begin * group:(begin + span) * group]
    return full
