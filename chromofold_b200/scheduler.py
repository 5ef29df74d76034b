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

MultiGpuScheduler is the other way to run the same split: ONE process drives every GPU of the box through the C ABI
of include/chromofold_b200/sealed_kv_multigpu.h (a stream per GPU, the placement rules above in C++, query rows out and
output rows back as peer copies).
"""
import ctypes as C

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


class MultiGpuScheduler:
    """One process, several GPUs: cf_b200_mg_* over one SealedKvLayer per device (layers[0] lives on the root device,
    where the queries arrive and the outputs are gathered)."""

    def __init__(self, layers, max_rows, query_dtype=None):
        import torch
        from . import _native as N
        self.N, self.torch, self.lib = N, torch, N.lib()
        self.layers = list(layers)
        self.ordinals = [lay.device.index if lay.device.index is not None else 0 for lay in self.layers]
        first = self.layers[0]
        self.query_dtype = query_dtype or torch.float16
        self._ordinals = (C.c_int32 * len(self.ordinals))(*self.ordinals)
        cfg = N.MgConfig()
        cfg.struct_size, cfg.abi_version = C.sizeof(N.MgConfig), N.ABI_VERSION
        cfg.device_count, cfg.device_ordinals = len(self.ordinals), C.cast(self._ordinals, C.c_void_p)
        cfg.max_rows, cfg.query_head_count, cfg.head_dim = max_rows, first.query_heads, first.head_dim
        cfg.query_type = N.F16 if self.query_dtype == torch.float16 else N.F32
        self.handle = self.lib.cf_b200_mg_create(C.byref(cfg))
        if not self.handle:
            raise RuntimeError("cf_b200_mg_create failed (bad config or no such CUDA devices)")
        self.max_rows = max_rows
        shape = (max_rows, first.query_heads, first.head_dim)
        self.q_local = [torch.zeros(shape, dtype=self.query_dtype, device=lay.device) for lay in self.layers]
        self.out_local = [torch.zeros(shape, dtype=torch.float32, device=lay.device) for lay in self.layers]
        self._keep = None

    def close(self):
        if self.handle:
            self.lib.cf_b200_mg_destroy(C.c_void_p(self.handle))
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, what, status):
        if status != self.N.CF_OK:
            raise self.N.CfError(what + ": " + self.lib.cf_b200_mg_last_error(C.c_void_p(self.handle)).decode(), status)

    def set_device_failed(self, ordinal, failed=True):
        self._check("set_device_failed", self.lib.cf_b200_mg_set_device_failed(C.c_void_p(self.handle), C.c_int32(ordinal),
                                                                              C.c_uint32(1 if failed else 0)))

    def plan_sequences(self, context_lengths):
        """-> per device index the list of sequence indices it serves (ascending)."""
        lengths = np.ascontiguousarray(context_lengths, np.uint64)
        out = np.zeros(len(lengths), np.uint32)
        self._check("plan_sequences", self.lib.cf_b200_mg_plan_sequences(
            C.c_void_p(self.handle), lengths.ctypes.data_as(C.c_void_p), C.c_uint32(len(lengths)), C.c_uint32(len(self.layers)),
            out.ctypes.data_as(C.c_void_p)))
        return [np.nonzero(out == d)[0].tolist() for d in range(len(self.layers))]

    def plan_kv_heads(self, kv_heads):
        begin = np.zeros(len(self.layers), np.uint32)
        span = np.zeros(len(self.layers), np.uint32)
        self._check("plan_kv_heads", self.lib.cf_b200_mg_plan_kv_heads(
            C.c_void_p(self.handle), C.c_uint32(kv_heads), C.c_uint32(len(self.layers)), begin.ctypes.data_as(C.c_void_p),
            span.ctypes.data_as(C.c_void_p)))
        return list(zip(begin.tolist(), span.tolist()))

    def counters(self):
        c = self.N.MgCounters()
        self._check("get_counters", self.lib.cf_b200_mg_get_counters(C.c_void_p(self.handle), C.byref(c)))
        return {name: int(getattr(c, name)) for name, _ in c._fields_}

    def _shards(self, per_device, mode, row_count, **desc_kw):
        """per_device[d] = (local slots, root rows or None, kv_head_begin, kv_head_span)."""
        N = self.N
        shards = (N.MgShard * len(self.layers))()
        keep = []
        for d, lay in enumerate(self.layers):
            slots, rows, begin, span = per_device[d]
            n = len(slots)
            if n == 0:
                continue
            out = self.out_local[d] if not (mode == N.MG_BY_KV_HEAD and d == 0 and desc_kw.get("root_out") is not None) else desc_kw["root_out"]
            desc = lay._attention_desc(self.q_local[d], out, n, slots)
            desc.softmax_scale = 1.0 / float(np.sqrt(lay.head_dim))
            desc.kv_head_begin, desc.kv_head_span = begin, span
            desc.min_pages_per_unit = desc_kw.get("min_pages_per_unit", 0)
            keep.append(lay._slots_keepalive)
            shards[d].desc = desc
            if rows is not None:
                arr = np.ascontiguousarray(rows, np.uint32)
                keep.append(arr)
                shards[d].rows = arr.ctypes.data_as(C.c_void_p)
        self._keep = keep
        return shards

    def prepare_by_sequence(self, assignment, local_slots, **kw):
        """The per-device descriptors of a placement, built once: assignment[d] = rows served by device d, local_slots[d] =
        the slots those sequences occupy in layers[d] (same order). Returns a handle for run()."""
        per = [(local_slots[d], assignment[d], 0, 0) for d in range(len(self.layers))]
        rows = sum(len(a) for a in assignment)
        return (self._shards(per, self.N.MG_BY_SEQUENCE, rows, **kw), self._keep, self.N.MG_BY_SEQUENCE, None)

    def prepare_by_kv_head(self, head_shards, slots, root_out, root_queries, **kw):
        """Every device serves every row with its block of kv heads (head_shards[d] = (begin, span)); device-local slot ids
        are `slots` on every device. The root device reads `root_queries` and writes its columns of `root_out` in place."""
        per = [(slots if head_shards[d][1] else [], None, head_shards[d][0], head_shards[d][1]) for d in range(len(self.layers))]
        shards = self._shards(per, self.N.MG_BY_KV_HEAD, len(slots), root_out=root_out, **kw)
        if head_shards[0][1]:
            shards[0].desc.queries = root_queries.data_ptr()
        return (shards, self._keep, self.N.MG_BY_KV_HEAD, (root_queries.data_ptr(), root_out.data_ptr()))

    def run(self, prepared, queries, out):
        """One step of a prepared placement: a single call into the library."""
        shards, _, mode, bound = prepared
        if bound is not None and bound != (queries.data_ptr(), out.data_ptr()):
            raise ValueError("a kv-head placement is bound to the query / output tensors it was prepared with")
        stream = self.torch.cuda.current_stream(self.layers[0].device).cuda_stream
        self._check("mg_execute", self.lib.cf_b200_mg_execute_async(
            C.c_void_p(self.handle), shards, C.c_uint32(len(self.layers)), C.c_void_p(queries.data_ptr()), C.c_void_p(out.data_ptr()),
            C.c_uint32(queries.shape[0]), C.c_uint32(mode), C.c_void_p(stream)))
        return out

    def attention_by_sequence(self, queries, out, assignment, local_slots, **kw):
        return self.run(self.prepare_by_sequence(assignment, local_slots, **kw), queries, out)

    def attention_by_kv_head(self, queries, out, head_shards, slots, **kw):
        return self.run(self.prepare_by_kv_head(head_shards, slots, out, queries, **kw), queries, out)
