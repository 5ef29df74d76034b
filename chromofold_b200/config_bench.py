"""Measurements of the benchmark configurations other than the headline one (which `bench.py` at the repository
root times): the coder crossover sweep, the long-context 70B-shaped decode with kv-head sharding, and the
cross-request dedup decode with GPU-sealed suffixes. One JSON line per measured point.

    python -m chromofold_b200.config_bench --config 3
    python -m chromofold_b200.config_bench --config 4            # one GPU: every shard width timed in turn
    python -m torch.distributed.run --nproc-per-node N -m chromofold_b200.config_bench --config 4   # N GPUs, gather timed
    python -m chromofold_b200.config_bench --config 4 --one-process N   # N GPUs, one process, the C-ABI batch scheduler
    python -m chromofold_b200.config_bench --config 5

Timing: CUDA events around `--steps` launches after `--warmup` untimed ones; every configuration reads more sealed
bytes per launch than the L2 holds, except the shared prefix of configuration 5, whose re-reads are meant to hit it.
"""
import argparse
import json
import os

import numpy as np
import torch

from . import _native as N
from .scheduler import gather_head_outputs, shard_kv_heads
from .workloads import build_sealed_layer


def _time(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def _queries(n, heads, seed, device):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn((n, heads, 128), generator=g, device=device, dtype=torch.float32).half()


def _checked(result, check, layer, q, out, slots=None, rows=None):
    """Adds the caller's comparison of `out` with its own reference (bench.py passes the CPU oracle; nothing in this
    package computes attention on the CPU) to a result row."""
    if check is not None:
        result["oracle_check"] = check(layer, q, out, slots=slots, rows=rows)
    return result


def config3(a, device, check=None, coders=("rans", "huffman", "rans4", "huffman4"), ps=(0.05, 0.1, 0.2, 0.4, 0.7)):
    """Coder crossover: 32 query / 8 kv heads, batch 32, context 8192, two-sided geometric codes."""
    contexts = np.full(32, 8192)
    results = []
    for p in ps:
        for coder in coders:
            layer, info = build_sealed_layer(contexts, coder=coder, dist=("geometric", p), seed=40, device=device)
            q = _queries(32, 32, 41, device)
            out = torch.zeros((32, 32, 128), dtype=torch.float32, device=device)
            ms = _time(lambda: layer.attention(q, out=out), a.steps, a.warmup)
            tokens = int(contexts.sum())
            results.append(_checked({
                "config": 3, "p": p, "coder": coder, "h0_bits_per_code": round(info["h0_bits_k"], 3),
                "sealed_bytes_per_seq_token": round(info["bytes_per_seq_token"], 1),
                "kv_memory_reduction_vs_fp16": round(4096 / info["bytes_per_seq_token"], 3),
                "ms_per_step": round(ms, 4), "seq_tokens_per_s": round(tokens / ms * 1e3),
                "sealed_gbs": round(info["sealed_bytes"] / ms / 1e6, 1), "device_status": layer.device_status()},
                check, layer, q, out, rows=[0, 13, 31]))
            del layer, info
            torch.cuda.empty_cache()
    return results


def config3_blocks(a, device, check=None):
    """Block-size dial of the coder crossover: what 128- and 256-symbol blocks save in bytes (fewer per-block states
    and offsets) and what they cost in the lane-per-block kernel (16 / 8 blocks per stream are decoded into a
    shared-memory tile first; with 8 blocks half the lanes of a warp have no block to decode). Batch 32 x 8192 as in
    the p sweep."""
    contexts = np.full(32, 8192)
    results = []
    only = getattr(a, "cell", "")   # "coder:block" runs that one cell at p = 0.1 (for profiler captures)
    for p in (0.1, 0.4):
        for coder in ("rans", "huffman", "rans4", "huffman4"):
            for block in (64, 128, 256):
                if only and (only != f"{coder}:{block}" or p != 0.1):
                    continue
                layer, info = build_sealed_layer(contexts, coder=coder, dist=("geometric", p), seed=40, device=device,
                                                 block_size=block)
                q = _queries(32, 32, 41, device)
                out = torch.zeros((32, 32, 128), dtype=torch.float32, device=device)
                ms = _time(lambda: layer.attention(q, out=out), a.steps, a.warmup)
                results.append({"config": 3, "p": p, "coder": coder, "block_size": block,
                                "sealed_bytes_per_seq_token": round(info["bytes_per_seq_token"], 1),
                                "bits_per_code_stored": round(info["bytes_per_seq_token"] * 8 / 2048, 3),
                                "h0_bits_per_code": round(info["h0_bits_k"], 3),
                                "ms_per_step": round(ms, 4),
                                "seq_tokens_per_s": round(int(contexts.sum()) / ms * 1e3),
                                "device_status": layer.device_status()})
                _checked(results[-1], check, layer, q, out, rows=[0, 31])
                del layer, info
                torch.cuda.empty_cache()
    return results


def config4(a, device, rank, world, check=None):
    """Long context, 70B shape: 64 query / 8 kv heads, 8 sequences x 131072 tokens, kv heads sharded. One process:
    every shard width timed in turn on this GPU. Several processes (torchrun): a shard per rank, outputs gathered to
    rank 0 with torch.distributed (the one-process scheduler's version of the same split is config4_one_process)."""
    import torch.distributed as dist
    contexts = np.full(a.batch4, a.ctx4)
    layer, info = build_sealed_layer(contexts, query_heads=64, kv_heads=8, coder=a.coder, seed=50, device=device)
    q = _queries(len(contexts), 64, 51, device)
    out = torch.zeros((len(contexts), 64, 128), dtype=torch.float32, device=device)
    tokens = int(contexts.sum())
    results = []
    if world == 1:
        for ways in (1, 2, 4, 8):
            begin, span = shard_kv_heads(8, ways)[0]
            ms = _time(lambda: layer.attention(q, out=out, kv_head_begin=begin, kv_head_span=span), a.steps, a.warmup)
            row = {"config": 4, "gpus": 1, "coder": a.coder, "shard_ways": ways, "kv_heads_on_this_gpu": span, "ms_per_step": round(ms, 4),
                   "seq_tokens_per_s_if_every_shard_takes_this_long": round(tokens / ms * 1e3),
                   "sealed_gbs_this_gpu": round(info["sealed_bytes"] * span / 8 / ms / 1e6, 1),
                   "sealed_bytes_per_seq_token": round(info["bytes_per_seq_token"], 1),
                   "device_status": layer.device_status()}
            if ways == 1:
                _checked(row, check, layer, q, out)     # all eight sequences, every head
            results.append(row)
        return results
    shards = shard_kv_heads(8, world)
    begin, span = shards[rank]
    step = lambda: layer.attention(q, out=out, kv_head_begin=begin, kv_head_span=span)
    for _ in range(a.warmup):
        step()
        gather_head_outputs(out, shards, 8, rank, world, dist)   # also sets up the communicator's connections
    e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
    dist.barrier()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    for _ in range(a.steps):
        gathered = gather_head_outputs(out, shards, 8, rank, world, dist)
    e2.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / a.steps, e1.elapsed_time(e2) / a.steps], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        whole = layer.attention(q)   # every head on this rank, to check the gathered result
        results.append({"config": 4, "gpus": world, "shard_ways": world, "kv_heads_per_gpu": span,
                        "attention_ms_max_over_ranks": round(float(t[0]), 4), "gather_ms_max_over_ranks": round(float(t[1]), 4),
                        "seq_tokens_per_s": round(tokens / float(t[0]) * 1e3),
                        "seq_tokens_per_s_with_gather": round(tokens / float(t[0] + t[1]) * 1e3),
                        "gathered_equals_single_gpu": bool(torch.equal(gathered, whole)),
                        "device_status": layer.device_status()})
    return results


def _time_on(stream_device, fn, steps, warmup):
    """CUDA events on the current stream of `stream_device` (the scheduler's root stream) around `steps` calls."""
    with torch.cuda.device(stream_device):
        for _ in range(warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for d in range(torch.cuda.device_count()):
            torch.cuda.synchronize(d)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps


def config4_one_process(a, devices, check=None):
    """Configuration 4 through the one-process batch scheduler (cf_b200_mg_*): a replica of the store on every GPU,
    kv heads sharded `len(devices)` ways, query rows out and query-head columns back as peer copies. The timed step
    is everything between two events on the root stream: copies out, attention on every GPU, gather."""
    from .scheduler import MultiGpuScheduler
    contexts = np.full(a.batch4, a.ctx4)
    layers = [build_sealed_layer(contexts, query_heads=64, kv_heads=8, coder=a.coder, seed=50, device=d)[0] for d in devices]
    root = devices[0]
    q = _queries(len(contexts), 64, 51, root)
    out = torch.zeros((len(contexts), 64, 128), dtype=torch.float32, device=root)
    sched = MultiGpuScheduler(layers, max_rows=len(contexts))
    heads = sched.plan_kv_heads(8)
    slots = list(range(len(contexts)))
    prepared = sched.prepare_by_kv_head(heads, slots, out, q)
    ms = _time_on(root, lambda: sched.run(prepared, q, out), a.steps, max(a.warmup, 3))
    with torch.cuda.device(root):
        begin, span = heads[0]
        local = torch.zeros_like(out)
        ms_attn = _time(lambda: layers[0].attention(q, out=local, kv_head_begin=begin, kv_head_span=span), a.steps, 2)
        whole = layers[0].attention(q)
        sched.attention_by_kv_head(q, out, heads, slots)
        torch.cuda.synchronize()
    tokens = int(contexts.sum())
    row = {"config": 4, "gpus": len(devices), "coder": a.coder, "how": "one process, cf_b200_mg_execute_async, kv heads sharded",
           "kv_head_blocks": heads, "step_ms_copies_attention_gather": round(ms, 4),
           "attention_ms_root_shard_alone": round(ms_attn, 4), "copies_and_gather_ms": round(max(ms - ms_attn, 0.0), 4),
           "seq_tokens_per_s": round(tokens / ms * 1e3), "max_abs_diff_vs_one_gpu_all_heads": float((out - whole).abs().max().item()),
           "counters": sched.counters(), "device_status": [lay.device_status() for lay in layers]}
    _checked(row, check, layers[0], q, out)
    sched.close()
    return [row]


def strong_scaling_one_process(a, devices, contexts, coder, check=None, single_gpu_ms=None):
    """One batch (the headline workload's sequences) placed over the GPUs by the C planner (longest context first),
    every GPU holding only its own sequences' pages, timed through cf_b200_mg_execute_async."""
    from .scheduler import MultiGpuScheduler, imbalance
    from . import _native as N
    contexts = np.asarray(contexts, np.int64)
    import ctypes as C
    out_dev = np.zeros(len(contexts), np.uint32)
    lengths = contexts.astype(np.uint64)
    N.check("plan", N.lib().cf_b200_mg_plan_sequences(None, lengths.ctypes.data_as(C.c_void_p), C.c_uint32(len(contexts)),
                                                       C.c_uint32(len(devices)), out_dev.ctypes.data_as(C.c_void_p)))
    assignment = [np.nonzero(out_dev == d)[0].tolist() for d in range(len(devices))]
    layers = [build_sealed_layer(contexts[assignment[d]], coder=coder, seed=4 + 17 * d, device=dev)[0] for d, dev in enumerate(devices)]
    root = devices[0]
    q = _queries(len(contexts), 32, 6, root)
    out = torch.zeros((len(contexts), 32, 128), dtype=torch.float32, device=root)
    sched = MultiGpuScheduler(layers, max_rows=len(contexts))
    local_slots = [list(range(len(assignment[d]))) for d in range(len(devices))]
    prepared = sched.prepare_by_sequence(assignment, local_slots)
    ms = _time_on(root, lambda: sched.run(prepared, q, out), a.steps, max(a.warmup, 3))
    with torch.cuda.device(root):
        sched.attention_by_sequence(q, out, assignment, local_slots)
        torch.cuda.synchronize()
    tokens = int(contexts.sum())
    row = {"scaling": "strong", "gpus": len(devices), "coder": coder, "how": "one process, cf_b200_mg_execute_async, sequences placed longest first",
           "sequences": len(contexts), "seq_tokens": tokens, "load_imbalance_max_over_mean": round(imbalance(contexts, assignment), 4),
           "step_ms_copies_attention_gather": round(ms, 4), "seq_tokens_per_s": round(tokens / ms * 1e3),
           "counters": sched.counters(), "device_status": [lay.device_status() for lay in layers]}
    if single_gpu_ms:
        row["single_gpu_step_ms_same_batch"] = round(single_gpu_ms, 4)
        row["speedup_vs_one_gpu"] = round(single_gpu_ms / ms, 3)
        row["efficiency"] = round(single_gpu_ms / ms / len(devices), 3)
    if check is not None:   # the root device's own sequences against the caller's reference
        with torch.cuda.device(root):
            rows = assignment[0][:4]
            row["oracle_check"] = check(layers[0], q[rows].contiguous(), out[rows].contiguous(), slots=local_slots[0][:4])
    sched.close()
    return [row]


def config5(a, device, check=None):
    """Dedup: 256 sequences share one sealed 16384-token prefix (one copy) and own a 512-token sealed suffix each; a
    step appends one token to every sequence, seals the pages that filled up, and runs the decode attention."""
    n, prefix, suffix = a.seqs5, a.prefix5, a.suffix5
    contexts = np.array([prefix] + [0] * (n - 1))
    layer, info = build_sealed_layer(contexts, coder=a.coder, seed=60, device=device,
                                     extra_pages_per_sequence=suffix // 16 + 8, reserve_pages=n * (suffix // 16 + 8))
    one_copy = layer.sealed_bytes()
    for s in range(1, n):
        layer.copy_sequence(0, s)
    assert layer.sealed_bytes() == one_copy
    g = torch.Generator(device=device)
    g.manual_seed(61)
    slots = list(range(n))
    rows = lambda: (torch.randn((n, 8, 128), generator=g, device=device) * 0.7).half()
    for _ in range(suffix):   # private suffixes, sealed on the GPU as they fill
        layer.append(slots, rows(), rows())
        layer.seal_full_pages()
    q = _queries(n, 32, 62, device)
    out = torch.zeros((n, 32, 128), dtype=torch.float32, device=device)
    k_new, v_new = rows(), rows()
    budget = layer.max_pages_per_sequence * 16 - prefix - suffix - 16
    assert a.steps + a.warmup < budget, "not enough page-table room for the timed appends"

    shared = prefix // 16

    def step():
        layer.append(slots, k_new, v_new)
        layer.seal_full_pages()
        layer.attention(q, out=out, shared_prefix_pages=shared)

    ms = _time(step, a.steps, a.warmup)
    ms_attn = _time(lambda: layer.attention(q, out=out, shared_prefix_pages=shared), a.steps, a.warmup)
    ms_per_sequence = _time(lambda: layer.attention(q, out=out), max(a.steps // 4, 2), 2)   # every page decoded per sequence
    layer.attention(q, out=out, shared_prefix_pages=shared)
    torch.cuda.synchronize()
    logical_tokens = n * (prefix + suffix)
    unique_bytes = layer.sealed_bytes()
    flops = 4 * 128 * 32 * logical_tokens
    row = {"config": 5, "coder": a.coder, "sequences": n, "shared_prefix_tokens": prefix, "private_suffix_tokens": suffix,
           "unique_sealed_bytes": unique_bytes, "logical_sealed_bytes": int(one_copy * n + (unique_bytes - one_copy)),
           "ms_per_step_append_seal_attention": round(ms, 4), "ms_attention_only": round(ms_attn, 4),
           "ms_attention_without_the_shared_prefix_kernel": round(ms_per_sequence, 4),
           "seq_tokens_per_s": round(logical_tokens / ms * 1e3),
           "unique_gbs": round(unique_bytes / ms_attn / 1e6, 1),
           "logical_gbs": round((one_copy * n + unique_bytes - one_copy) / ms_attn / 1e6, 1),
           "attention_tflops": round(flops / ms_attn / 1e9, 2), "device_status": layer.device_status()}
    picked = sorted({0, n - 1} | set(range(0, n, max(n // 14, 1))))[:16] if n > 16 else list(range(n))
    picked = sorted(set(picked) | {n - 1})
    _checked(row, check, layer, q, out, rows=picked)   # slot 0, the last slot and an even spread between them
    return [row]


def transfer(a, device):
    """Pack / verify-unpack rate of transfer images: one 32768-token sequence (2048 pages x 8 kv heads) moved from one
    store into another on the same GPU, device buffers only."""
    import ctypes as C
    contexts = np.array([32768])
    src, info = build_sealed_layer(contexts, coder="rans", seed=70, device=device)
    dst, _ = build_sealed_layer(np.array([0]), coder="rans", seed=71, device=device, extra_pages_per_sequence=2100,
                                reserve_pages=2100 * (a.steps + a.warmup + 2))
    n = 2048
    ids = torch.as_tensor(src.h_page_table[0, :n].astype(np.int32), device=device)
    manifest = torch.zeros(n * 8 * 16, dtype=torch.uint8, device=device)
    payload = torch.zeros(info["sealed_bytes"] + 4096, dtype=torch.uint8, device=device)
    cursor = torch.zeros(1, dtype=torch.int64, device=device)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())

    def pack():
        cursor.zero_()
        N.check("pack", src.lib.cf_b200_pages_pack_async(p(src.arena), p(src.page_dir), C.c_uint32(8), p(ids), C.c_uint32(n),
                                                         p(manifest), p(payload), C.c_uint64(payload.numel()), p(cursor),
                                                         p(src.status), stream))
    next_id = [1]

    def unpack():
        d_ids = torch.arange(next_id[0], next_id[0] + n, dtype=torch.int32, device=device)
        next_id[0] += n
        N.check("unpack", dst.lib.cf_b200_pages_unpack_async(p(manifest), p(payload), C.c_uint64(info["sealed_bytes"]),
                                                             C.c_uint32(8), p(d_ids), C.c_uint32(n), p(dst.arena),
                                                             C.c_uint64(dst.arena_units), p(dst.cursor), p(dst.page_dir),
                                                             p(dst.status), stream))
    ms_pack = _time(pack, a.steps, a.warmup)
    ms_unpack = _time(unpack, a.steps, a.warmup)
    gb = info["sealed_bytes"] / 1e9
    return [{"transfer": "2048 pages x 8 kv heads", "sealed_bytes": info["sealed_bytes"],
             "pack_ms": round(ms_pack, 4), "pack_gbs_read_plus_write": round(2 * gb / ms_pack * 1e3, 1),
             "unpack_ms": round(ms_unpack, 4), "unpack_gbs_read_plus_write": round(2 * gb / ms_unpack * 1e3, 1),
             "status": [src.device_status(), dst.device_status()]}]


def head_dim_dial(a, device, check=None):
    """16 x 96, 16 x 64 (the shape of the reference's own live runs) and 16 x 32 pages through the lane-per-block
    kernel's staging path and, for comparison, through the any-geometry kernel: batch 32 x 8192, Laplace(b=12) codes."""
    contexts = np.full(32, 8192)
    results = []
    only = getattr(a, "cell", "")   # "coder:head_dim:block" runs that one cell (for profiler captures)
    for coder in ("rans4", "huffman4", "rans", "huffman", "fixed8"):
        for dim, block in ((96, 64), (64, 64), (64, 128), (32, 64)):
            if only and only != f"{coder}:{dim}:{block}":
                continue
            layer, info = build_sealed_layer(contexts, coder=coder, seed=45, device=device, head_dim=dim, block_size=block)
            g = torch.Generator(device=device)
            g.manual_seed(46)
            q = torch.randn((32, 32, dim), generator=g, device=device, dtype=torch.float32).half()
            out = torch.zeros((32, 32, dim), dtype=torch.float32, device=device)
            ms = _time(lambda: layer.attention(q, out=out), a.steps, a.warmup)
            ms_generic = _time(lambda: layer.attention(q, out=out, kernel=N.KERNEL_GENERIC), 3, 1)
            results.append(_checked({"head_dim": dim, "coder": coder, "block_size": block,
                                     "sealed_bytes_per_seq_token": round(info["bytes_per_seq_token"], 1),
                                     "ms_per_step": round(ms, 4), "seq_tokens_per_s": round(int(contexts.sum()) / ms * 1e3),
                                     "sealed_gbs": round(info["sealed_bytes"] / ms / 1e6, 1),
                                     "ms_per_step_any_geometry_kernel": round(ms_generic, 4),
                                     "device_status": layer.device_status()}, check, layer, q, out, rows=[0, 31]))
            del layer, info
            torch.cuda.empty_cache()
    return results


def seal_rate(a, device, coders=("rans4", "huffman4", "rans", "huffman", "fixed8")):
    """cf_b200_seal_pages_async alone: 2048 full pages x 8 kv heads per launch (quantise, code both streams, take arena
    room, publish), Laplace(b=12) tiles resident in HBM, CUDA events around every launch; the same tiles are sealed
    again and again into fresh page ids. Algorithmic bytes per page-head: 8192 in (binary16 K and V tiles) + the record out."""
    import ctypes as C
    from .workloads import laplace_codes, tiles_from_codes
    rows, n, hkv = [], 2048, 8
    launches = a.steps + a.warmup + 1
    for coder in coders:
        layer, info = build_sealed_layer(np.array([16 * n]), coder=coder, seed=90, device=device, reserve_pages=n * launches)
        gen = torch.Generator(device=device)
        gen.manual_seed(91)
        k = tiles_from_codes(laplace_codes((n, hkv, 16, 128), 12.0, gen, device), 0.005, 0.02, gen)
        v = tiles_from_codes(laplace_codes((n, hkv, 16, 128), 12.0, gen, device), 0.005, 0.02, gen)
        tiles = torch.arange(n, dtype=torch.int32, device=device)
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

        def seal():
            ids = torch.arange(layer.next_page_id, layer.next_page_id + n, dtype=torch.int32, device=device)
            layer.next_page_id += n
            d = layer._seal_desc(tiles, ids, None)
            d.tail_k, d.tail_v = k.data_ptr(), v.data_ptr()
            N.check("seal_pages", layer.lib.cf_b200_seal_pages_async(C.byref(d), stream))
        before = int(layer.cursor.item())
        seal()
        torch.cuda.synchronize()
        record_bytes = (int(layer.cursor.item()) - before) * 16
        ms = _time(seal, a.steps, a.warmup)
        rows.append({"seal": f"{n} pages x {hkv} kv heads per launch", "coder": coder, "ms_per_launch": round(ms, 4),
                     "page_heads_per_s": round(n * hkv / ms * 1e3), "tokens_per_s_all_kv_heads": round(n * 16 / ms * 1e3),
                     "gbs_in_plus_out": round((n * hkv * 8192 + record_bytes) / ms / 1e6, 1),
                     "record_bytes_per_launch": record_bytes, "device_status": layer.device_status()})
    return rows


def delta_fetch(a, device):
    """cf_delta_fetch_async (token-id look-up in a reference/delta cluster, src/cuda/delta_apply.cu:30-44; the reference
    quotes 6.1 G tokens/s on a 2080 Ti): 256 members of 1 Mi tokens each over one base, 2 % of the positions overridden,
    every token of every member fetched in order. Algorithmic bytes per token: leaf + position in, token out, one base
    read = 16 B; the binary search over the member's overrides (log2(21 k) = 15 probes) is what the kernel actually pays."""
    import ctypes as C
    lib = N.lib()
    lib.cf_delta_fetch_async.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 7 + [C.c_size_t, C.c_void_p]
    g = torch.Generator(device=device)
    g.manual_seed(80)
    nbase, leaves, per_leaf = 1 << 20, 256, (1 << 20) // 50
    base = torch.randint(0, 128000, (nbase,), generator=g, device=device, dtype=torch.int32)
    dpos = torch.stack([torch.sort(torch.randperm(nbase, generator=g, device=device)[:per_leaf])[0] for _ in range(leaves)]).to(torch.int32).reshape(-1)
    dval = torch.randint(0, 128000, (leaves * per_leaf,), generator=g, device=device, dtype=torch.int32)
    dstart = (torch.arange(leaves, device=device, dtype=torch.int32) * per_leaf)
    dlen = torch.full((leaves,), per_leaf, device=device, dtype=torch.int32)
    count = 1 << 26                                    # 64 members' worth per launch
    leaf = (torch.arange(count, device=device, dtype=torch.int64) // nbase).to(torch.int32)
    pos = (torch.arange(count, device=device, dtype=torch.int64) % nbase).to(torch.int32)
    out = torch.zeros(count, device=device, dtype=torch.int32)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def fetch():
        N.check("delta_fetch", lib.cf_delta_fetch_async(base.data_ptr(), nbase, dpos.data_ptr(), dval.data_ptr(), dstart.data_ptr(),
                                                        dlen.data_ptr(), leaf.data_ptr(), pos.data_ptr(), out.data_ptr(), count, stream))
    ms = _time(fetch, a.steps, a.warmup)
    want0 = int(base[5].item())
    hit = (dpos[:per_leaf] == 5).nonzero()
    if hit.numel():
        want0 = int(dval[int(hit[0].item())].item())
    return [{"delta_fetch": "256 members x 1 Mi tokens, 2 % overridden, sequential fetch of 64 Mi tokens per launch",
             "ms": round(ms, 4), "tokens_per_s": round(count / ms * 1e3), "algorithmic_gbs_at_16_bytes_per_token": round(16 * count / ms / 1e6, 1),
             "spot_check": int(out[5].item()) == want0}]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=0, choices=[0, 3, 4, 5])
    ap.add_argument("--transfer", action="store_true", help="time the pack / unpack kernels of transfer images instead")
    ap.add_argument("--delta", action="store_true", help="time cf_delta_fetch_async instead")
    ap.add_argument("--seal", action="store_true", help="time cf_b200_seal_pages_async alone, every coder")
    ap.add_argument("--head-dims", action="store_true", help="time attention over 16 x 96, 16 x 64 and 16 x 32 pages")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--coder", default="rans", choices=["rans", "huffman", "fixed8", "rans4", "huffman4"], help="configurations 4 and 5")
    ap.add_argument("--blocks", action="store_true", help="configuration 3: the block-size dial instead of the p sweep")
    ap.add_argument("--cell", default="", help="with --blocks: coder:block, with --head-dims: coder:head_dim:block — run that one cell")
    ap.add_argument("--one-process", type=int, default=0, metavar="N",
                    help="configuration 4 on N GPUs driven by this one process through the C-ABI batch scheduler")
    ap.add_argument("--batch4", type=int, default=8)
    ap.add_argument("--ctx4", type=int, default=131072)
    ap.add_argument("--seqs5", type=int, default=256)
    ap.add_argument("--prefix5", type=int, default=16384)
    ap.add_argument("--suffix5", type=int, default=512)
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("config_bench needs a CUDA device: the library has no CPU path")
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = f"cuda:{local}"
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(device))
    if a.delta:
        rows = delta_fetch(a, device)
    elif a.seal:
        rows = seal_rate(a, device)
    elif a.head_dims:
        rows = head_dim_dial(a, device)
    elif a.transfer:
        rows = transfer(a, device)
    elif a.config == 3 and a.blocks:
        rows = config3_blocks(a, device)
    elif a.config == 3:
        rows = config3(a, device)
    elif a.config == 4 and a.one_process:
        rows = config4_one_process(a, [f"cuda:{d}" for d in range(a.one_process)])
    elif a.config == 4:
        rows = config4(a, device, rank, world)
    else:
        rows = config5(a, device)
    for row in rows:
        print(json.dumps(row))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
