"""Measurements of the benchmark configurations other than the headline one (which `bench.py` at the repository
root times): the coder crossover sweep, the long-context 70B-shaped decode with kv-head sharding, and the
cross-request dedup decode with GPU-sealed suffixes. One JSON line per measured point.

    python -m chromofold_b200.config_bench --config 3
    python -m chromofold_b200.config_bench --config 4            # one GPU: every shard width timed in turn
    python -m torch.distributed.run --nproc-per-node N -m chromofold_b200.config_bench --config 4   # N GPUs, gather timed
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


def config3(a, device):
    """Coder crossover: 32 query / 8 kv heads, batch 32, context 8192, two-sided geometric codes."""
    contexts = np.full(32, 8192)
    for p in (0.05, 0.1, 0.2, 0.4, 0.7):
        for coder in ("rans", "huffman"):
            layer, info = build_sealed_layer(contexts, coder=coder, dist=("geometric", p), seed=40, device=device)
            q = _queries(32, 32, 41, device)
            out = torch.zeros((32, 32, 128), dtype=torch.float32, device=device)
            ms = _time(lambda: layer.attention(q, out=out), a.steps, a.warmup)
            tokens = int(contexts.sum())
            print(json.dumps({"config": 3, "p": p, "coder": coder, "h0_bits_per_code": round(info["h0_bits_k"], 3),
                              "sealed_bytes_per_seq_token": round(info["bytes_per_seq_token"], 1),
                              "kv_memory_reduction_vs_fp16": round(4096 / info["bytes_per_seq_token"], 3),
                              "ms_per_step": round(ms, 4), "seq_tokens_per_s": round(tokens / ms * 1e3),
                              "sealed_gbs": round(info["sealed_bytes"] / ms / 1e6, 1), "device_status": layer.device_status()}))
            del layer, info
            torch.cuda.empty_cache()


def config3_blocks(a, device):
    """Block-size dial of the coder crossover: what 128- and 256-symbol blocks save in bytes (fewer per-block states
    and offsets) and what they cost (they run on the any-geometry kernel; the lane-per-block kernel is built for
    32 blocks of 64 symbols per stream)."""
    contexts = np.full(8, 8192)
    for p in (0.1, 0.4):
        for coder in ("rans", "huffman"):
            for block in (64, 128, 256):
                layer, info = build_sealed_layer(contexts, coder=coder, dist=("geometric", p), seed=40, device=device,
                                                 block_size=block)
                q = _queries(8, 32, 41, device)
                out = torch.zeros((8, 32, 128), dtype=torch.float32, device=device)
                ms = _time(lambda: layer.attention(q, out=out), max(a.steps // 3, 3), 2)
                print(json.dumps({"config": 3, "p": p, "coder": coder, "block_size": block,
                                  "sealed_bytes_per_seq_token": round(info["bytes_per_seq_token"], 1),
                                  "bits_per_code_stored": round(info["bytes_per_seq_token"] * 8 / 2048, 3),
                                  "h0_bits_per_code": round(info["h0_bits_k"], 3),
                                  "kernel": "lanes" if block == 64 else "generic", "ms_per_step": round(ms, 4),
                                  "seq_tokens_per_s": round(int(contexts.sum()) / ms * 1e3),
                                  "device_status": layer.device_status()}))
                del layer, info
                torch.cuda.empty_cache()


def config4(a, device, rank, world):
    """Long context, 70B shape: 64 query / 8 kv heads, 8 sequences x 131072 tokens, kv heads sharded."""
    import torch.distributed as dist
    contexts = np.full(a.batch4, a.ctx4)
    layer, info = build_sealed_layer(contexts, query_heads=64, kv_heads=8, coder=a.coder, seed=50, device=device)
    q = _queries(len(contexts), 64, 51, device)
    out = torch.zeros((len(contexts), 64, 128), dtype=torch.float32, device=device)
    tokens = int(contexts.sum())
    if world == 1:
        for ways in (1, 2, 4, 8):
            begin, span = shard_kv_heads(8, ways)[0]
            ms = _time(lambda: layer.attention(q, out=out, kv_head_begin=begin, kv_head_span=span), a.steps, a.warmup)
            print(json.dumps({"config": 4, "gpus": 1, "shard_ways": ways, "kv_heads_on_this_gpu": span, "ms_per_step": round(ms, 4),
                              "seq_tokens_per_s_if_every_shard_takes_this_long": round(tokens / ms * 1e3),
                              "sealed_gbs_this_gpu": round(info["sealed_bytes"] * span / 8 / ms / 1e6, 1),
                              "sealed_bytes_per_seq_token": round(info["bytes_per_seq_token"], 1),
                              "device_status": layer.device_status()}))
        return
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
        print(json.dumps({"config": 4, "gpus": world, "shard_ways": world, "kv_heads_per_gpu": span,
                          "attention_ms_max_over_ranks": round(float(t[0]), 4), "gather_ms_max_over_ranks": round(float(t[1]), 4),
                          "seq_tokens_per_s": round(tokens / float(t[0]) * 1e3),
                          "seq_tokens_per_s_with_gather": round(tokens / float(t[0] + t[1]) * 1e3),
                          "gathered_equals_single_gpu": bool(torch.equal(gathered, whole)),
                          "device_status": layer.device_status()}))


def config5(a, device):
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
    logical_tokens = n * (prefix + suffix)
    unique_bytes = layer.sealed_bytes()
    flops = 4 * 128 * 32 * logical_tokens
    print(json.dumps({"config": 5, "coder": a.coder, "sequences": n, "shared_prefix_tokens": prefix, "private_suffix_tokens": suffix,
                      "unique_sealed_bytes": unique_bytes, "logical_sealed_bytes": int(one_copy * n + (unique_bytes - one_copy)),
                      "ms_per_step_append_seal_attention": round(ms, 4), "ms_attention_only": round(ms_attn, 4),
                      "ms_attention_without_the_shared_prefix_kernel": round(ms_per_sequence, 4),
                      "seq_tokens_per_s": round(logical_tokens / ms * 1e3),
                      "unique_gbs": round(unique_bytes / ms_attn / 1e6, 1),
                      "logical_gbs": round((one_copy * n + unique_bytes - one_copy) / ms_attn / 1e6, 1),
                      "attention_tflops": round(flops / ms_attn / 1e9, 2), "device_status": layer.device_status()}))


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
    print(json.dumps({"transfer": "2048 pages x 8 kv heads", "sealed_bytes": info["sealed_bytes"],
                      "pack_ms": round(ms_pack, 4), "pack_gbs_read_plus_write": round(2 * gb / ms_pack * 1e3, 1),
                      "unpack_ms": round(ms_unpack, 4), "unpack_gbs_read_plus_write": round(2 * gb / ms_unpack * 1e3, 1),
                      "status": [src.device_status(), dst.device_status()]}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", type=int, default=0, choices=[0, 3, 4, 5])
    ap.add_argument("--transfer", action="store_true", help="time the pack / unpack kernels of transfer images instead")
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--coder", default="rans", choices=["rans", "huffman", "fixed8", "rans4", "huffman4"], help="configurations 4 and 5")
    ap.add_argument("--blocks", action="store_true", help="configuration 3: the block-size dial instead of the p sweep")
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
    if a.transfer:
        transfer(a, device)
    elif a.config == 3 and a.blocks:
        config3_blocks(a, device)
    elif a.config == 3:
        config3(a, device)
    elif a.config == 4:
        config4(a, device, rank, world)
    else:
        config5(a, device)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
