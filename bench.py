#!/usr/bin/env python
"""Benchmark of the sealed-KV decode-attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--coder rans|huffman|fixed8]

One "step" is one decode-step attention of the whole batch over one layer: plan + attention + combine launched
through the C ABI. The workload at N = 1 is the Llama-3-8B-shaped GQA decode step the metric is quoted on:
32 query heads, 8 kv heads, head_dim 128, 64 sequences with context lengths uniform in [2048, 32768] (whole
16-token pages), int8 codes from a discretised Laplace(b=12), one binary16 scale per (page, kv head, K|V), pages
sealed with rANS by the GPU sealer. At N > 1 every rank holds its own batch of 64 sequences (weak scaling, no
collective on the data path). One JSON line is printed by rank 0.

  value      seq-tokens/s of the whole job, inputs resident in HBM, CUDA events around K steps, max over ranks
  e2e        the same with the step's host inputs copied in (queries, pinned) and its result copied out
  roofline   the page-reading kernel alone: sealed bytes it must read / its mean duration (events between stages)
  cpu_baseline  the CPU oracle (restated reference decoders + double online softmax) on all host cores, on a sample
  dense      the same attention over uncompressed binary16 pages on the same GPU (memory / speed comparison)

--impl reference times the reference's own CPU code (reference::paged_attention over its int4 sealed pages, built
into oracle/_ref) on the host cores, on a bounded sample of the same shapes.
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# DRAM bytes (read + write) of one attention launch over its algorithmic bytes, from the ncu captures of the batch-16
# case of the same workload (profiles/lanes_attention_kernel_batch16.md); traffic grows in proportion to the pages read.
DRAM_TRAFFIC_RATIO = {"rans": 410.8 / 387.9, "huffman": 388.5 / 365.6, "fixed8": 481.9 / 457.0,
                      "rans4": 416.4 / 393.3, "huffman4": 393.6 / 370.7}
METRIC = "sealed-KV decode attn seq-tokens/s"
UNIT = "seq-tokens/s"
HQ, HKV, D, T, BLOCK = 32, 8, 128, 16, 64
BATCH, CTX_LO, CTX_HI = 64, 2048, 32768


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--coder", default="rans4", choices=["rans", "huffman", "fixed8", "rans4", "huffman4"],
                    help="page coder; rans4 / huffman4 are the nibble-split variants (raw low nibbles, pairs of high nibbles coded)")
    ap.add_argument("--laplace-b", type=float, default=12.0)
    ap.add_argument("--batch", type=int, default=BATCH)
    ap.add_argument("--ctx-lo", type=int, default=CTX_LO)
    ap.add_argument("--ctx-hi", type=int, default=CTX_HI)
    ap.add_argument("--kernel", default="auto", choices=["auto", "generic", "lanes"])
    ap.add_argument("--min-pages-per-unit", type=int, default=0)
    ap.add_argument("--f32-queries", action="store_true",
                    help="pass the queries as fp32, as the reference's own ABIs do (split-query kernel); default fp16")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-dense", action="store_true", help="skip the uncompressed comparison kernel")
    ap.add_argument("--no-others", action="store_true", help="skip the legs that time the same workload sealed with the other coders")
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the other configurations (3, 4, 5 at full size with their oracle checks; on several GPUs the "
                         "strong-scaling and kv-head-sharding legs of the one-process scheduler)")
    ap.add_argument("--cpu-seconds", type=float, default=15.0)
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every rank has its own batch; strong: one batch sharded over the ranks by the scheduler")
    return ap.parse_args()


def workload_name(a):
    return (f"llama3-8b-gqa-decode: {HQ}q/{HKV}kv heads, head_dim {D}, batch {a.batch}, ctx U[{a.ctx_lo},{a.ctx_hi}], "
            f"{T}-token pages, int8 Laplace(b={a.laplace_b:g}) codes, fp16 scale per page-head, {a.coder}-sealed, 1 layer"
            + (", fp32 queries" if getattr(a, "f32_queries", False) else ""))


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 200 ms while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [x.strip() for x in line.split(",")]))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        inside = [r for (t, r) in self.rows if t0 <= t <= t1 + 0.25] or [r for (_, r) in self.rows]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no sample"]}
        sm = sorted(float(r[0]) for r in inside)
        reasons = set()
        for r in inside:
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": float(inside[0][1]), "samples": len(inside),
                "power_w_max": max(float(r[2]) for r in inside), "reasons": sorted(reasons)}


def run_reference(a, rank):
    """The reference's CPU implementation of the path (reference::paged_attention over pages sealed by its own
    seal_int4_page), all host threads, on a bounded sample of the workload's sequences."""
    if rank != 0:
        return
    from oracle import binding as ob
    from chromofold_b200.workloads import uniform_contexts
    ref = ob.ref_cpu()
    line = {"impl": "reference", "metric": METRIC, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": workload_name(a)}}
    if ref is None:
        line = {"impl": "reference", "unavailable": "oracle/_ref/libcfref_cpu.so was not built (reference tree absent at build time)"}
        print(json.dumps(line))
        return
    ref.ref_cache_create.restype = C.c_void_p
    ref.ref_cache_bytes.restype = C.c_uint64
    cores = os.cpu_count() or 1
    contexts = uniform_contexts(a.batch, a.ctx_lo, a.ctx_hi, T, 3)
    # bounded sample: the first sequences of the batch, at most one per host thread, at most ~400k tokens
    sample, tokens = [], 0
    for c in contexts:
        if len(sample) >= cores or tokens + c > 400_000:
            break
        sample.append(int(c))
        tokens += int(c)
    rng = np.random.default_rng(7)
    caches, queries = [], []
    for c in sample:
        k = rng.standard_normal((HKV, c, D), dtype=np.float32)
        v = rng.standard_normal((HKV, c, D), dtype=np.float32)
        h = ref.ref_cache_create(k.ctypes.data_as(C.c_void_p), v.ctypes.data_as(C.c_void_p), C.c_uint32(c),
                                 C.c_uint32(T), C.c_uint32(HKV), C.c_uint32(D))
        assert h, "reference sealing failed"
        caches.append(C.c_void_p(h))
        queries.append(rng.standard_normal((HQ, D), dtype=np.float32))
    outs = [np.zeros((HQ, D), np.float32) for _ in sample]
    scale = C.c_float(1.0 / np.sqrt(D))

    def one(i):
        rc = ref.ref_cache_attention(caches[i], queries[i].ctypes.data_as(C.c_void_p), C.c_uint32(HQ), C.c_uint32(0),
                                     scale, outs[i].ctypes.data_as(C.c_void_p))
        assert rc == 0

    def step():
        threads = [threading.Thread(target=one, args=(i,)) for i in range(len(sample))]
        for t in threads:
            t.start()
        for t in threads:
            t.join()

    for _ in range(a.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(a.steps):
        step()
    dt = time.perf_counter() - t0
    value = tokens * a.steps / dt
    for h in caches:
        ref.ref_cache_destroy(h)
    desc = (f"first {len(sample)} of {a.batch} sequences ({tokens} seq-tokens), reference int4 pages (K per-channel, "
            f"V per-token fp32 scales), fp32 queries, one thread per sequence")
    line.update({"value": value, "ms_per_step": dt / a.steps * 1e3,
                 "cpu_baseline": {"value": value, "unit": UNIT, "cores": min(cores, len(sample)), "kind": "reference",
                                  "sample": desc},
                 "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                 "gpu_launches": 0})
    print(json.dumps(line))


def _oracle_books(layer):
    """The oracle's codebooks filled with the very tables the device uses."""
    from oracle import binding as ob
    books = []
    for host in layer.host_tables:
        cb = ob.codebook_from_hist(np.ones(256, np.uint64))
        slot = np.ctypeslib.as_array(host.rans_slot)
        cb.slot2sym[:] = (slot & 0xFF).astype(np.int32).tolist()
        cb.freq[:] = np.ctypeslib.as_array(host.rans_freq).astype(np.int32).tolist()
        cb.cum[:] = np.ctypeslib.as_array(host.rans_cum).astype(np.int32).tolist()
        cb.lut[:] = np.ctypeslib.as_array(host.huff_lut).astype(np.int32).tolist()
        books.append(cb)
    return books


def oracle_check(layer, q, out, slots=None, rows=None):
    """The checker handed to the configuration runs: the CPU oracle (restated reference decoders, dequantise, double
    online softmax) over the very records, page table and tails `layer` holds on the GPU, for the batch entries `rows`
    of q / out (entry i = slot i), or for all of q / out when `slots` names their slots."""
    from oracle import binding as ob
    import torch
    if rows is not None:
        idx = torch.as_tensor(rows, device=q.device)
        q, out, slots = q[idx], out[idx], list(rows)
    elif slots is None:
        slots = list(range(q.shape[0]))
    kcb, vcb = _oracle_books(layer)
    with torch.cuda.device(layer.device):
        arena = layer.arena[:layer.sealed_bytes() + 64].cpu().numpy()
        offsets = (layer.page_dir.cpu().numpy().astype(np.uint64) & np.uint64(0xFFFFFFFFFF)) * np.uint64(16)
        sel = np.asarray(slots)
        table = layer.page_table.cpu().numpy().astype(np.uint32)[sel]
        sealed = layer.sealed_tokens.cpu().numpy().astype(np.uint32)[sel]
        tails = layer.tail_tokens.cpu().numpy().astype(np.uint32)[sel]
        tk, tv = layer.tail_k.cpu().numpy()[sel], layer.tail_v.cpu().numpy()[sel]
    want = ob.sealed_decode_attention(arena, offsets, table, sealed, q.cpu().numpy(), layer.query_heads, layer.kv_heads,
                                      layer.head_dim, layer.page_tokens, layer.block_size, 0, 1.0 / np.sqrt(layer.head_dim),
                                      kcb, vcb, tail_k=tk, tail_v=tv, tail_count=tails, threads=os.cpu_count() or 1)
    err = np.abs(out.cpu().numpy() - want)
    return {"sequences_checked": len(slots), "seq_tokens_checked": int(sealed.sum() + tails.sum()), "max_abs_err": float(err.max()),
            "within_2e-3_rel_1e-3_abs": bool(np.all(err <= 1e-3 + 2e-3 * np.abs(want)))}


def other_configurations(a, device):
    """Configurations 3, 4 and 5 of the benchmark at their stated sizes on this GPU, each checked against the CPU oracle
    on a sample of its sequences (configuration 4: all eight); with them the block-size dial of configuration 3, the
    other head dimensions the fast kernel serves, and the sealer's own rate."""
    from types import SimpleNamespace
    from chromofold_b200 import config_bench as cb
    args = SimpleNamespace(steps=max(a.steps // 5, 5), warmup=3, coder=a.coder, batch4=8, ctx4=131072, seqs5=256,
                           prefix5=16384, suffix5=512)
    extra = {"config3": cb.config3(args, device, check=oracle_check)}
    extra["config3_block_sizes"] = cb.config3_blocks(args, device, check=oracle_check)   # 64 / 128 / 256 symbols per block
    extra["config4"] = cb.config4(args, device, 0, 1, check=oracle_check)
    extra["config5"] = cb.config5(args, device, check=oracle_check)
    extra["head_dims"] = cb.head_dim_dial(args, device, check=oracle_check)   # 16 x 96 / 64 / 32 pages
    extra["sealer"] = cb.seal_rate(args, device)
    rows = [r for rows in extra.values() for r in rows if "oracle_check" in r]
    extra["all_within_2e-3_rel_1e-3_abs"] = all(r["oracle_check"]["within_2e-3_rel_1e-3_abs"] for r in rows)
    return extra


def one_process_legs(a, world, contexts, single_gpu_ms):
    """What rank 0 adds to a multi-GPU run: the same batch placed over all GPUs (strong scaling) and configuration 4 with
    its kv heads sharded, both driven by this one process through the C-ABI batch scheduler (cf_b200_mg_*)."""
    from types import SimpleNamespace
    from chromofold_b200 import config_bench as cb
    devices = [f"cuda:{d}" for d in range(world)]
    args = SimpleNamespace(steps=max(a.steps // 2, 10), warmup=5, coder=a.coder, batch4=8, ctx4=131072)
    legs = {"strong_scaling": cb.strong_scaling_one_process(args, devices, contexts, a.coder, check=oracle_check,
                                                            single_gpu_ms=single_gpu_ms)}
    import torch
    torch.cuda.empty_cache()
    legs["config4"] = cb.config4_one_process(args, devices, check=oracle_check)
    return legs


def reference_abi_leg(a, contexts, device):
    """The same decode step through one of the reference's OWN calls: cf_llama_server_execute_batch_async (the llama-server
    runtime ABI, include/chromofold/llama_server_runtime.h:58-86) over slots filled with cf_llama_server_append_layer_async,
    with host buffers: every timed step copies the fp32 queries (the only query type that ABI has) from pinned host
    memory, makes the one call for all sequences, and copies the outputs back. The rows appended are Laplace values; the
    store behind the ABI quantises them per 16-token tile and seals them on the GPU as they arrive."""
    import ctypes as C
    import torch
    from chromofold_b200 import _native as N
    from chromofold_b200.workloads import laplace_codes
    lib = N.lib()
    lib.cf_llama_server_runtime_create.restype = C.c_void_p
    lib.cf_llama_server_last_error.restype = C.c_char_p
    cfg = N.LlamaServerConfig(1, HQ, HKV, D, T, BLOCK, 1 << 20, HQ // HKV, int(str(device).split(":")[-1]), 1, None,
                              b"benchmark", b"0" * 64)
    rt = C.c_void_p(lib.cf_llama_server_runtime_create(C.byref(cfg)))
    if not rt.value:
        return {"unavailable": "cf_llama_server_runtime_create refused the configuration"}
    err = lambda: lib.cf_llama_server_last_error(rt).decode()
    gen = torch.Generator(device=device)
    gen.manual_seed(11)
    n = len(contexts)
    t_build = time.time()
    for i, ctx in enumerate(contexts):
        if lib.cf_llama_server_slot_create(rt, C.c_int64(i + 1)) != 0:
            return {"unavailable": "slot_create: " + err()}
        for begin in range(0, int(ctx), 4096):
            tokens = min(4096, int(ctx) - begin)
            k = laplace_codes((tokens, HKV, D), a.laplace_b, gen, device) * 0.01
            v = laplace_codes((tokens, HKV, D), a.laplace_b, gen, device) * 0.01
            if lib.cf_llama_server_append_layer_async(rt, C.c_int64(i + 1), 0, begin, C.c_void_p(k.data_ptr()),
                                                      C.c_void_p(v.data_ptr()), tokens, None) != 0:
                return {"unavailable": "append_layer: " + err()}
    torch.cuda.synchronize()
    t_build = time.time() - t_build
    q_pin = torch.randn((n, HQ, D), dtype=torch.float32).pin_memory()
    out_pin = torch.zeros((n, HQ, D), dtype=torch.float32).pin_memory()
    q_dev = torch.zeros((n, HQ, D), dtype=torch.float32, device=device)
    out_dev = torch.zeros((n, HQ, D), dtype=torch.float32, device=device)
    items = (N.SequenceAttentionItem * n)()
    for i, ctx in enumerate(contexts):
        it = items[i]
        it.sequence_id, it.layer = i + 1, 0
        it.query = N.TensorView(q_dev[i].data_ptr(), N.F32, 1, HQ, D, HQ * D * 4, D * 4, 4, 0)
        it.output, it.output_type = out_dev[i].data_ptr(), N.F32
        it.output_token_stride_bytes, it.output_head_stride_bytes, it.output_element_stride_bytes = HQ * D * 4, D * 4, 4
        it.query_token_begin, it.softmax_scale, it.causal_window = int(ctx), 1.0 / float(np.sqrt(D)), 0
    batch = N.LlamaServerBatch(None, 0, C.cast(items, C.c_void_p), n)

    def step():
        q_dev.copy_(q_pin, non_blocking=True)
        if lib.cf_llama_server_execute_batch_async(rt, C.byref(batch), C.c_void_p(torch.cuda.current_stream().cuda_stream)) != 0:
            raise RuntimeError("execute_batch: " + err())
        out_pin.copy_(out_dev, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(3):
        step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(a.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / a.steps
    tokens = int(np.sum(contexts))
    result = {"call": "cf_llama_server_execute_batch_async (fp32 queries, one call for the batch)", "value": tokens / ms * 1e3,
              "unit": UNIT, "ms_per_step": ms, "h2d_bytes_per_step": int(q_pin.numel() * 4), "d2h_bytes_per_step": int(out_pin.numel() * 4),
              "fill_seconds_append_and_seal": round(t_build, 2), "finite_output": bool(torch.isfinite(out_pin).all().item())}
    lib.cf_llama_server_shutdown_async(rt, None)
    lib.cf_llama_server_runtime_destroy(rt, None)
    return result


def cpu_baseline(a, layer, contexts, q_host, out_gpu):
    """The CPU oracle on the same sealed records: restated reference decoders, dequantise, double online softmax,
    all host threads. Also the full-size parity check of the GPU result on the sampled sequences."""
    from oracle import binding as ob
    import torch
    cores = os.cpu_count() or 1
    kcb = ob.codebook_from_hist(np.ones(256, np.uint64))
    vcb = ob.codebook_from_hist(np.ones(256, np.uint64))
    for cb, host in ((kcb, layer.host_tables[0]), (vcb, layer.host_tables[1])):  # same tables as the device uses
        slot = np.ctypeslib.as_array(host.rans_slot)
        cb.slot2sym[:] = (slot & 0xFF).astype(np.int32).tolist()
        cb.freq[:] = np.ctypeslib.as_array(host.rans_freq).astype(np.int32).tolist()
        cb.cum[:] = np.ctypeslib.as_array(host.rans_cum).astype(np.int32).tolist()
        cb.lut[:] = np.ctypeslib.as_array(host.huff_lut).astype(np.int32).tolist()
    arena = layer.arena[:layer.sealed_bytes() + 64].cpu().numpy()
    entries = layer.page_dir.cpu().numpy().astype(np.uint64)
    offsets = (entries & np.uint64(0xFFFFFFFFFF)) * np.uint64(16)
    table = layer.h_page_table.astype(np.uint32)
    scale = 1.0 / np.sqrt(D)

    def run(n):
        t0 = time.perf_counter()
        out = ob.sealed_decode_attention(arena, offsets, table[:n], contexts[:n].astype(np.uint32), q_host[:n], HQ, HKV,
                                         D, T, BLOCK, 0, scale, kcb, vcb, threads=cores)
        return time.perf_counter() - t0, out

    n = min(2, len(contexts))
    dt, out = run(n)
    rate = contexts[:n].sum() / dt
    budget_tokens = rate * a.cpu_seconds
    n_full = int(np.searchsorted(np.cumsum(contexts), budget_tokens)) + 1
    n_full = max(n, min(len(contexts), n_full))
    if n_full > n:
        dt, out = run(n_full)
        n = n_full
    tokens = int(contexts[:n].sum())
    got = out_gpu[:n].cpu().numpy()
    err = np.abs(got - out)
    ok = bool(np.all(err <= 1e-3 + 2e-3 * np.abs(out)))
    return ({"value": tokens / dt, "unit": UNIT, "cores": cores, "kind": "port",
             "sample": f"first {n} of {len(contexts)} sequences ({tokens} seq-tokens), same sealed records, all host threads"},
            {"sequences_checked": n, "max_abs_err": float(err.max()), "within_2e-3_rel_1e-3_abs": ok})


def main():
    a = parse()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if a.impl == "reference":
        run_reference(a, rank)
        return

    import torch
    import torch.distributed as dist
    from chromofold_b200 import _native as N
    from chromofold_b200.workloads import build_sealed_layer, uniform_contexts

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the library has no CPU path")
    torch.cuda.set_device(local_rank)
    device = f"cuda:{local_rank}"
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(device))

    if a.scaling == "strong" and world > 1:
        from chromofold_b200.scheduler import shard_sequences
        everyone = uniform_contexts(a.batch, a.ctx_lo, a.ctx_hi, T, 3)
        contexts = everyone[shard_sequences(everyone, world)[rank]]
    else:
        # weak scaling: the same context-length multiset on every rank (fixed work per GPU), different codes and queries
        contexts = uniform_contexts(a.batch, a.ctx_lo, a.ctx_hi, T, 3)
    n_local = len(contexts)
    layer, info = build_sealed_layer(contexts, query_heads=HQ, kv_heads=HKV, head_dim=D, page_tokens=T, block_size=BLOCK,
                                     coder=a.coder, dist=("laplace", a.laplace_b), seed=4 + 1000 * rank, device=device,
                                     keep_dense=not a.no_dense)
    gen = torch.Generator(device=device)
    gen.manual_seed(5 + 1000 * rank)
    q = torch.randn((n_local, HQ, D), generator=gen, device=device, dtype=torch.float32).half()
    if a.f32_queries:
        q = q.float()
    out = torch.zeros((n_local, HQ, D), dtype=torch.float32, device=device)
    kernel = {"auto": N.KERNEL_AUTO, "generic": N.KERNEL_GENERIC, "lanes": N.KERNEL_LANES}[a.kernel]
    kw = dict(kernel=kernel, min_pages_per_unit=a.min_pages_per_unit)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    step = lambda: layer.attention(q, out=out, **kw)
    for _ in range(max(a.warmup, 3)):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    t0 = time.time()
    ms = timed(step, a.steps)

    # end to end: queries come from pinned host memory, the result goes back to pinned host memory, every step
    q_pin = q.cpu().pin_memory()
    out_pin = torch.zeros((n_local, HQ, D), dtype=torch.float32).pin_memory()
    q_dev = torch.empty_like(q)

    def e2e_step():
        q_dev.copy_(q_pin, non_blocking=True)
        layer.attention(q_dev, out=out, **kw)
        out_pin.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()  # the caller needs the result before the next step

    for _ in range(3):
        e2e_step()
    ms_e2e = timed(e2e_step, a.steps)

    # the page-reading kernel alone: events between the three stages
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(a.steps)]
    torch.cuda.synchronize()
    for s in range(a.steps):
        ev[s][0].record()
        layer.attention(q, out=out, stages=N.STAGE_PLAN, **kw)
        ev[s][1].record()
        layer.attention(q, out=out, stages=N.STAGE_ATTENTION, **kw)
        ev[s][2].record()
        layer.attention(q, out=out, stages=N.STAGE_COMBINE, **kw)
        ev[s][3].record()
    # the decode floor: the same launch without its attention (page fetch + entropy decode only)
    probe_kw = dict(kw, kernel=N.KERNEL_DECODE_PROBE)
    for _ in range(3):
        layer.attention(q, out=out, stages=N.STAGE_PLAN | N.STAGE_ATTENTION, **probe_kw)
    pe = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(a.steps)]
    for s_ in range(a.steps):   # the plan stage re-arms the kernel's work counter, so it runs before every launch
        layer.attention(q, out=out, stages=N.STAGE_PLAN, **probe_kw)
        pe[s_][0].record()
        layer.attention(q, out=out, stages=N.STAGE_ATTENTION, **probe_kw)
        pe[s_][1].record()
    torch.cuda.synchronize()
    decode_only_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in pe])) if a.kernel != "generic" else None
    layer.attention(q, out=out, **kw)   # leave a real result in `out`
    torch.cuda.synchronize()
    t1 = time.time()
    stage_ms = [float(np.mean([ev[s][i].elapsed_time(ev[s][i + 1]) for s in range(a.steps)])) for i in range(3)]
    per_launch = np.array([ev[s][1].elapsed_time(ev[s][2]) for s in range(a.steps)])   # the attention kernel, launch by launch
    clocks = sampler.stop(t0, t1) if sampler else None
    status = layer.device_status()

    tokens_rank = int(contexts.sum())
    tokens_all = torch.tensor([tokens_rank], device=device, dtype=torch.float64)
    bytes_all = torch.tensor([float(info["sealed_bytes"])], device=device, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(tokens_all)
        dist.all_reduce(bytes_all)
    tokens_total = float(tokens_all.item())

    dense = None
    if not a.no_dense:
        from chromofold_b200.cache import dense_attention
        try:
            out_d = torch.zeros_like(out)
            dfn = lambda: dense_attention(layer, info["dense_k"], info["dense_v"], q.half(), out_d)
            for _ in range(3):
                dfn()
            ms_d = timed(dfn, a.steps)
            err = float((out_d - out).abs().max().item())
            dense_bytes = tokens_rank * info["fp16_bytes_per_seq_token"]
            dense = {"value": tokens_total * a.steps / (ms_d * 1e-3), "unit": UNIT, "ms_per_step": ms_d / a.steps,
                     "hbm_gbs": dense_bytes * a.steps / (ms_d * 1e-3) / 1e9, "bytes_per_seq_token": info["fp16_bytes_per_seq_token"],
                     "max_abs_diff_vs_sealed": err}
        except N.CfError as e:
            dense = {"unavailable": str(e)}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        pass
    peak = float(peaks.get("hbm_gbs", 6650.0))
    peak_kind = "measured" if "hbm_gbs" in peaks else "fallback"
    # algorithmic bytes of one attention launch on this rank: every sealed record once, the page table, Q in, partials out
    algo_bytes = info["sealed_bytes"] + 4 * info["pages"] + n_local * HQ * D * 2
    att_s = stage_ms[1] * 1e-3
    achieved = algo_bytes / att_s / 1e9
    line = {
        "metric": METRIC, "value": tokens_total * a.steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": a.steps,
        "warmup": max(a.warmup, 3), "ms_per_step": ms / a.steps, "higher_is_better": True, "scaling": a.scaling,
        "vs_baseline": None, "dtype": "u8 codes, f16 mma operands, f32 accumulate", "data": "synthetic",
        "config": {"workload": workload_name(a), "global_batch": a.batch * world if a.scaling == "weak" else a.batch,
                   "seq_tokens_per_step": tokens_total,
                   "sharding": (f"sequences, {a.batch} per GPU, same context lengths on every GPU, no collective" if a.scaling == "weak" else
                                f"{a.batch} sequences bin-packed over {world} GPUs by context length, no collective"), "l2": "inputs larger than L2 (sealed bytes per GPU "
                   f"{info['sealed_bytes'] / 1e9:.2f} GB vs 126 MB)", "kernel": a.kernel,
                   "h0_bits_per_code": {"k": info["h0_bits_k"], "v": info["h0_bits_v"]},
                   "sealed_bytes_per_seq_token": info["bytes_per_seq_token"],
                   "fp16_bytes_per_seq_token": info["fp16_bytes_per_seq_token"],
                   "kv_memory_reduction_vs_fp16": info["fp16_bytes_per_seq_token"] / info["bytes_per_seq_token"],
                   "whole_model_32_layers_seq_tokens_per_s": tokens_total * a.steps / (ms * 1e-3) / 32},
        "e2e": {"value": tokens_total * a.steps / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e / a.steps,
                "h2d_bytes_per_step": int(q_pin.numel() * 2), "d2h_bytes_per_step": int(out_pin.numel() * 4)},
        "gpu_launches": 3 * a.steps,
        "roofline": {"bound": "hbm", "kernel": "lanes_attention_kernel" if a.kernel != "generic" else "generic_attention_kernel",
                     "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind,
                     "frac_of_nominal_8000": achieved / 8000.0,
                     "traffic": (int(algo_bytes * DRAM_TRAFFIC_RATIO[a.coder]) if a.kernel != "generic" else None),
                     "traffic_source": "ncu dram bytes of the batch-16 capture scaled by algorithmic bytes",
                     "algorithmic_bytes_per_launch": algo_bytes, "kernel_ms": stage_ms[1],
                     "plan_ms": stage_ms[0], "combine_ms": stage_ms[2], "decode_only_ms": decode_only_ms,
                     "kernel_ms_median": float(np.median(per_launch)), "kernel_ms_p5": float(np.percentile(per_launch, 5)),
                     "kernel_ms_p95": float(np.percentile(per_launch, 95)),
                     "kernel_ms_cv": float(per_launch.std() / per_launch.mean()),
                     "decompressed_equivalent_gbs": tokens_rank * info["fp16_bytes_per_seq_token"] / att_s / 1e9},
        "clocks": clocks, "device_status": status, "dense_fp16": dense,
    }
    if world == 1 and not a.no_cpu:
        base, parity = cpu_baseline(a, layer, contexts, q.cpu().numpy(), out)
        line["cpu_baseline"] = base
        line["parity_full_size"] = parity
    if world == 1 and not a.no_others:
        # the same codes sealed with the other coders of the format, timed the same way (device-resident inputs)
        others = {}
        info.pop("dense_k", None)
        info.pop("dense_v", None)
        del layer
        torch.cuda.empty_cache()
        for coder in ("rans", "rans4", "huffman", "huffman4", "fixed8"):
            if coder == a.coder:
                continue
            other, oinfo = build_sealed_layer(contexts, query_heads=HQ, kv_heads=HKV, head_dim=D, page_tokens=T,
                                              block_size=BLOCK, coder=coder, dist=("laplace", a.laplace_b), seed=4,
                                              device=device)
            ostep = lambda: other.attention(q, out=out, **kw)
            for _ in range(5):
                ostep()
            oms = timed(ostep, a.steps)
            others[coder] = {"value": tokens_total * a.steps / (oms * 1e-3), "unit": UNIT, "ms_per_step": oms / a.steps,
                             "sealed_bytes_per_seq_token": oinfo["bytes_per_seq_token"],
                             "kv_memory_reduction_vs_fp16": oinfo["fp16_bytes_per_seq_token"] / oinfo["bytes_per_seq_token"],
                             "sealed_gbs": oinfo["sealed_bytes"] * a.steps / (oms * 1e-3) / 1e9,
                             "frac_of_peak": oinfo["sealed_bytes"] * a.steps / (oms * 1e-3) / 1e9 / peak,
                             "device_status": other.device_status()}
            del other, oinfo
            torch.cuda.empty_cache()
        line["other_coders"] = others
    if world > 1:
        dist.destroy_process_group()
    if world == 1 and not a.no_configs:
        try:
            del layer
        except NameError:
            pass
        torch.cuda.empty_cache()
        line["e2e"]["reference_abi"] = reference_abi_leg(a, contexts, device)
    if not a.no_configs:
        try:
            del layer
        except NameError:
            pass
        torch.cuda.empty_cache()
        line["extra"] = (other_configurations(a, device) if world == 1
                         else one_process_legs(a, world, contexts, ms / a.steps))
    print(json.dumps(line))


if __name__ == "__main__":
    main()
