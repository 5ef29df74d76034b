"""The one-process batch scheduler (include/chromofold_b200/sealed_kv_multigpu.h) on the GPUs that are there: with one
GPU it still goes through its own streams, row permutation and copies; with two or more it shards for real."""
import numpy as np
import pytest

from helpers import attention_close, oracle_from_layer

pytestmark = pytest.mark.gpu


def _queries(n, hq, seed, device):
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return torch.randn((n, hq, 128), generator=g, device=device, dtype=torch.float32).half()


def _devices():
    import torch
    return min(torch.cuda.device_count(), 4)


@pytest.mark.parametrize("coder", ["rans4", "huffman"])
def test_sequences_sharded_over_the_devices_of_one_process(native, oracle, coder):
    """A batch of 11 sequences placed by the C planner; every device holds only its own sequences' pages; the gathered
    output equals what one store holding everything returns, and the oracle's result."""
    import torch
    from chromofold_b200.scheduler import MultiGpuScheduler
    from chromofold_b200.workloads import build_sealed_layer
    world = _devices()
    contexts = (np.arange(11) * 37 % 23 + 1) * 16 * 4
    whole, _ = build_sealed_layer(contexts, coder=coder, seed=90, device="cuda:0")
    q = _queries(11, 32, 91, "cuda:0")
    want = whole.attention(q, min_pages_per_unit=16).cpu().numpy()   # units pinned: the same split-KV cut in every store
    ok, err = attention_close(want, oracle_from_layer(whole, q.cpu().numpy()))
    assert ok, err
    # the same pages, spread: the records are copied out of the one store into per-device stores, page by page
    from chromofold_b200.scheduler import shard_sequences
    assignment = shard_sequences(contexts, world)     # the C planner gives the same placement (checked below)
    layers, local_slots = [], []
    for d in range(world):
        mine = assignment[d]
        lay, _ = build_sealed_layer(np.array([0] * max(len(mine), 1)), coder=coder, seed=93 + d, device=f"cuda:{d}",
                                    extra_pages_per_sequence=int(contexts.max()) // 16 + 2, reserve_pages=int(contexts.sum()) // 16 + 8)
        lay.k_tables.copy_(whole.k_tables.to(lay.device))
        lay.v_tables.copy_(whole.v_tables.to(lay.device))
        lay.host_tables = whole.host_tables
        for local, seq in enumerate(mine):
            pages = int(contexts[seq]) // 16
            recs = [[whole.record_bytes(int(whole.h_page_table[seq, p]), h) for h in range(8)] for p in range(pages)]
            lay.import_records(local, recs)
        layers.append(lay)
        local_slots.append(list(range(len(mine))))
    # the copy path first (staging, row permutation, copies back), then the default, which stores the output rows
    # straight into the root's tensor wherever the GPUs have the root's memory mapped
    import os
    os.environ["CHROMOFOLD_B200_MG_COPIES"] = "1"
    try:
        copying = MultiGpuScheduler(layers, max_rows=16)
    finally:
        del os.environ["CHROMOFOLD_B200_MG_COPIES"]
    out = torch.zeros((11, 32, 128), dtype=torch.float32, device="cuda:0")
    copying.attention_by_sequence(q, out, assignment, local_slots, min_pages_per_unit=16)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), want) and copying.counters()["direct_steps"] == 0
    copying.close()
    sched = MultiGpuScheduler(layers, max_rows=16)
    assert sched.plan_sequences(contexts) == assignment
    for _ in range(2):    # the second step reuses the cached row order
        out.zero_()
        sched.attention_by_sequence(q, out, assignment, local_slots, min_pages_per_unit=16)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want)
    c = sched.counters()
    assert c["steps"] == 2 and c["attention_launches"] == 2 * sum(1 for a in assignment if a)
    assert c["direct_steps"] in (0, 2) and (world > 1 or c["direct_steps"] == 2)
    assert all(lay.device_status() == 0 for lay in layers)
    # a device marked failed: the batch that names it is refused, the planner routes around it
    if world > 1:
        sched.set_device_failed(1)
        with pytest.raises(native.CfError):
            sched.attention_by_sequence(q, out, assignment, local_slots, min_pages_per_unit=16)
        assert sched.plan_sequences(contexts)[1] == []
        assert sched.counters()["refused_batches"] == 1
    sched.close()


def test_kv_heads_sharded_over_the_devices_of_one_process(native, oracle):
    """70B-shaped groups (64 query / 8 kv heads): every device serves all rows with its block of kv heads (a replica of
    the store per device here) and its query-head columns are gathered into the root's output."""
    import torch
    from chromofold_b200.scheduler import MultiGpuScheduler
    from chromofold_b200.workloads import build_sealed_layer
    world = _devices()
    contexts = np.array([1024, 2048, 512])
    layers = [build_sealed_layer(contexts, query_heads=64, kv_heads=8, coder="rans4", seed=95, device=f"cuda:{d}")[0] for d in range(world)]
    q = _queries(3, 64, 96, "cuda:0")
    want = layers[0].attention(q, min_pages_per_unit=16).cpu().numpy()
    ok, err = attention_close(want, oracle_from_layer(layers[0], q.cpu().numpy()))
    assert ok, err
    sched = MultiGpuScheduler(layers, max_rows=8)
    for ways in sorted({1, world}):
        heads = sched.plan_kv_heads(8) if ways == world else [(0, 8)] + [(0, 0)] * (world - 1)
        assert sum(s for _, s in heads) == 8
        out = torch.zeros((3, 64, 128), dtype=torch.float32, device="cuda:0")
        sched.attention_by_kv_head(q, out, heads, [0, 1, 2], min_pages_per_unit=16)
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), want), ways
    sched.close()


def test_memory_of_another_gpu_is_refused_before_any_launch(native):
    """The entry points launch on the current device; a descriptor whose arena lies on another GPU is turned down with
    CF_ERR_INVALID_ARGUMENT instead of being launched (nothing runs, nothing faults)."""
    import ctypes as C
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    layer, _ = build_sealed_layer(np.array([64, 32]), coder="rans4", seed=97, device="cuda:1")
    q = _queries(2, 32, 98, "cuda:1")
    out = torch.zeros((2, 32, 128), dtype=torch.float32, device="cuda:1")
    desc = layer._attention_desc(q, out, 2, None)
    desc.softmax_scale = 0.088
    with torch.cuda.device(0):
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert native.lib().cf_b200_sealed_attention_async(C.byref(desc), stream) == native.CF_ERR_INVALID_ARGUMENT
    with torch.cuda.device(1):
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert native.lib().cf_b200_sealed_attention_async(C.byref(desc), stream) == native.CF_OK
        torch.cuda.synchronize()
    assert layer.device_status() == 0


def _scheduler_run(native, seed):
    import os
    import torch
    from chromofold_b200.scheduler import MultiGpuScheduler
    from chromofold_b200.workloads import build_sealed_layer
    rng = np.random.default_rng(seed)
    world = min(torch.cuda.device_count(), 4)
    n = int(rng.integers(1, 24))
    hq, hkv = [(32, 8), (64, 8), (8, 8)][int(rng.integers(0, 3))]
    coder = ["rans4", "huffman4", "rans", "fixed8"][int(rng.integers(0, 4))]
    contexts = rng.integers(1, 60, n) * 16
    whole, _ = build_sealed_layer(contexts, query_heads=hq, kv_heads=hkv, coder=coder, seed=seed, device="cuda:0")
    where = rng.integers(0, world, n)           # an arbitrary placement, not the planner's
    layers, slot_of = [], {}
    for d in range(world):
        mine = [s for s in range(n) if where[s] == d]
        lay, _ = build_sealed_layer(np.array([0] * max(len(mine), 1)), query_heads=hq, kv_heads=hkv, coder=coder, seed=seed + 1 + d, device=f"cuda:{d}",
                                    extra_pages_per_sequence=int(contexts.max()) // 16 + 2, reserve_pages=int(contexts.sum()) // 16 + 8)
        lay.k_tables.copy_(whole.k_tables.to(lay.device)); lay.v_tables.copy_(whole.v_tables.to(lay.device)); lay.host_tables = whole.host_tables
        for local, seq in enumerate(mine):
            pages = int(contexts[seq]) // 16
            recs = [[whole.record_bytes(int(whole.h_page_table[seq, p]), h) for h in range(hkv)] for p in range(pages)]
            lay.import_records(local, recs); slot_of[seq] = (d, local)
        layers.append(lay)
    copies = rng.random() < 0.3
    if copies: os.environ["CHROMOFOLD_B200_MG_COPIES"] = "1"
    try: sched = MultiGpuScheduler(layers, max_rows=32)
    finally: os.environ.pop("CHROMOFOLD_B200_MG_COPIES", None)
    g = torch.Generator(device="cuda:0"); g.manual_seed(seed)
    for step in range(int(rng.integers(2, 6))):
        m = int(rng.integers(1, n + 1))
        subset = [int(x) for x in rng.choice(n, m, replace=False)]          # row i of the batch is sequence subset[i]
        if step and rng.random() < 0.4: subset = prev                        # the same placement again (cached row order)
        prev = subset; m = len(subset)
        q = torch.randn((m, hq, 128), generator=g, device="cuda:0", dtype=torch.float32).half()
        want = whole.attention(q, slots=subset, min_pages_per_unit=16).cpu().numpy()
        assignment = [[i for i, s in enumerate(subset) if slot_of[s][0] == d] for d in range(world)]
        local_slots = [[slot_of[subset[i]][1] for i in assignment[d]] for d in range(world)]
        out = torch.full((m, hq, 128), 5.0, dtype=torch.float32, device="cuda:0")
        sched.attention_by_sequence(q, out, assignment, local_slots, min_pages_per_unit=16)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        if not np.array_equal(got, want):
            return ("step", step, float(np.abs(got - want).max()), dict(seed=seed, n=n, m=m, heads=(hq, hkv), coder=coder, copies=copies, world=world))
    ok = all(l.device_status() == 0 for l in layers)
    sched.close()
    return None if ok else ("status",)


@pytest.mark.parametrize("first", range(0, 12, 6))
def test_random_placements_and_changing_batches(native, first):
    """Sequences placed on the devices at random (not by the planner), then several steps through ONE scheduler whose
    batches change from step to step — a random subset of the sequences in a random row order, or the same batch again
    (the cached row order) — on the direct-store path or the copy path: every step equals the answer of one store
    holding everything, bit for bit."""
    for seed in range(500 + first, 500 + first + 6):
        bad = _scheduler_run(native, seed)
        assert bad is None, bad
