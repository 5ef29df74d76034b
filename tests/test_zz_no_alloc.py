"""The allocation-free attention entry point (cf_b200_sealed_attention_static_async).

Some callers cannot hand the library a workspace because they cannot allocate device memory where they call it.
This entry point uses an array built into the library instead. The test drives it through the C ABI and checks
that it gives what the ordinary entry point gives, twice in a row (the array keeps the previous call's contents),
and that an over-sized batch is refused with a message instead of overrunning the array.

The file name sorts last on purpose: if this test fails, a run that stops at the first failure has already run
every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _small_layer(native, contexts, seed):
    import torch
    from chromofold_b200.cache import SealedKvLayer
    rng = np.random.default_rng(seed)
    hq, hkv, d, t = 8, 2, 128, 16
    pages = [c // t for c in contexts]
    layer = SealedKvLayer(kv_heads=hkv, query_heads=hq, head_dim=d, page_tokens=t, block_size=64,
                          coder=native.CODER_RANS, max_sequences=len(contexts), max_pages_per_sequence=max(pages) + 1,
                          max_pages=sum(pages) + 4, arena_bytes=(sum(pages) + 4) * hkv * 4200)
    codes = np.rint(rng.laplace(0, 12.0, 1 << 15)).clip(-128, 127).astype(np.int64) + 128
    hist = np.bincount(codes, minlength=256).astype(np.uint64)
    layer.set_codebooks(hist, hist)
    for p in range(max(pages)):
        live = [s for s in range(len(contexts)) if pages[s] > p]
        k = (np.rint(rng.laplace(0, 12.0, (len(live), hkv, t, d))).clip(-127, 127) * 0.01).astype(np.float16)
        v = (np.rint(rng.laplace(0, 12.0, (len(live), hkv, t, d))).clip(-127, 127) * 0.01).astype(np.float16)
        layer.seal_tiles(live, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
    tail = 5
    tk = (rng.standard_normal((len(contexts), hkv, t, d)) * 0.5).astype(np.float16)
    tv = (rng.standard_normal((len(contexts), hkv, t, d)) * 0.5).astype(np.float16)
    layer.fill_tails(list(range(len(contexts))), torch.from_numpy(tk).cuda(), torch.from_numpy(tv).cuda(), tail)
    q = torch.from_numpy(rng.standard_normal((len(contexts), hq, d)).astype(np.float16)).cuda()
    return layer, q


def test_no_alloc_entry_matches_the_ordinary_one_twice(native):
    import torch
    for round_, contexts in enumerate([[16 * 40, 16 * 3, 16 * 17], [16 * 9, 16 * 64]]):
        layer, q = _small_layer(native, contexts, seed=50 + round_)
        for kernel in (native.KERNEL_LANES, native.KERNEL_GENERIC):
            want = layer.attention(q, kernel=kernel).cpu().numpy()
            got1 = layer.attention_no_alloc(q, kernel=kernel).cpu().numpy()
            got2 = layer.attention_no_alloc(q, kernel=kernel).cpu().numpy()   # second call sees the first call's leftovers
            torch.cuda.synchronize()
            for got in (got1, got2):
                err = np.abs(got - want)
                assert np.all(err <= 1e-3 + 2e-3 * np.abs(want)), float(err.max())
            assert np.array_equal(got1, got2)
        assert layer.device_status() == 0


def test_no_alloc_entry_grows_its_units_to_fit_the_fixed_array(native):
    """The one code path a fixed-size workspace adds: a batch with more (chunk, head) partials at the usual unit size
    than the array holds. 4 sequences x 9000 pages at 16 pages per unit are 2250 chunks x 8 query heads x 520 B = 9.4 MB
    against the array's 8 MiB, so the plan kernel has to double its unit size; the result must still equal the ordinary
    entry point's (which has all the room it wants), on two calls in a row."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    layer, _ = build_sealed_layer(np.array([16 * 9000] * 4), query_heads=8, kv_heads=2, coder="rans4", seed=52)
    g = torch.Generator(device="cuda")
    g.manual_seed(53)
    q = torch.randn((4, 8, 128), generator=g, device="cuda", dtype=torch.float32).half()
    want = layer.attention(q, kernel=native.KERNEL_LANES, min_pages_per_unit=16).cpu().numpy()
    got1 = layer.attention_no_alloc(q, kernel=native.KERNEL_LANES).cpu().numpy()
    got2 = layer.attention_no_alloc(q, kernel=native.KERNEL_LANES).cpu().numpy()
    assert layer.device_status() == 0
    for got in (got1, got2):
        err = np.abs(got - want)
        assert np.all(err <= 1e-3 + 2e-3 * np.abs(want)), float(err.max())
    assert np.array_equal(got1, got2)


def test_no_alloc_entry_with_a_shared_prefix_hint(native):
    """The hint needs 16 more partials per sequence and query head. Six sequences that share 24 pages: it fits and the
    shared-prefix kernel runs. 900 batch entries over the same pages: only the plain partials fit (900 x 8 x 520 B =
    3.7 MB, x 17 with the hint), so the call is served without the hint instead of refused."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    layer, _ = build_sealed_layer(np.array([16 * 24] + [0] * 5), query_heads=8, kv_heads=2, coder="rans4", seed=54,
                                  extra_pages_per_sequence=4)
    for s in range(1, 6):
        layer.copy_sequence(0, s)
    g = torch.Generator(device="cuda")
    g.manual_seed(55)
    q = torch.randn((900, 8, 128), generator=g, device="cuda", dtype=torch.float32).half()
    launches = native.lib().cf_b200_shared_prefix_launches
    launches.restype = C.c_ulonglong
    before = launches()
    want = layer.attention(q[:6].contiguous(), kernel=native.KERNEL_LANES).cpu().numpy()
    got = layer.attention_no_alloc(q[:6].contiguous(), kernel=native.KERNEL_LANES, shared_prefix_pages=24).cpu().numpy()
    assert launches() == before + 1 and layer.device_status() == 0
    err = np.abs(got - want)
    assert np.all(err <= 1e-3 + 2e-3 * np.abs(want)), float(err.max())
    slots = [i % 6 for i in range(900)]
    big = layer.attention_no_alloc(q, slots=slots, kernel=native.KERNEL_LANES, shared_prefix_pages=24).cpu().numpy()
    assert launches() == before + 1 and layer.device_status() == 0          # served, without the shared-prefix kernel
    err = np.abs(big[:6] - want)                  # entries 0..5 are the six sequences with the same queries as above
    assert np.all(err <= 1e-3 + 2e-3 * np.abs(want)), float(err.max())


def test_no_alloc_entry_refuses_a_batch_that_cannot_fit(native):
    layer, q = _small_layer(native, [16 * 2], seed=60)
    d = layer._attention_desc(q, q.float(), 1, None)
    d.softmax_scale = 0.088
    d.workspace, d.workspace_bytes = None, 0
    d.seq_count = 200000   # 200000 sequences x 8 heads x 130 floats is far beyond the built-in array
    lib = native.lib()
    assert lib.cf_b200_sealed_attention_static_async(C.byref(d), None) == native.CF_ERR_UNSUPPORTED
    assert b"too large" in lib.cf_b200_sealed_attention_static_error()
    assert lib.cf_b200_sealed_attention_static_async(None, None) == native.CF_ERR_INVALID_ARGUMENT
