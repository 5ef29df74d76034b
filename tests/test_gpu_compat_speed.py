"""The reference's own CUDA entry points, timed on the same inputs against the reference's own kernels (compiled from
its sources into oracle/_ref): this library must not be slower on any of them. Prints the timings (pytest -s)."""
import ctypes as C

import numpy as np
import pytest

from compat_types import DevicePage, PagedAttentionDesc
from helpers import hist_of, laplace_codes
from test_gpu_compat import _dev, _fixture_pages

pytestmark = pytest.mark.gpu


def _time_us(fn, steps):
    import torch
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps * 1000.0


def _both(native, oracle):
    ref = oracle.ref_cuda()
    if ref is None:
        pytest.skip("needs oracle/_ref (the reference's kernels)")
    return (("this library", native.lib()), ("reference kernel", ref))


def test_rans_decode_entry_is_not_slower_than_the_reference_kernel(native, oracle):
    """specs/03-roadmap.md:130-136 quotes this micro-benchmark (block 64) for the reference."""
    import torch
    rng = np.random.default_rng(8)
    n, block = 16 * 1024 * 1024, 64   # large enough for the device time to dominate the launch overhead of the two calls
    sym = (laplace_codes(rng, n, 12.0).astype(np.int16) + 128).astype(np.uint8)
    cb = oracle.codebook_from_hist(hist_of(sym))
    data, off, st = oracle.rans_encode(sym, block, cb)
    args = [_dev(np.concatenate([data, np.zeros(8, np.uint8)])), _dev(off), _dev(st), _dev(cb.np("slot2sym")), _dev(cb.np("freq")),
            _dev(cb.np("cum"))]
    times = {}
    for name, lib in _both(native, oracle):
        out = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        call = lambda: lib.cf_rans_decode_async(*[C.c_void_p(x.data_ptr()) for x in args], C.c_int(block), C.c_int(n),
                                                C.c_void_p(out.data_ptr()), None)
        times[name] = _time_us(call, 20)
        assert np.array_equal(out.cpu().numpy(), sym.astype(np.int32))
        print(f"cf_rans_decode_async, {n} symbols, block {block}: {name:17s} {times[name]:9.1f} us = {n / times[name] / 1e3:6.1f} G symbols/s")
    assert times["this library"] <= times["reference kernel"]


@pytest.mark.parametrize("case", [(32, 8, 1), (32, 4, 1), (16, 8, 8)], ids=str)
def test_paged_attention_entry_is_not_slower_than_the_reference_kernel(native, oracle, case):
    """cf_kv_paged_attention_async over the reference's own fixed-width pages: a decode step (one query token) and a small
    prompt batch of a 32-query-head / 8-kv-head model, 128-token pages."""
    import torch
    npages, bits, nq = case
    hq, hkv, d, page = 32, 8, 128, 128
    rng = np.random.default_rng(1)
    pages, keep, dk, dv = _fixture_pages(oracle, rng, hkv, d, [page] * npages, bits)
    sealed, tail = page * npages, 6
    tk = rng.standard_normal((tail, hkv, d)).astype(np.float32)
    tv = rng.standard_normal((tail, hkv, d)).astype(np.float32)
    q = rng.standard_normal((nq, hq, d)).astype(np.float32)
    arr = (DevicePage * len(pages))(*pages)
    d_pages = _dev(np.frombuffer(bytes(arr), np.uint8))
    d_tk, d_tv, d_q = _dev(tk), _dev(tv), _dev(q)
    desc = PagedAttentionDesc()
    desc.struct_size, desc.abi_version = C.sizeof(desc), 0
    desc.pages, desc.page_count = d_pages.data_ptr(), len(pages)
    desc.kv_head_count, desc.query_head_count, desc.gqa_group_size = hkv, hq, hq // hkv
    desc.active_k, desc.active_v, desc.active_token_begin, desc.active_token_count = d_tk.data_ptr(), d_tv.data_ptr(), sealed, tail
    desc.queries, desc.query_token_begin, desc.query_count = d_q.data_ptr(), sealed + tail - nq, nq
    desc.head_dim, desc.causal_window, desc.softmax_scale = d, 0, 1.0 / np.sqrt(d)
    times, outs = {}, {}
    for name, lib in _both(native, oracle):
        out = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda")
        desc.output = out.data_ptr()

        def call():
            assert lib.cf_kv_paged_attention_async(C.byref(desc), None) == 0
        times[name] = _time_us(call, 10)
        outs[name] = out.cpu().numpy()
        print(f"cf_kv_paged_attention_async, int{bits}, {npages} x {page} tokens, {nq} query tokens: {name:17s} {times[name]:9.1f} us")
    assert np.abs(outs["this library"] - outs["reference kernel"]).max() <= 2e-4
    assert times["this library"] <= times["reference kernel"]


def test_flat_fused_attention_entry_is_not_slower_than_the_reference_kernel(native, oracle):
    """cf_kv_attn_fused_async (include/chromofold/chromofold.h:81-89): one head, block-Huffman K / V, sliding window."""
    import torch
    seq, dim, nq, window, block = 4096, 128, 4096, 512, 64
    rng = np.random.default_rng(2)
    ksym = (laplace_codes(rng, seq * dim, 9.0).astype(np.int16) + 128).astype(np.uint8)
    vsym = (laplace_codes(rng, seq * dim, 14.0).astype(np.int16) + 128).astype(np.uint8)
    kcb, vcb = oracle.codebook_from_hist(hist_of(ksym)), oracle.codebook_from_hist(hist_of(vsym))
    kw, kb = oracle.huff_encode(ksym, block, kcb)
    vw, vb = oracle.huff_encode(vsym, block, vcb)
    kscale = rng.uniform(0.005, 0.02, dim).astype(np.float32)
    vscale = rng.uniform(0.005, 0.02, seq).astype(np.float32)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    pad = np.zeros(2, np.uint32)
    dev = [_dev(np.concatenate([kw, pad])), _dev(kb), _dev(kcb.np("lut")), _dev(np.concatenate([vw, pad])), _dev(vb),
           _dev(vcb.np("lut")), _dev(kscale), _dev(vscale), _dev(q)]
    p = [C.c_void_p(t.data_ptr()) for t in dev]
    times, outs = {}, {}
    for name, lib in _both(native, oracle):
        fused = torch.zeros((nq, dim), dtype=torch.float32, device="cuda")
        tail = (C.c_int(seq), C.c_int(dim), C.c_int(nq), C.c_int(window), C.c_int(block), C.c_int(128), C.c_float(1.0 / np.sqrt(dim)), None)
        head = (p[0], p[1], p[2], C.c_int(12), p[3], p[4], p[5], C.c_int(12), p[6], p[7], p[8])
        times[name] = _time_us(lambda: lib.cf_kv_attn_fused_async(*head, C.c_void_p(fused.data_ptr()), *tail), 5)
        outs[name] = fused.cpu().numpy()
        print(f"cf_kv_attn_fused_async, {seq} tokens x {nq} queries, window {window}: {name:17s} {times[name]:9.1f} us")
    assert np.allclose(outs["this library"], outs["reference kernel"], rtol=1e-5, atol=1e-6)
    assert times["this library"] <= times["reference kernel"]


def test_paged_attention_entry_can_be_captured_in_a_cuda_graph(native, oracle):
    """The split-KV form of cf_kv_paged_attention_async hands out slots guarded by events; under stream capture the call
    keeps to the single launch, so that a caller's CUDA graph still captures it, and replays give the eager result."""
    import torch
    hq, hkv, d, page, npages = 32, 8, 128, 128, 8
    rng = np.random.default_rng(4)
    made = _fixture_pages(oracle, rng, hkv, d, [page] * npages, 8)
    if made is None:
        pytest.skip("needs oracle/_ref (the reference's fixture encoder)")
    pages, keep, dk, dv = made
    q = rng.standard_normal((1, hq, d)).astype(np.float32)
    arr = (DevicePage * len(pages))(*pages)
    d_pages, d_q = _dev(np.frombuffer(bytes(arr), np.uint8)), _dev(q)
    desc = PagedAttentionDesc()
    desc.struct_size, desc.abi_version = C.sizeof(desc), 0
    desc.pages, desc.page_count = d_pages.data_ptr(), len(pages)
    desc.kv_head_count, desc.query_head_count, desc.gqa_group_size = hkv, hq, hq // hkv
    desc.queries, desc.query_token_begin, desc.query_count = d_q.data_ptr(), page * npages - 1, 1
    desc.head_dim, desc.causal_window, desc.softmax_scale = d, 0, 1.0 / np.sqrt(d)
    lib = native.lib()
    eager = torch.zeros((1, hq, d), dtype=torch.float32, device="cuda")
    desc.output = eager.data_ptr()
    assert lib.cf_kv_paged_attention_async(C.byref(desc), None) == 0          # split-KV, events
    torch.cuda.synchronize()
    captured = torch.zeros_like(eager)
    desc.output = captured.data_ptr()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph.capture_begin()
        rc = lib.cf_kv_paged_attention_async(C.byref(desc), C.c_void_p(side.cuda_stream))
        graph.capture_end()
    assert rc == 0
    torch.cuda.current_stream().wait_stream(side)
    assert float(captured.abs().max()) == 0.0                                   # captured, not run
    graph.replay()
    torch.cuda.synchronize()
    assert float((captured - eager).abs().max()) <= 1e-6 and float(eager.abs().max()) > 0
