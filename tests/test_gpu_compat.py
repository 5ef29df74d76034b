"""GPU tests of the reference-ABI entry points (compat_kv.h, compat_adapter.h), modelled on the reference's own GPU
tests: tests/paged_kv_cuda_correctness.cu, tests/cache_roundtrip_attention.cu, tests/adapter_attention_test.cu.
Where oracle/_ref holds the reference's CUDA sources compiled for sm_100a, the reference kernels run on the same
inputs and must agree."""
import ctypes as C

import numpy as np
import pytest

from compat_types import DevicePage, LlamaKvOptions, LlamaKvStats, PagedAttentionDesc
from helpers import hist_of, laplace_codes

pytestmark = pytest.mark.gpu


def _dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _softmax_attention(k, v, q, positions, first_tokens, scale, group):
    """fp64 softmax attention over dense rows: k, v [Hkv][T][D], q [Q][Hq][D] (the CPU check of
    tests/paged_kv_cuda_correctness.cu:90-118)."""
    nq, hq, d = q.shape
    out = np.zeros((nq, hq, d))
    for i in range(nq):
        for h in range(hq):
            kv = h // group
            lo, hi = first_tokens[i], positions[i] + 1
            s = (k[kv, lo:hi].astype(np.float64) @ q[i, h].astype(np.float64)) * scale
            w = np.exp(s - s.max())
            out[i, h] = (w[:, None] * v[kv, lo:hi]).sum(0) / w.sum()
    return out


def test_rans_decode_entry_matches_oracle_and_reference_kernel(native, oracle):
    """cf_rans_decode_async on a flat block-rANS stream (layout of tools/export_rans.py:13-17) written by the oracle's
    encoder: equals the source symbols, and equals what the reference's own cf_rans_decode_async kernel returns."""
    import torch
    rng = np.random.default_rng(8)
    # block 64 with more than 64 blocks takes the lane-per-block decoder for its whole groups of 64 blocks and the
    # reference-shaped kernel for the rest; 64 * 64 + 1 symbols leave exactly one symbol to the latter
    for block, n, b in [(64, 100000, 12.0), (1024, 70001, 0.6), (100, 5000, 40.0), (64, 1 << 20, 3.0), (64, 64 * 64 + 1, 0.05),
                        (64, 64 * 65, 25.0), (64, 4096, 12.0)]:
        sym = (laplace_codes(rng, n, b).astype(np.int16) + 128).astype(np.uint8)
        cb = oracle.codebook_from_hist(hist_of(sym))
        data, off, st = oracle.rans_encode(sym, block, cb)
        args = [_dev(np.concatenate([data, np.zeros(8, np.uint8)])), _dev(off), _dev(st), _dev(cb.np("slot2sym")),
                _dev(cb.np("freq")), _dev(cb.np("cum"))]
        outs = []
        libs = [native.lib()] + ([oracle.ref_cuda()] if oracle.ref_cuda() is not None else [])
        for lib in libs:
            out = torch.full((n,), -1, dtype=torch.int32, device="cuda")
            rc = lib.cf_rans_decode_async(*[C.c_void_p(t.data_ptr()) for t in args], C.c_int(block), C.c_int(n),
                                          C.c_void_p(out.data_ptr()), None)
            assert rc == 0
            torch.cuda.synchronize()
            outs.append(out.cpu().numpy())
        assert np.array_equal(outs[0], sym.astype(np.int32))
        for o in outs[1:]:
            assert np.array_equal(o, outs[0])
    assert native.lib().cf_rans_decode_async(None, None, None, None, None, None, 64, 10, None, None) == 1


def _fixture_pages(oracle, rng, hkv, d, page_sizes, bits):
    """Pages encoded by the reference's own gpu_fixture encoder (through oracle/_ref) or None when it is absent."""
    ref = oracle.ref_cpu()
    if ref is None:
        return None
    pages, keep = [], []
    begin = 0
    dense_k = np.zeros((hkv, sum(page_sizes), d), np.float32)
    dense_v = np.zeros_like(dense_k)
    for tokens in page_sizes:
        for h in range(hkv):
            n = tokens * d
            k = rng.standard_normal(n).astype(np.float32)
            v = rng.standard_normal(n).astype(np.float32)
            words = (n * bits + 31) // 32
            nb = (n + 63) // 64
            kw, vw = np.zeros(words + 1, np.uint32), np.zeros(words + 1, np.uint32)
            ko, vo = np.zeros(nb, np.int32), np.zeros(nb, np.int32)
            lut = np.zeros(1 << bits, np.int32)
            ks, vs = np.zeros(d, np.float32), np.zeros(tokens, np.float32)
            dk, dv = np.zeros(n, np.float32), np.zeros(n, np.float32)
            p = lambda a: a.ctypes.data_as(C.c_void_p)
            assert ref.ref_fixture_encode(p(k), p(v), C.c_uint32(begin), C.c_uint32(tokens), C.c_uint32(d), C.c_uint32(h),
                                          C.c_uint32(64), C.c_uint32(bits), p(kw), p(ko), p(vw), p(vo), p(lut), p(ks), p(vs),
                                          p(dk), p(dv), None) == 0
            dense_k[h, begin:begin + tokens] = dk.reshape(tokens, d)
            dense_v[h, begin:begin + tokens] = dv.reshape(tokens, d)
            t = [_dev(x) for x in (kw, ko, lut, ks, vw, vo, lut, vs)]
            keep.append(t)
            pg = DevicePage()
            (pg.k_words, pg.k_block_offsets, pg.k_lut, pg.k_scales, pg.v_words, pg.v_block_offsets, pg.v_lut,
             pg.v_scales) = [x.data_ptr() for x in t]
            pg.token_begin, pg.token_count, pg.head_dim, pg.block_size = begin, tokens, d, 64
            pg.k_max_code_length = pg.v_max_code_length = bits
            pg.zero_point, pg.kv_head, pg.fixed_code_length = 1 << (bits - 1), h, bits
            pages.append(pg)
        begin += tokens
    return pages, keep, dense_k, dense_v


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("shape", [(14, 2, 64), (8, 8, 128), (4, 2, 32), (6, 2, 96)], ids=str)
def test_reference_descriptor_attention(native, oracle, bits, shape):
    """cf_kv_paged_attention_async over the reference's own fixed-width pages + fp32 tail, several query rows with a
    causal window; bar of the reference's GPU tests: max abs error <= 2e-4 against fp32/fp64 softmax over the
    dequantised values. The reference's kernel (when built) must agree too."""
    import torch
    hq, hkv, d = shape
    rng = np.random.default_rng(9001)
    made = _fixture_pages(oracle, rng, hkv, d, [32, 32, 5], bits)
    if made is None:
        pytest.skip("needs oracle/_ref (the reference's fixture encoder)")
    pages, keep, dense_k, dense_v = made
    sealed, tail, nq, window = 69, 6, 3, 50
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
    desc.head_dim, desc.causal_window, desc.softmax_scale = d, window, 1.0 / np.sqrt(d)
    k_all = np.concatenate([dense_k, tk.transpose(1, 0, 2)], axis=1)
    v_all = np.concatenate([dense_v, tv.transpose(1, 0, 2)], axis=1)
    pos = [sealed + tail - nq + i for i in range(nq)]
    want = _softmax_attention(k_all, v_all, q, pos, [max(0, p + 1 - window) for p in pos], 1.0 / np.sqrt(d), hq // hkv)
    results = []
    libs = [native.lib()] + ([oracle.ref_cuda()] if oracle.ref_cuda() is not None else [])
    for lib in libs:
        out = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda")
        desc.output = out.data_ptr()
        assert lib.cf_kv_validate_paged_attention_desc(C.byref(desc)) == 0
        assert lib.cf_kv_paged_attention_async(C.byref(desc), None) == 0
        torch.cuda.synchronize()
        results.append(out.cpu().numpy())
    assert np.abs(results[0] - want).max() <= 2e-4
    for r in results[1:]:
        assert np.abs(r - results[0]).max() <= 2e-4
    desc.gqa_group_size += 1
    assert native.lib().cf_kv_paged_attention_async(C.byref(desc), None) == 1     # tests/paged_kv_cuda_seam.cu:8-46


def test_reference_descriptor_attention_variable_length_pages(native, oracle):
    """Variable-length Huffman pages (fixed_code_length 0) through the reference descriptor: words, block bit offsets
    and int32 LUT written by the oracle's encoder; checked against fp64 softmax over the dequantised values."""
    import torch
    rng = np.random.default_rng(12)
    hq, hkv, d, tokens = 8, 2, 128, 40
    pages, keep = [], []
    dense_k = np.zeros((hkv, tokens, d), np.float32)
    dense_v = np.zeros_like(dense_k)
    for h in range(hkv):
        ksym = (laplace_codes(rng, tokens * d, 9.0).astype(np.int16) + 128).astype(np.uint8)
        vsym = (laplace_codes(rng, tokens * d, 5.0).astype(np.int16) + 128).astype(np.uint8)
        kcb, vcb = oracle.codebook_from_hist(hist_of(ksym)), oracle.codebook_from_hist(hist_of(vsym))
        kw, ko = oracle.huff_encode(ksym, 64, kcb)
        vw, vo = oracle.huff_encode(vsym, 64, vcb)
        ks = rng.uniform(0.005, 0.02, d).astype(np.float32)
        vs = rng.uniform(0.005, 0.02, tokens).astype(np.float32)
        dense_k[h] = (ksym.reshape(tokens, d).astype(np.float32) - 128) * ks[None, :]
        dense_v[h] = (vsym.reshape(tokens, d).astype(np.float32) - 128) * vs[:, None]
        t = [_dev(x) for x in (kw, ko, kcb.np("lut"), ks, vw, vo, vcb.np("lut"), vs)]
        keep.append(t)
        pg = DevicePage()
        (pg.k_words, pg.k_block_offsets, pg.k_lut, pg.k_scales, pg.v_words, pg.v_block_offsets, pg.v_lut,
         pg.v_scales) = [x.data_ptr() for x in t]
        pg.token_begin, pg.token_count, pg.head_dim, pg.block_size = 0, tokens, d, 64
        pg.k_max_code_length = pg.v_max_code_length = 12
        pg.zero_point, pg.kv_head, pg.fixed_code_length = 128, h, 0
        pages.append(pg)
    q = rng.standard_normal((1, hq, d)).astype(np.float32)
    arr = (DevicePage * len(pages))(*pages)
    d_pages, d_q = _dev(np.frombuffer(bytes(arr), np.uint8)), _dev(q)
    out = torch.zeros((1, hq, d), dtype=torch.float32, device="cuda")
    desc = PagedAttentionDesc()
    desc.struct_size, desc.abi_version = C.sizeof(desc), 0
    desc.pages, desc.page_count = d_pages.data_ptr(), len(pages)
    desc.kv_head_count, desc.query_head_count, desc.gqa_group_size = hkv, hq, hq // hkv
    desc.queries, desc.output, desc.query_token_begin, desc.query_count = d_q.data_ptr(), out.data_ptr(), tokens - 1, 1
    desc.head_dim, desc.causal_window, desc.softmax_scale = d, 0, 1.0 / np.sqrt(d)
    assert native.lib().cf_kv_paged_attention_async(C.byref(desc), None) == 0
    torch.cuda.synchronize()
    want = _softmax_attention(dense_k, dense_v, q, [tokens - 1], [0], 1.0 / np.sqrt(d), hq // hkv)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-4


@pytest.mark.parametrize("head_dim", [32, 64, 96, 128])
@pytest.mark.parametrize("coder", ["rans", "huffman", "fixed8"])
def test_adapter_round_trip(native, oracle, head_dim, coder, monkeypatch):
    """The sweep of the reference's tests/adapter_attention_test.cu:22-112: 70 tokens = 2 sealed pages of 32 + 6 active,
    GQA 14Q/2KV, N(0,1) inputs, host append per (layer, kv head), device fp32 attention. Expected values: fp64 softmax
    over what this library's quantiser stores (int8 per-stream scale; the oracle's quantiser) plus the raw tail."""
    import torch
    monkeypatch.setenv("CHROMOFOLD_B200_CODER", coder)
    lib = native.lib()
    lib.cf_llama_kv_create.restype = C.c_void_p
    lib.cf_llama_kv_last_error.restype = C.c_char_p
    hq, hkv, page, tokens, layers = 14, 2, 32, 70, 2
    o = LlamaKvOptions()
    o.struct_size, o.backend = C.sizeof(o), 1
    o.layer_count, o.kv_head_count, o.query_head_count, o.head_dim, o.page_size, o.gqa_group_size, o.kv_bits = layers, hkv, hq, head_dim, page, hq // hkv, 8
    a = C.c_void_p(lib.cf_llama_kv_create(C.byref(o)))
    assert a.value
    rng = np.random.default_rng(9001)
    k = rng.standard_normal((layers, hkv, tokens, head_dim)).astype(np.float32)
    v = rng.standard_normal((layers, hkv, tokens, head_dim)).astype(np.float32)
    p = lambda x: np.ascontiguousarray(x).ctypes.data_as(C.c_void_p)
    for layer in range(layers):
        for begin, count in [(0, 50), (50, 20)]:                  # two appends per head, the first spans a page boundary
            for h in range(hkv):
                assert lib.cf_llama_kv_append(a, layer, h, begin, p(k[layer, h, begin:begin + count]),
                                              p(v[layer, h, begin:begin + count]), count, None) == 0, lib.cf_llama_kv_last_error(a)
    assert lib.cf_llama_kv_append(a, 0, 0, 99, p(k[0, 0, :1]), p(v[0, 0, :1]), 1, None) == -1
    assert b"contiguous" in lib.cf_llama_kv_last_error(a)
    st = LlamaKvStats()
    assert lib.cf_llama_kv_get_stats(a, C.byref(st)) == 0
    assert st.appended_tokens == layers * hkv * tokens and st.sealed_pages == layers * hkv * 2
    assert st.sealed_tokens == layers * hkv * 64 and st.active_tokens == layers * hkv * 6
    assert 0 < st.compressed_bytes < layers * hkv * 64 * head_dim * 2 * 2      # smaller than fp16
    # expected: tiles of T tokens quantised per stream: T = 16 at these head_dims (the record geometry of the
    # lane-per-block kernels), else the largest divisor of the page with T * head_dim <= 4096
    tile = 16
    deq_k, deq_v = k.copy(), v.copy()
    for layer in range(layers):
        for h in range(hkv):
            for t0 in range(0, 64, tile):
                for src, dst in ((k, deq_k), (v, deq_v)):
                    rc, bits, codes = oracle.quantize_stream(src[layer, h, t0:t0 + tile])
                    scale = np.array([bits], np.uint16).view(np.float16)[0].astype(np.float32)
                    dst[layer, h, t0:t0 + tile] = codes.reshape(tile, head_dim).astype(np.float32) * scale
    nq, window = 3, 40
    q = rng.standard_normal((nq, hq, head_dim)).astype(np.float32)
    pos = [tokens - nq + i for i in range(nq)]
    d_q = _dev(q)
    for layer in range(layers):
        out = torch.zeros((nq, hq, head_dim), dtype=torch.float32, device="cuda")
        rc = lib.cf_llama_kv_attention(a, layer, C.c_void_p(d_q.data_ptr()), C.c_void_p(out.data_ptr()), nq, hq, hq // hkv,
                                       tokens - nq, C.c_float(1.0 / np.sqrt(head_dim)), window, None)
        assert rc == 0, lib.cf_llama_kv_last_error(a)
        torch.cuda.synchronize()
        want = _softmax_attention(deq_k[layer], deq_v[layer], q, pos, [max(0, x + 1 - window) for x in pos],
                                  1.0 / np.sqrt(head_dim), hq // hkv)
        assert np.abs(out.cpu().numpy() - want).max() <= 2e-4
        host_out = np.zeros((nq, hq, head_dim), np.float32)
        assert lib.cf_llama_kv_attention_host(a, layer, p(q), p(host_out), nq, hq, hq // hkv, tokens - nq,
                                              C.c_float(1.0 / np.sqrt(head_dim)), window, None) == 0
        assert np.abs(host_out - want).max() <= 2e-4
    # flush seals the partial tail; the answer for the last position does not change beyond quantisation of 6 rows
    assert lib.cf_llama_kv_flush(a, None) == 0
    assert lib.cf_llama_kv_get_stats(a, C.byref(st)) == 0 and st.active_tokens == 0 and st.sealed_pages == layers * hkv * 3
    assert lib.cf_llama_kv_seq_cp(a, 0, 1) == -1 and lib.cf_llama_kv_seq_cp(a, 0, 0) == 0
    assert lib.cf_llama_kv_seq_shift(a, 0, 0) == 0 and lib.cf_llama_kv_seq_shift(a, 0, 1) == -1
    assert lib.cf_llama_kv_seq_rm(a, 1) == -1 and lib.cf_llama_kv_seq_rm(a, 0) == 0
    assert lib.cf_llama_kv_get_stats(a, C.byref(st)) == 0 and st.appended_tokens == 0 and st.sealed_pages == 0
    assert lib.cf_llama_kv_append(a, 0, 0, 0, p(k[0, 0, :4]), p(v[0, 0, :4]), 4, None) == 0      # usable after clear
    lib.cf_llama_kv_destroy(a)


def _read_device(ptr, count, dtype):
    """`count` elements of raw device memory (not a torch tensor) to the host."""
    from cuda.bindings import runtime as cudart
    out = np.zeros(count, dtype)
    err, = cudart.cudaMemcpy(out.ctypes.data, ptr, out.nbytes, cudart.cudaMemcpyKind.cudaMemcpyDeviceToHost)
    assert int(err) == 0
    return out


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("head_dim", [64, 128])
def test_adapter_default_pages_are_the_references_own(native, oracle, bits, head_dim, monkeypatch):
    """Without CHROMOFOLD_B200_CODER the adapter stores what the reference's adapter stores: kv_bits picks int4 / int8,
    K quantised per channel and V per token (gpu_fixture::encode_int{4,8}_page). Every page the GPU quantiser made is
    compared bit for bit — packed words, fp32 scales, block offsets — with the reference's own encoder (oracle/_ref) on
    the same rows, and attention is compared with a double-precision softmax over the reference's dequantised values
    plus the raw tail at the reference's 2e-4."""
    import torch
    ref = oracle.ref_cpu()
    if ref is None:
        pytest.skip("the reference's encoder was not built (oracle/_ref)")
    monkeypatch.delenv("CHROMOFOLD_B200_CODER", raising=False)
    lib = native.lib()
    lib.cf_llama_kv_create.restype = C.c_void_p
    lib.cf_llama_kv_last_error.restype = C.c_char_p
    hq, hkv, page, tokens, layers = 14, 2, 32, 70, 2
    o = LlamaKvOptions()
    o.struct_size, o.backend = C.sizeof(o), 1
    o.layer_count, o.kv_head_count, o.query_head_count, o.head_dim, o.page_size, o.gqa_group_size = layers, hkv, hq, head_dim, page, hq // hkv
    o.kv_bits = bits if bits == 8 else 0                 # anything but 8 means int4 in the reference
    a = C.c_void_p(lib.cf_llama_kv_create(C.byref(o)))
    assert a.value
    rng = np.random.default_rng(9100 + bits)
    k = rng.standard_normal((layers, hkv, tokens, head_dim)).astype(np.float32)
    v = rng.standard_normal((layers, hkv, tokens, head_dim)).astype(np.float32)
    k[0, 0, 40:64, 3] = 0.0                              # an all-zero channel of a page: its scale must be 1
    p = lambda x: np.ascontiguousarray(x).ctypes.data_as(C.c_void_p)
    for layer in range(layers):
        for begin, count in [(0, 50), (50, 20)]:
            for h in range(hkv):
                assert lib.cf_llama_kv_append(a, layer, h, begin, p(k[layer, h, begin:begin + count]),
                                              p(v[layer, h, begin:begin + count]), count, None) == 0, lib.cf_llama_kv_last_error(a)
    st = LlamaKvStats()
    assert lib.cf_llama_kv_get_stats(a, C.byref(st)) == 0
    assert st.sealed_pages == layers * hkv * 2 and st.active_tokens == layers * hkv * 6
    deq_k, deq_v = k.copy(), v.copy()
    n = page * head_dim
    words, nb = (n * bits + 31) // 32, (n + 63) // 64
    seen = set()
    for layer in range(layers):
        for index in range(hkv * 2):
            pg = DevicePage()
            assert lib.cf_b200_llama_kv_reference_page(a, layer, index, C.byref(pg)) == 0
            h, begin = pg.kv_head, pg.token_begin
            seen.add((layer, h, begin))
            assert (pg.token_count, pg.head_dim, pg.block_size, pg.fixed_code_length, pg.zero_point) == (page, head_dim, 64, bits, 1 << (bits - 1))
            kw, vw = np.zeros(words + 1, np.uint32), np.zeros(words + 1, np.uint32)
            ko, vo = np.zeros(nb, np.int32), np.zeros(nb, np.int32)
            lut = np.zeros(1 << bits, np.int32)
            ks, vs = np.zeros(head_dim, np.float32), np.zeros(page, np.float32)
            dk, dv = np.zeros(n, np.float32), np.zeros(n, np.float32)
            rows_k, rows_v = k[layer, h, begin:begin + page].ravel(), v[layer, h, begin:begin + page].ravel()
            assert ref.ref_fixture_encode(p(rows_k), p(rows_v), C.c_uint32(begin), C.c_uint32(page), C.c_uint32(head_dim), C.c_uint32(h),
                                          C.c_uint32(64), C.c_uint32(bits), p(kw), p(ko), p(vw), p(vo), p(lut), p(ks), p(vs),
                                          p(dk), p(dv), None) == 0
            assert np.array_equal(_read_device(pg.k_words, words, np.uint32), kw[:words])
            assert np.array_equal(_read_device(pg.v_words, words, np.uint32), vw[:words])
            assert np.array_equal(_read_device(pg.k_scales, head_dim, np.float32).view(np.uint32), ks.view(np.uint32))
            assert np.array_equal(_read_device(pg.v_scales, page, np.float32).view(np.uint32), vs.view(np.uint32))
            assert np.array_equal(_read_device(pg.k_block_offsets, nb, np.int32), ko)
            assert np.array_equal(_read_device(pg.k_lut, 1 << bits, np.int32), lut)
            deq_k[layer, h, begin:begin + page] = dk.reshape(page, head_dim)
            deq_v[layer, h, begin:begin + page] = dv.reshape(page, head_dim)
    assert len(seen) == layers * hkv * 2
    assert lib.cf_b200_llama_kv_reference_page(a, 0, hkv * 2, C.byref(DevicePage())) == -1
    nq, window = 3, 40
    q = rng.standard_normal((nq, hq, head_dim)).astype(np.float32)
    pos = [tokens - nq + i for i in range(nq)]
    d_q = _dev(q)
    for layer in range(layers):
        out = torch.zeros((nq, hq, head_dim), dtype=torch.float32, device="cuda")
        assert lib.cf_llama_kv_attention(a, layer, C.c_void_p(d_q.data_ptr()), C.c_void_p(out.data_ptr()), nq, hq, hq // hkv,
                                         tokens - nq, C.c_float(1.0 / np.sqrt(head_dim)), window, None) == 0, lib.cf_llama_kv_last_error(a)
        torch.cuda.synchronize()
        want = _softmax_attention(deq_k[layer], deq_v[layer], q, pos, [max(0, x + 1 - window) for x in pos], 1.0 / np.sqrt(head_dim), hq // hkv)
        assert np.abs(out.cpu().numpy() - want).max() <= 2e-4
    # a non-finite row is refused as the reference's quantiser refuses it (kv_gpu_fixture.cpp:13)
    bad = np.full((26, head_dim), np.nan, np.float32)
    assert lib.cf_llama_kv_append(a, 0, 0, tokens, p(bad), p(bad), 26, None) == -1
    assert b"invalid quantization input" in lib.cf_llama_kv_last_error(a)
    # flush makes a short page of the six active rows, and the cache keeps growing after it, as the reference's does
    b = C.c_void_p(lib.cf_llama_kv_create(C.byref(o)))
    for h in range(hkv):
        assert lib.cf_llama_kv_append(b, 0, h, 0, p(k[0, h, :38]), p(v[0, h, :38]), 38, None) == 0
    assert lib.cf_llama_kv_flush(b, None) == 0
    for h in range(hkv):
        assert lib.cf_llama_kv_append(b, 0, h, 38, p(k[0, h, 38:45]), p(v[0, h, 38:45]), 7, None) == 0, lib.cf_llama_kv_last_error(b)
    assert lib.cf_llama_kv_get_stats(b, C.byref(st)) == 0 and st.sealed_pages == hkv * 2 and st.active_tokens == hkv * 7
    lib.cf_llama_kv_destroy(a)
    lib.cf_llama_kv_destroy(b)


@pytest.mark.parametrize("shape", [(64, 32, 64, 16, 64), (300, 128, 40, 512, 64), (97, 80, 97, 33, 100)], ids=str)
def test_flat_fused_and_dense_attention(native, oracle, shape):
    """cf_kv_attn_fused_async / cf_kv_attn_dense_async (include/chromofold/chromofold.h:81-98) on block-Huffman K / V
    with per-channel K and per-token V scales: fused == dense bit for bit (src/cuda/fused_kv_attention.cu:1-8), both
    match fp64 softmax attention, and match the reference's own kernels where oracle/_ref holds them."""
    import torch
    seq, dim, nq, window, block = shape
    rng = np.random.default_rng(seq * 7 + dim)
    ksym = (laplace_codes(rng, seq * dim, 9.0).astype(np.int16) + 128).astype(np.uint8)
    vsym = (laplace_codes(rng, seq * dim, 14.0).astype(np.int16) + 128).astype(np.uint8)
    kcb, vcb = oracle.codebook_from_hist(hist_of(ksym)), oracle.codebook_from_hist(hist_of(vsym))
    kw, kb = oracle.huff_encode(ksym, block, kcb)
    vw, vb = oracle.huff_encode(vsym, block, vcb)
    kscale = rng.uniform(0.005, 0.02, dim).astype(np.float32)
    vscale = rng.uniform(0.005, 0.02, seq).astype(np.float32)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    sscale = 1.0 / np.sqrt(dim)
    kd = (ksym.astype(np.float32).reshape(seq, dim) - 128.0) * kscale[None, :]
    vd = (vsym.astype(np.float32).reshape(seq, dim) - 128.0) * vscale[:, None]
    positions = np.arange(nq)
    firsts = np.maximum(0, positions - window + 1)
    expect = _softmax_attention(kd[None], vd[None], q[:, None, :], positions, firsts, sscale, 1)[:, 0]

    pad = np.zeros(2, np.uint32)
    dev = [_dev(np.concatenate([kw, pad])), _dev(kb), _dev(kcb.np("lut")), _dev(np.concatenate([vw, pad])), _dev(vb),
           _dev(vcb.np("lut")), _dev(kscale), _dev(vscale), _dev(q)]
    p = [C.c_void_p(t.data_ptr()) for t in dev]
    libs = [native.lib()] + ([oracle.ref_cuda()] if oracle.ref_cuda() is not None else [])
    results = []
    for lib in libs:
        fused = torch.zeros((nq, dim), dtype=torch.float32, device="cuda")
        dense = torch.zeros_like(fused)
        kdd = torch.zeros((seq, dim), dtype=torch.float32, device="cuda")
        vdd = torch.zeros_like(kdd)
        tail = (C.c_int(seq), C.c_int(dim), C.c_int(nq), C.c_int(window), C.c_int(block), C.c_int(128), C.c_float(sscale),
                None)
        head = (p[0], p[1], p[2], C.c_int(12), p[3], p[4], p[5], C.c_int(12), p[6], p[7], p[8])
        assert lib.cf_kv_attn_fused_async(*head, C.c_void_p(fused.data_ptr()), *tail) == 0
        assert lib.cf_kv_attn_dense_async(*head, C.c_void_p(kdd.data_ptr()), C.c_void_p(vdd.data_ptr()),
                                          C.c_void_p(dense.data_ptr()), *tail) == 0
        torch.cuda.synchronize()
        assert torch.equal(fused, dense)
        assert np.array_equal(kdd.cpu().numpy(), kd) and np.array_equal(vdd.cpu().numpy(), vd)
        results.append(fused.cpu().numpy())
        assert np.allclose(results[-1], expect, rtol=1e-4, atol=1e-5)
    for r in results[1:]:
        assert np.allclose(r, results[0], rtol=1e-5, atol=1e-6)

    mine = native.lib()
    out = torch.zeros((nq, dim), dtype=torch.float32, device="cuda")
    head = (p[0], p[1], p[2], C.c_int(12), p[3], p[4], p[5], C.c_int(12), p[6], p[7], p[8], C.c_void_p(out.data_ptr()))

    def call(seq_=seq, dim_=dim, nq_=nq, window_=window, block_=block, scale_=sscale, head_=head):
        return mine.cf_kv_attn_fused_async(*head_, C.c_int(seq_), C.c_int(dim_), C.c_int(nq_), C.c_int(window_),
                                           C.c_int(block_), C.c_int(128), C.c_float(scale_), None)
    assert call(nq_=0) == 0
    assert call(nq_=seq + 1) == 1 and call(window_=0) == 1 and call(block_=0) == 1 and call(scale_=float("nan")) == 1
    assert call(head_=(None,) + head[1:]) == 1
    assert call(dim_=129) == 2 and call(window_=513) == 2


def test_adapter_reserves_its_page_memory_up_front_when_asked(native, monkeypatch):
    """CHROMOFOLD_B200_RESERVE_TOKENS: the adapter takes its page chunks and descriptor arrays at create; appending that
    many tokens then allocates nothing more (the reserved byte count does not move). Without it page memory starts
    empty and grows with the first sealed page."""
    lib = native.lib()
    lib.cf_llama_kv_create.restype = C.c_void_p
    lib.cf_b200_llama_kv_reserved_bytes.restype = C.c_uint64
    monkeypatch.delenv("CHROMOFOLD_B200_CODER", raising=False)
    hq, hkv, page, layers, d, tokens = 8, 2, 32, 3, 128, 8192
    o = LlamaKvOptions()
    o.struct_size, o.backend = C.sizeof(o), 1
    o.layer_count, o.kv_head_count, o.query_head_count, o.head_dim, o.page_size, o.gqa_group_size = layers, hkv, hq, d, page, hq // hkv
    o.kv_bits = 8
    plain = C.c_void_p(lib.cf_llama_kv_create(C.byref(o)))
    assert plain.value and lib.cf_b200_llama_kv_reserved_bytes(plain) == 0
    lib.cf_llama_kv_destroy(plain)
    monkeypatch.setenv("CHROMOFOLD_B200_RESERVE_TOKENS", str(tokens))
    a = C.c_void_p(lib.cf_llama_kv_create(C.byref(o)))
    assert a.value
    reserved = lib.cf_b200_llama_kv_reserved_bytes(a)
    # int8 page of 32 x 128: 2 x 4096 B of words + scales + offsets, rounded to 256 B; 256 pages per layer and head
    assert reserved >= layers * hkv * (tokens // page) * 2 * 4096
    rng = np.random.default_rng(77)
    rows = rng.standard_normal((512, d)).astype(np.float32)
    p = lambda x: np.ascontiguousarray(x).ctypes.data_as(C.c_void_p)
    for begin in range(0, tokens, 512):
        for layer in range(layers):
            for h in range(hkv):
                assert lib.cf_llama_kv_append(a, layer, h, begin, p(rows), p(rows), 512, None) == 0
    st = LlamaKvStats()
    assert lib.cf_llama_kv_get_stats(a, C.byref(st)) == 0 and st.sealed_pages == layers * hkv * (tokens // page)
    assert lib.cf_b200_llama_kv_reserved_bytes(a) == reserved
    lib.cf_llama_kv_destroy(a)
