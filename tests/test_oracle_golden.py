"""The CPU oracle against the golden vectors produced by the reference's own sources (tests/golden/make_golden.py),
and, where oracle/_ref is built, against those sources live."""
import ctypes as C
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def _names(z):
    return sorted({k.split(".")[0] for k in z.files})


def near(a, b, tol=2e-5):
    """The reference's own comparison, tests/kv_reference_test.cpp:21-23."""
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.all(np.abs(a - b) <= tol * np.maximum(1.0, np.maximum(np.abs(a), np.abs(b))))


def test_fixed_width_decode_matches_reference_fixture(oracle):
    """8-bit pages packed by the reference's gpu_fixture::encode_int8_page decode to the reference's symbols through
    the oracle's fixed-width reader (the FIXED8 part of a record is exactly such a word stream)."""
    z = np.load(os.path.join(GOLD, "fixture_pages.npz"))
    for name in _names(z):
        tokens, dim, block, bits, _ = z[f"{name}.shape"]
        if bits != 8:
            continue
        n = int(tokens * dim)
        for side in "kv":
            words = z[f"{name}.{side}_words"]
            # wrap the reference's word stream as a FIXED8 record part and open it with the oracle
            part = np.zeros((n + 15) // 16 * 16, np.uint8)
            part[:words.size * 4] = words.view(np.uint8)
            rec = np.zeros(16 + 2 * part.size, np.uint8)
            hdr = np.zeros(8, np.uint16)
            hdr[0] = hdr[1] = part.size // 16
            hdr[3] = tokens
            rec[:16] = hdr.view(np.uint8)
            rec[15] = 1
            rec[16:16 + part.size] = part
            rec[16 + part.size:] = part
            cb = oracle.codebook_from_hist(np.ones(256, np.uint64))
            ks, vs = oracle.open_record(rec, int(dim), int(tokens), int(block), cb, cb)
            assert np.array_equal(ks, z[f"{name}.{side}_symbols"])
            assert np.array_equal(vs, z[f"{name}.{side}_symbols"])
        # dequantisation rule (sym - zero_point) * scale, paged_kv_attention.cu:222
        ksym = z[f"{name}.k_symbols"].astype(np.int32).reshape(tokens, dim)
        deq = ((ksym - 128).astype(np.float32) * z[f"{name}.k_scales"][None, :]).ravel()
        assert np.array_equal(deq, z[f"{name}.dequantized_k"])


def test_huffman_streams_decode_under_the_reference_decoder(oracle):
    """Streams written by the oracle's Huffman encoder were decoded by the reference's cf_bh_decode_at when the
    golden file was made; the oracle's restated decoder must give the same symbols from the same words."""
    z = np.load(os.path.join(GOLD, "huffman_decode.npz"))
    for name in _names(z):
        words, off, lut = z[f"{name}.words"], z[f"{name}.offsets"], z[f"{name}.lut"]
        want = z[f"{name}.decoded_by_reference"]
        got = np.zeros(want.size, np.uint8)
        padded = np.concatenate([words, np.zeros(2, np.uint32)])
        oracle.lib().orc_huff_decode(_p(padded), _p(off), _p(np.ascontiguousarray(lut, np.int32)), C.c_int(12),
                                     C.c_int(64), C.c_int(want.size), _p(got))
        assert np.array_equal(got, want)
        # and symbol by symbol through the single-symbol entry
        pos = int(off[3])
        for j in range(64):
            sl = oracle.lib().orc_bh_decode_at(_p(padded), _p(np.ascontiguousarray(lut, np.int32)), C.c_int(12), C.c_int(pos))
            assert (sl & 0xFF) == want[3 * 64 + j]
            pos += sl >> 8


def test_attention_matches_reference_paged_attention(oracle):
    """reference::paged_attention over int4 pages + fp32 tails (GQA, ragged pages, window, several queries):
    replaying its dequantised rows through the oracle's dense attention gives the same output."""
    z = np.load(os.path.join(GOLD, "paged_attention.npz"))
    for name in _names(z):
        hq, hkv, d, tail, nq, qbegin, window = (int(x) for x in z[f"{name}.shape"])
        dk, dv = z[f"{name}.dequantized_k"], z[f"{name}.dequantized_v"]
        keys = np.concatenate([dk, z[f"{name}.tail_k"]], axis=1)
        values = np.concatenate([dv, z[f"{name}.tail_v"]], axis=1)
        rc, out = oracle.dense_attention(keys, values, 0, z[f"{name}.q"], qbegin, window, 1.0 / np.sqrt(np.float32(d)))
        assert rc == 0
        assert near(out, z[f"{name}.output"]), name
        assert near(out, z[f"{name}.output_reversed_pages"]), name  # page order is irrelevant


def test_online_softmax_merge_matches_reference(oracle):
    """cf_online_softmax_merge / finalize: merging the reference's own partial states with the oracle's merge
    reproduces the reference's merged state and output (scores from -1000 to 900 included)."""
    z = np.load(os.path.join(GOLD, "online_softmax.npz"))
    for name in _names(z):
        pm, ps, pw = z[f"{name}.partial_max"], z[f"{name}.partial_sum"], z[f"{name}.partial_weighted"]
        dim = pw.shape[1]
        m, s, init = C.c_double(-np.inf), C.c_double(0.0), C.c_int(0)
        w = np.zeros(dim, np.float64)
        for i in range(pm.size):
            oracle.lib().orc_online_merge(C.byref(m), C.byref(s), _p(w), C.byref(init), C.c_double(pm[i]),
                                          C.c_double(ps[i]), _p(np.ascontiguousarray(pw[i])), C.c_int(1), C.c_uint32(dim))
        assert m.value == float(z[f"{name}.merged_max"])
        assert np.isclose(s.value, float(z[f"{name}.merged_sum"]), rtol=1e-14)
        assert np.allclose(w, z[f"{name}.merged_weighted"], rtol=1e-14, atol=0)
        assert np.allclose((w / s.value).astype(np.float32), z[f"{name}.output"], atol=1e-6)


def test_oracle_against_live_reference_sources(oracle):
    """Where the reference's sources are built (oracle/_ref), run them live on fresh inputs."""
    ref = oracle.ref_cpu()
    if ref is None:
        pytest.skip("oracle/_ref not built here")
    rng = np.random.default_rng(77)
    hkv, hq, d, tokens = 2, 6, 64, 37
    k = rng.standard_normal((hkv, tokens, d)).astype(np.float32)
    v = rng.standard_normal((hkv, tokens, d)).astype(np.float32)
    q = rng.standard_normal((2, hq, d)).astype(np.float32)
    want = np.zeros((2, hq, d), np.float32)
    rc = ref.ref_paged_attention_dense(_p(k), _p(v), C.c_uint32(0), C.c_uint32(tokens), _p(q), C.c_uint32(2),
                                       C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(d), C.c_uint32(35), C.c_uint32(20),
                                       C.c_float(0.125), _p(want))
    assert rc == 0
    rc, got = oracle.dense_attention(k, v, 0, q, 35, 20, 0.125)
    assert rc == 0 and near(got, want)
    # no visible token: the reference throws (kv_reference.cpp:235), the oracle reports it
    rc = ref.ref_paged_attention_dense(_p(k), _p(v), C.c_uint32(100), C.c_uint32(tokens), _p(q), C.c_uint32(1),
                                       C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(d), C.c_uint32(5), C.c_uint32(0),
                                       C.c_float(0.125), _p(want))
    assert rc == 1
    rc, _ = oracle.dense_attention(k, v, 100, q[:1], 5, 0, 0.125)
    assert rc == 1


def test_oracle_against_live_reference_sources_on_random_inputs(oracle):
    """The same, swept: the oracle's dense attention beside reference::paged_attention on random shapes, windows and query
    positions (positions with no visible token included: both must refuse), and the oracle's block-Huffman decoder
    beside the reference's cf_bh_decode_at, bit position by bit position, on random streams."""
    ref = oracle.ref_cpu()
    if ref is None:
        pytest.skip("oracle/_ref not built here")
    from helpers import hist_of, laplace_codes
    rng = np.random.default_rng(177)
    for _ in range(150):
        hkv = int(rng.choice([1, 2, 4]))
        hq = hkv * int(rng.choice([1, 3, 4, 7]))
        d = int(rng.choice([8, 32, 64, 128]))
        tokens, begin = int(rng.integers(1, 80)), int(rng.choice([0, 0, 5, 100]))
        nq = int(rng.integers(1, 4))
        k = (rng.standard_normal((hkv, tokens, d)) * 10.0 ** rng.uniform(-2, 1)).astype(np.float32)
        v = (rng.standard_normal((hkv, tokens, d)) * 10.0 ** rng.uniform(-3, 2)).astype(np.float32)
        q = rng.standard_normal((nq, hq, d)).astype(np.float32)
        qpos = int(rng.integers(0, begin + tokens + 10))
        window = int(rng.choice([0, 0, 1, 7, 1000]))
        scale = float(rng.choice([0.125, 1.0 / np.sqrt(d)]))
        want = np.zeros((nq, hq, d), np.float32)
        rc_ref = ref.ref_paged_attention_dense(_p(k), _p(v), C.c_uint32(begin), C.c_uint32(tokens), _p(q), C.c_uint32(nq),
                                               C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(d), C.c_uint32(qpos),
                                               C.c_uint32(window), C.c_float(scale), _p(want))
        rc, got = oracle.dense_attention(k, v, begin, q, qpos, window, scale)
        assert rc == rc_ref, (rc, rc_ref, begin, tokens, qpos, window, nq)
        if rc == 0:
            assert near(got, want), (begin, tokens, qpos, window)
    for _ in range(60):
        n, block = int(rng.integers(1, 3000)), int(rng.choice([16, 64, 100, 1024]))
        sym = (laplace_codes(rng, n, float(10.0 ** rng.uniform(-0.5, 1.6))).astype(np.int16) + 128).astype(np.uint8)
        cb = oracle.codebook_from_hist(hist_of(sym) if rng.random() < 0.7 else hist_of(sym) + 1)
        words, off = oracle.huff_encode(sym, block, cb)
        assert np.array_equal(oracle.huff_decode(words, off, cb, block, n), sym)
        padded = np.concatenate([words, np.zeros(2, np.uint32)])
        lut = cb.np("lut").astype(np.int32)
        # the reference's decoder walks a block from its bit offset: entry = symbol | length << 8 (block_huffman_device.cuh)
        for b in rng.choice(off.size, min(off.size, 6), replace=False):
            pos = int(off[b])
            for i in range(int(b) * block, min((int(b) + 1) * block, n)):
                entry = ref.ref_bh_decode_at(_p(padded), _p(lut), C.c_int(12), C.c_int(pos))
                assert (entry & 0xFF) == int(sym[i]), (n, block, int(b), i)
                pos += entry >> 8
