"""Codec round trips of the oracle: decode(encode(x)) == x through the restated reference decoders, record layout,
quantiser properties, edge cases."""
import numpy as np
import pytest

from helpers import geometric_codes, hist_for_coder, hist_of, laplace_codes


def _streams(rng):
    yield "laplace12", laplace_codes(rng, 6000, 12.0)
    yield "laplace4", laplace_codes(rng, 6000, 4.0)
    for p in (0.05, 0.1, 0.2, 0.4, 0.7):
        yield f"geom{p}", geometric_codes(rng, 6000, p)
    yield "constant", np.zeros(6000, np.int8)
    yield "uniform", rng.integers(-128, 128, 6000).astype(np.int8)
    yield "two_point", rng.choice(np.array([-128, 127], np.int8), 6000)


@pytest.mark.parametrize("block", [16, 64, 100, 1024])
def test_rans_and_huffman_round_trip(oracle, block):
    rng = np.random.default_rng(1)
    for name, codes in _streams(rng):
        sym = (codes.astype(np.int16) + 128).astype(np.uint8)
        for hist in (hist_of(sym), hist_of(sym[:50]), np.zeros(256, np.uint64)):  # matched, mismatched, empty model
            cb = oracle.codebook_from_hist(hist)
            freq = cb.np("freq")
            assert freq.sum() == 4096 and freq.min() >= 1 and freq.max() <= 3841
            for n in (sym.size, 1, block, block + 1, 777):
                data, off, st = oracle.rans_encode(sym[:n], block, cb)
                assert np.array_equal(oracle.rans_decode(data, off, st, cb, block, n), sym[:n]), (name, n)
                assert st.min() >= (1 << 23)
                words, boff = oracle.huff_encode(sym[:n], block, cb)
                assert np.array_equal(oracle.huff_decode(words, boff, cb, block, n), sym[:n]), (name, n)
            assert cb.np("hlen").max() <= 12 and cb.np("hlen").min() >= 1
            assert np.sum(2.0 ** -cb.np("hlen").astype(np.float64)) <= 1.0 + 1e-12


def test_rans_size_tracks_entropy(oracle):
    rng = np.random.default_rng(2)
    sym = (laplace_codes(rng, 1 << 18, 12.0).astype(np.int16) + 128).astype(np.uint8)
    hist = hist_of(sym)
    p = hist[hist > 0] / hist.sum()
    h0 = float(-(p * np.log2(p)).sum())
    cb = oracle.codebook_from_hist(hist)
    data, off, st = oracle.rans_encode(sym, 64, cb)
    bits = (data.size * 8 + st.size * 32) / sym.size
    assert h0 < bits < h0 + 0.65   # 32-bit start state per 64 symbols is 0.5 bit/symbol


@pytest.mark.parametrize("coder", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("geo", [(128, 16, 64), (64, 32, 64), (32, 16, 32), (96, 16, 128), (128, 32, 1024)])
def test_record_round_trip(oracle, coder, geo):
    d, t, block = geo
    rng = np.random.default_rng(4)
    cb = oracle.codebook_from_hist(hist_for_coder(laplace_codes(rng, 1 << 15, 6.0).astype(np.int16) + 128, coder))
    for rows in (t, 1, t - 1):
        k = (rng.standard_normal((rows, d)) * 0.3).astype(np.float16).astype(np.float32)
        v = (rng.standard_normal((rows, d)) * 2.0).astype(np.float16).astype(np.float32)
        rec, ks, vs = oracle.seal_record(k, v, rows, d, t, block, coder, 3, cb, cb)
        assert rec.size % 16 == 0 and rec.size <= 16 + 2 * ((d * t + 15) // 16 * 16)
        hdr = rec[:16].view(np.uint16)
        assert 16 * (1 + int(hdr[0]) + int(hdr[1])) == rec.size and hdr[3] == rows and hdr[6] == 3 and rec[15] == 1
        ks2, vs2 = oracle.open_record(rec, d, t, block, cb, cb)
        assert np.array_equal(ks, ks2) and np.array_equal(vs, vs2)
        # quantiser: symbol = clamp(rint(x / scale)) + 128 with scale = fp16(absmax / 127); error <= 0.51 * scale
        # (the bound the reference checks for its own sealer, tests/kv_reference_test.cpp:70-71)
        ksc = float(np.array([hdr[4]], np.uint16).view(np.float16)[0])
        kq = (ks.reshape(t, d)[:rows].astype(np.float32) - 128.0) * ksc
        assert np.max(np.abs(kq - k)) <= 0.51 * ksc
        vsc = float(np.array([hdr[5]], np.uint16).view(np.float16)[0])
        vq = (vs.reshape(d, t).T[:rows].astype(np.float32) - 128.0) * vsc   # V is stored token-minor
        assert np.max(np.abs(vq - v)) <= 0.51 * vsc
        assert np.all(ks.reshape(t, d)[rows:] == 128) and np.all(vs.reshape(d, t)[:, rows:] == 128)


def test_nibble_split_record_layout_and_size(oracle):
    """CF_B200_CODER_RANS_SPLIT4 / _HUFFMAN_SPLIT4: the part is table | raw low-nibble plane | coded pair symbols; the
    plane holds exactly the low nibbles in the documented bit positions; at Laplace(b = 12) the record is within 3 % of
    the plain coder's."""
    rng = np.random.default_rng(5)
    calib = (laplace_codes(rng, 1 << 16, 12.0).astype(np.int16) + 128).astype(np.uint8)
    codes = laplace_codes(rng, (16, 128), 12.0)
    codes[0, 0] = 127
    k = (codes.astype(np.float32) * 0.01).astype(np.float16).astype(np.float32)
    sizes = {}
    for coder in (1, 2, 3, 4):
        cb = oracle.codebook_from_hist(hist_for_coder(calib, coder))
        rec, ks, vs = oracle.seal_record(k, k, 16, 128, 16, 64, coder, 0, cb, cb)
        assert rec[4] == coder and rec[5] == coder
        sizes[coder] = rec.size
        assert np.array_equal(ks, (codes.astype(np.int16) + 128).astype(np.uint8).ravel())
        if coder in (3, 4):
            table = 192 if coder == 3 else 64
            plane = rec[16 + table:16 + table + 1024].view("<u4").reshape(8, 32)       # lo[j][block]
            for block in (0, 7, 31):
                for i in range(64):
                    shift = 8 * (i % 4) + (4 if i % 8 >= 4 else 0)
                    assert (int(plane[i // 8, block]) >> shift) & 15 == int(ks[64 * block + i]) & 15
    assert sizes[3] <= 1.03 * sizes[2] and sizes[4] <= 1.03 * sizes[1]


def test_incompressible_stream_falls_back_to_fixed_width(oracle):
    rng = np.random.default_rng(6)
    cb = oracle.codebook_from_hist(hist_of(np.full(1000, 128, np.uint8)))   # model expects zeros only
    k = rng.uniform(-1, 1, (16, 128)).astype(np.float16).astype(np.float32)
    rec, _, _ = oracle.seal_record(k, k, 16, 128, 16, 64, 2, 0, cb, cb)
    assert rec[4] == 0 and rec[5] == 0 and rec.size == 16 + 2 * 2048


def test_quantiser_rejects_non_finite_and_handles_zero(oracle):
    x = np.zeros(64, np.float32)
    rc, bits, codes = oracle.quantize_stream(x)
    assert rc == 0 and bits == 0x3C00 and not codes.any()
    x[5] = np.inf
    assert oracle.quantize_stream(x)[0] == 1
    x[5] = np.nan
    assert oracle.quantize_stream(x)[0] == 1
    assert oracle.seal_record(x.reshape(1, 64), x.reshape(1, 64), 1, 64, 16, 64, 2, 0,
                              oracle.codebook_from_hist(np.ones(256, np.uint64)),
                              oracle.codebook_from_hist(np.ones(256, np.uint64))) is None


def test_half_conversion_matches_numpy(oracle):
    rng = np.random.default_rng(9)
    x = np.concatenate([rng.standard_normal(2000) * 10.0 ** rng.integers(-9, 6, 2000), [0.0, 65504.0, 65520.0, 1e-8, 6e-8]])
    for f in x.astype(np.float32):
        want = np.array([f], np.float32).astype(np.float16)
        got = oracle.lib().orc_float_to_half(float(f))
        assert got == int(want.view(np.uint16)[0]), f
        if np.isfinite(want[0]):
            assert oracle.lib().orc_half_to_float(got) == float(want[0])
