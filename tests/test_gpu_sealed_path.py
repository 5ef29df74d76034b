"""GPU parity tests of the sealed-KV path, through the C ABI, against the CPU oracle."""
import numpy as np
import pytest

from helpers import HostCache, attention_close, hist_for_coder, hist_of, laplace_codes

pytestmark = pytest.mark.gpu

CODERS = {"fixed8": 0, "huffman": 1, "rans": 2, "rans4": 3, "huffman4": 4}   # the last two: nibble-split


def _layer(native, **kw):
    from chromofold_b200.cache import SealedKvLayer
    args = dict(kv_heads=2, query_heads=4, head_dim=128, page_tokens=16, block_size=64, coder=2, max_sequences=4,
                max_pages_per_sequence=16, max_pages=256, arena_bytes=2 << 20)
    args.update(kw)
    return SealedKvLayer(**args)


def _random_kv(rng, hkv, tokens, d, b=12.0, scale=0.01):
    k = (laplace_codes(rng, (hkv, tokens, d), b).astype(np.float32) * scale).astype(np.float16).astype(np.float32)
    v = (laplace_codes(rng, (hkv, tokens, d), b).astype(np.float32) * scale).astype(np.float16).astype(np.float32)
    return k, v


def _build(native, oracle, rng, *, hq, hkv, d, t, block, coder, contexts, tails, b=12.0, noisy_k_pages=(), **layer_kw):
    """A GPU layer and a CPU HostCache holding the same sealed pages (sealed by the ORACLE and imported).
    noisy_k_pages: (sequence, page) pairs whose K values are uniform over the code range, so that their K stream does
    not shrink and is stored fixed-width while the V stream keeps the page's coder (a mixed-coder record)."""
    import torch
    n = len(contexts)
    stride = max(1, max((c + t - 1) // t for c in contexts))
    calib = laplace_codes(rng, 1 << 16, b)
    hist = hist_for_coder(calib.astype(np.int16) + 128, coder)
    kcb = oracle.codebook_from_hist(hist)
    vcb = oracle.codebook_from_hist(hist[::-1].copy())
    layer = _layer(native, kv_heads=hkv, query_heads=hq, head_dim=d, page_tokens=t, block_size=block, coder=coder,
                   max_sequences=n, max_pages_per_sequence=stride, max_pages=n * stride + 2,
                   arena_bytes=max(1 << 16, n * stride * hkv * (2 * d * t + 64)), **layer_kw)
    layer.set_codebooks(hist, hist[::-1].copy())
    host = HostCache(hkv, d, t, block, coder, kcb, vcb)
    tail_k = np.zeros((n, hkv, t, d), np.float16)
    tail_v = np.zeros((n, hkv, t, d), np.float16)
    for s, ctx in enumerate(contexts):
        done = 0
        while done < ctx:
            tokens = min(t, ctx - done)
            k, v = _random_kv(rng, hkv, tokens, d, b)
            if (s, done // t) in noisy_k_pages:
                k = (rng.integers(-127, 128, (hkv, tokens, d)).astype(np.float32) * 0.01).astype(np.float16).astype(np.float32)
            host.seal_page(s, k, v)
            done += tokens
        if s in host.records:
            layer.import_records(s, host.records[s], host.tokens[s])
        if tails[s]:
            k, v = _random_kv(rng, hkv, tails[s], d, b)
            tail_k[s, :, :tails[s]] = k
            tail_v[s, :, :tails[s]] = v
            layer.fill_tails([s], torch.from_numpy(tail_k[s:s + 1]).cuda(), torch.from_numpy(tail_v[s:s + 1]).cuda(), tails[s])
    return layer, host, kcb, vcb, tail_k, tail_v, stride


def _oracle_attention(oracle, host, kcb, vcb, contexts, tails, tail_k, tail_v, q16, hq, stride, window=0):
    arena, offsets, table, sealed = host.flat(list(range(len(contexts))), stride)
    return oracle.sealed_decode_attention(arena, offsets, table, sealed, q16, hq, host.hkv, host.d, host.t, host.block,
                                          window, 1.0 / np.sqrt(host.d), kcb, vcb, tail_k=tail_k, tail_v=tail_v,
                                          tail_count=np.array(tails, np.uint32))


@pytest.mark.parametrize("coder", list(CODERS))
def test_gpu_decode_is_bit_exact(native, oracle, coder):
    """Codes decoded on the GPU == codes the CPU quantiser produced == codes the restated reference decoders
    recover from the same bytes."""
    rng = np.random.default_rng(11)
    contexts = [48, 16, 37]
    layer, host, kcb, vcb, *_ = _build(native, oracle, rng, hq=4, hkv=2, d=128, t=16, block=64, coder=CODERS[coder],
                                       contexts=contexts, tails=[0, 0, 0])
    pid = 1
    for s in range(len(contexts)):
        ids = list(range(pid, pid + len(host.records[s])))
        pid += len(ids)
        ks, vs = layer.decode_pages(ids)
        ks, vs = ks.cpu().numpy(), vs.cpu().numpy()
        for p in range(len(ids)):
            for h in range(2):
                want_k, want_v = host.symbols[s][p][h]
                assert np.array_equal(ks[p, h], want_k)
                assert np.array_equal(vs[p, h], want_v)
                back_k, back_v = oracle.open_record(host.records[s][p][h], 128, 16, 64, kcb, vcb)
                assert np.array_equal(back_k, want_k) and np.array_equal(back_v, want_v)
    assert layer.device_status() == 0


def _expect_dump(dump, host, oracle, kcb, vcb, sequences, first_page_of=None, block=64, d=128):
    """Every record of `sequences` (page ids in import order from 1): the dumped K and V symbols against the symbols
    the CPU quantiser produced and against what the restated reference decoders recover from the record's bytes."""
    pid, checked = 1, 0
    for s in sorted(host.records):
        for p, page in enumerate(host.records[s]):
            if s in sequences:
                for h, rec in enumerate(page):
                    want_k, want_v = host.symbols[s][p][h]
                    back_k, back_v = oracle.open_record(rec, d, 16, block, kcb, vcb)
                    assert np.array_equal(back_k, want_k) and np.array_equal(back_v, want_v)
                    assert np.array_equal(dump[pid, h, 0], want_k), ("K", s, p, h)
                    assert np.array_equal(dump[pid, h, 1], want_v), ("V", s, p, h)
                    checked += 1
            pid += 1
    return checked


@pytest.mark.parametrize("coder", list(CODERS))
def test_lane_decoders_yield_exactly_the_oracle_symbols(native, oracle, coder):
    """CF_B200_KERNEL_DECODE_DUMP: the per-lane block decoders of the attention kernel (RansLane / HuffLane / FixedLane in
    lanes_attention_kernel, the code that is timed) write out every symbol they decode; all of them must equal the CPU
    quantiser's codes and the restated reference decoders' output. Covers a ragged last page (5 tokens), a
    single-page sequence and a mixed-coder record (K fixed-width, V entropy coded)."""
    import torch
    rng = np.random.default_rng(12)
    contexts = [48, 16, 37, 160]
    layer, host, kcb, vcb, *_ = _build(native, oracle, rng, hq=4, hkv=2, d=128, t=16, block=64, coder=CODERS[coder],
                                       contexts=contexts, tails=[0, 0, 0, 0], noisy_k_pages={(3, 1), (3, 7)})
    if coder != "fixed8":   # the noisy K streams fell back to fixed width, their V streams did not
        rec = host.records[3][1][0]
        assert rec[4] == CODERS["fixed8"] and rec[5] == CODERS[coder]
    q = torch.zeros((4, 4, 128), dtype=torch.float16, device="cuda")
    dump = layer.dump_lane_decoders(q).cpu().numpy()
    assert layer.device_status() == 0
    assert _expect_dump(dump, host, oracle, kcb, vcb, {0, 1, 2, 3}) == 2 * (3 + 1 + 3 + 10)


@pytest.mark.parametrize("block", [128, 256])
@pytest.mark.parametrize("coder", list(CODERS))
def test_larger_blocks_are_decoded_exactly_and_attend_like_the_oracle(native, oracle, coder, block):
    """Blocks of 128 / 256 symbols (16 / 8 blocks per stream) run the lane-per-block kernel behind its staging step:
    the symbols the lanes hold after the tile pass equal the oracle's, symbol for symbol (ragged last page and a
    mixed-coder record included), and attention agrees with the oracle for fp16 queries in groups of four and eight
    heads and for fp32 queries."""
    import torch
    rng = np.random.default_rng(31)
    contexts, tails = [48, 16, 37, 160], [3, 0, 0, 9]
    layer, host, kcb, vcb, tail_k, tail_v, stride = _build(native, oracle, rng, hq=16, hkv=2, d=128, t=16, block=block,
                                                           coder=CODERS[coder], contexts=contexts, tails=tails,
                                                           noisy_k_pages={(3, 1), (3, 7)})
    if coder != "fixed8":
        rec = host.records[3][1][0]
        assert rec[4] == CODERS["fixed8"] and rec[5] == CODERS[coder]
    q = rng.standard_normal((4, 16, 128)).astype(np.float16)
    dump = layer.dump_lane_decoders(torch.from_numpy(q).cuda()).cpu().numpy()
    assert layer.device_status() == 0
    assert _expect_dump(dump, host, oracle, kcb, vcb, {0, 1, 2, 3}, block=block) == 2 * (3 + 1 + 3 + 10)
    want = _oracle_attention(oracle, host, kcb, vcb, contexts, tails, tail_k, tail_v, q, 16, stride)
    for qt in (torch.from_numpy(q).cuda(), torch.from_numpy(q.astype(np.float32)).cuda()):
        got = layer.attention(qt, kernel=native.KERNEL_LANES, min_pages_per_unit=2).cpu().numpy()
        assert layer.device_status() == 0
        ok, err = attention_close(got, want)
        assert ok, f"max abs error {err}"
    # groups of four heads (the register-resident query operands) and the decode-only probe
    layer4, host4, kcb4, vcb4, tk4, tv4, stride4 = _build(native, oracle, rng, hq=4, hkv=2, d=128, t=16, block=block,
                                                          coder=CODERS[coder], contexts=[80, 33], tails=[0, 5])
    q4 = rng.standard_normal((2, 4, 128)).astype(np.float16)
    want4 = _oracle_attention(oracle, host4, kcb4, vcb4, [80, 33], [0, 5], tk4, tv4, q4, 4, stride4)
    got4 = layer4.attention(torch.from_numpy(q4).cuda(), kernel=native.KERNEL_LANES).cpu().numpy()
    assert layer4.device_status() == 0
    ok, err = attention_close(got4, want4)
    assert ok, f"max abs error {err}"


@pytest.mark.parametrize("geometry", [(64, 64), (64, 128), (96, 64), (96, 128), (32, 64)], ids=lambda g: f"d{g[0]}b{g[1]}")
@pytest.mark.parametrize("coder", list(CODERS))
def test_smaller_head_dims_run_the_lane_kernel(native, oracle, coder, geometry):
    """16 x 64, 16 x 96 and 16 x 32 pages go through the staging tile of the lane-per-block kernel with smaller lane
    shares (at 16 x 96 with 64-symbol blocks the 48 blocks of a record are dealt over the 32 lanes in two rounds):
    symbols exact against the oracle, attention against the oracle for groups of four and eight heads, fp16 and fp32
    queries."""
    import torch
    d, block = geometry
    rng = np.random.default_rng(41)
    contexts, tails = [48, 16, 37, 160], [3, 0, 0, 9]
    for hq in (16, 8):
        layer, host, kcb, vcb, tail_k, tail_v, stride = _build(native, oracle, rng, hq=hq, hkv=2, d=d, t=16, block=block,
                                                               coder=CODERS[coder], contexts=contexts, tails=tails,
                                                               noisy_k_pages={(3, 1), (3, 7)})
        q = rng.standard_normal((4, hq, d)).astype(np.float16)
        if hq == 16:
            dump = layer.dump_lane_decoders(torch.from_numpy(q).cuda()).cpu().numpy()
            assert layer.device_status() == 0
            assert _expect_dump(dump, host, oracle, kcb, vcb, {0, 1, 2, 3}, block=block, d=d) == 2 * (3 + 1 + 3 + 10)
        want = _oracle_attention(oracle, host, kcb, vcb, contexts, tails, tail_k, tail_v, q, hq, stride)
        for qt in (torch.from_numpy(q).cuda(), torch.from_numpy(q.astype(np.float32)).cuda()):
            got = layer.attention(qt, kernel=native.KERNEL_LANES, min_pages_per_unit=2).cpu().numpy()
            assert layer.device_status() == 0
            ok, err = attention_close(got, want)
            assert ok, f"max abs error {err}"


@pytest.mark.parametrize("coder", list(CODERS))
def test_shared_prefix_decoders_yield_exactly_the_oracle_symbols(native, oracle, coder):
    """The same symbol-for-symbol check for the decoder warps of prefix_attention_kernel: five query rows over one
    sequence share its first eight pages (decoded by the shared-prefix kernel), the last two pages go through the
    per-entry kernel; together they must have written every record of the sequence."""
    import torch
    rng = np.random.default_rng(13)
    layer, host, kcb, vcb, *_ = _build(native, oracle, rng, hq=4, hkv=2, d=128, t=16, block=64, coder=CODERS[coder],
                                       contexts=[157], tails=[0], noisy_k_pages={(0, 2)}, workspace_bytes=4 << 20)
    before = native.lib().cf_b200_shared_prefix_launches()
    q = torch.zeros((5, 4, 128), dtype=torch.float16, device="cuda")
    positions = torch.tensor([156, 150, 140, 130, 128], dtype=torch.int32, device="cuda")
    dump = layer.dump_lane_decoders(q, slots=[0] * 5, shared_prefix_pages=8, query_positions=positions).cpu().numpy()
    assert layer.device_status() == 0
    assert native.lib().cf_b200_shared_prefix_launches() == before + 1
    assert _expect_dump(dump, host, oracle, kcb, vcb, {0}) == 2 * 10


GEOMETRIES = [
    # hq, hkv, d, t, block, contexts, tails, window
    (4, 2, 128, 16, 64, [64, 16, 40, 0], [0, 3, 5, 2], 0),
    (32, 8, 128, 16, 64, [128, 96], [7, 0], 0),
    (8, 8, 128, 16, 64, [80], [1], 0),
    (14, 2, 64, 32, 64, [96, 50], [0, 4], 0),
    (4, 4, 32, 16, 32, [33, 64], [2, 0], 0),
    (8, 2, 96, 16, 128, [48, 70], [3, 9], 0),
    (4, 2, 128, 16, 64, [160, 75], [5, 0], 50),
]


@pytest.mark.parametrize("coder", list(CODERS))
@pytest.mark.parametrize("geo", GEOMETRIES, ids=lambda g: f"hq{g[0]}kv{g[1]}d{g[2]}t{g[3]}b{g[4]}w{g[7]}")
def test_generic_attention_matches_oracle(native, oracle, coder, geo):
    import torch
    hq, hkv, d, t, block, contexts, tails, window = geo
    rng = np.random.default_rng(5)
    layer, host, kcb, vcb, tail_k, tail_v, stride = _build(native, oracle, rng, hq=hq, hkv=hkv, d=d, t=t, block=block,
                                                           coder=CODERS[coder], contexts=contexts, tails=tails)
    q = rng.standard_normal((len(contexts), hq, d)).astype(np.float16)
    want = _oracle_attention(oracle, host, kcb, vcb, contexts, tails, tail_k, tail_v, q, hq, stride, window)
    got = layer.attention(torch.from_numpy(q).cuda(), causal_window=window, kernel=native.KERNEL_GENERIC).cpu().numpy()
    ok, err = attention_close(got, want)
    assert layer.device_status() == 0
    assert ok, f"max abs error {err}"
    # sequences with no visible token give zeros (src/cuda/paged_kv_attention.cu:170-173)
    for s, (c, tl) in enumerate(zip(contexts, tails)):
        if c + tl == 0:
            assert np.all(got[s] == 0)


@pytest.mark.parametrize("coder", list(CODERS))
def test_gpu_sealer_is_byte_exact(native, oracle, coder):
    """Records written by the GPU sealer equal the oracle's records byte for byte (same quantiser rounding, same
    block streams, same fallback rule, zero padding)."""
    import torch
    rng = np.random.default_rng(23)
    hkv, d, t = 2, 128, 16
    hist = hist_for_coder(laplace_codes(rng, 1 << 16, 4.0).astype(np.int16) + 128, CODERS[coder])
    kcb = oracle.codebook_from_hist(hist)
    vcb = oracle.codebook_from_hist(hist)
    layer = _layer(native, kv_heads=hkv, query_heads=4, coder=CODERS[coder], max_sequences=5)
    layer.set_codebooks(hist, hist)
    cases = []
    for s, (b, rows) in enumerate([(4.0, 16), (12.0, 16), (40.0, 16), (4.0, 9), (0.0, 16)]):
        k, v = _random_kv(rng, hkv, rows, d, b) if b else (np.zeros((hkv, rows, d), np.float32),) * 2
        tk = np.zeros((1, hkv, t, d), np.float16)
        tv = np.zeros((1, hkv, t, d), np.float16)
        tk[0, :, :rows] = k
        tv[0, :, :rows] = v
        layer.fill_tails([s], torch.from_numpy(tk).cuda(), torch.from_numpy(tv).cuda(), rows)
        cases.append((k, v, rows))
    assert layer.seal_full_pages(force=True) == 5
    assert layer.device_status() == 0
    for s, (k, v, rows) in enumerate(cases):
        pid = int(layer.h_page_table[s, 0])
        for h in range(hkv):
            want = oracle.seal_record(k[h], v[h], rows, d, t, 64, CODERS[coder], 0, kcb, vcb)[0]
            got = layer.record_bytes(pid, h)
            assert got.size == want.size, (s, h, got.size, want.size)
            assert np.array_equal(got, want), (s, h)


@pytest.mark.parametrize("coder", list(CODERS))
def test_gpu_sealer_is_byte_exact_on_fp32_rows(native, oracle, coder):
    """The stores behind the reference's ABIs hand the sealer fp32 rows (values that binary16 cannot hold): the records
    must still equal the oracle's byte for byte, full pages and a page of eleven rows."""
    import ctypes as C
    import torch
    rng = np.random.default_rng(29)
    hkv, d, t = 2, 128, 16
    hist = hist_for_coder(laplace_codes(rng, 1 << 16, 12.0).astype(np.int16) + 128, CODERS[coder])
    kcb = oracle.codebook_from_hist(hist)
    vcb = oracle.codebook_from_hist(hist)
    layer = _layer(native, kv_heads=hkv, query_heads=4, coder=CODERS[coder], max_sequences=4)
    layer.set_codebooks(hist, hist)
    rows = [16, 16, 11, 16]
    k = (rng.laplace(0.0, 12.0, (4, hkv, t, d)) * 0.0137).astype(np.float32)
    v = (rng.laplace(0.0, 12.0, (4, hkv, t, d)) * 0.0071).astype(np.float32)
    k[3] = rng.uniform(-1.0, 1.0, (hkv, t, d)).astype(np.float32)      # does not shrink: stored fixed-width
    # values a hair's breadth from the rounding boundaries of the quantiser, x = scale * (n + 1/2) * (1 + j 2^-24): the
    # sealer's multiply-by-reciprocal path must hand exactly these to the division (the oracle divides every value)
    scale = np.float32(np.float16(0.0123))
    n_half = rng.integers(-127, 127, (hkv, t, d)).astype(np.float64) + 0.5
    jitter = 1.0 + rng.integers(-12, 13, (hkv, t, d)).astype(np.float64) * 2.0 ** -24
    v[1] = (np.float64(scale) * n_half * jitter).astype(np.float32)
    v[1, :, 0, 0] = np.float32(127.0) * scale                          # pins the stream's absmax, hence the scale
    dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    ids = torch.arange(1, 5, dtype=torch.int32, device="cuda")
    desc = layer._seal_desc(torch.arange(4, dtype=torch.int32, device="cuda"), ids,
                            torch.as_tensor(rows, dtype=torch.int32, device="cuda"))
    desc.tail_k, desc.tail_v, desc.tail_type = dk.data_ptr(), dv.data_ptr(), native.F32
    assert native.lib().cf_b200_seal_pages_async(C.byref(desc), None) == 0
    torch.cuda.synchronize()
    assert layer.device_status() == 0
    for s in range(4):
        for h in range(hkv):
            want = oracle.seal_record(k[s, h, :rows[s]], v[s, h, :rows[s]], rows[s], d, t, 64, CODERS[coder], 0, kcb, vcb)[0]
            got = layer.record_bytes(s + 1, h)
            assert got.size == want.size and np.array_equal(got, want), (s, h)


def test_gpu_sealer_rejects_non_finite(native, oracle):
    import torch
    layer = _layer(native, max_sequences=2)
    hist = np.ones(256, np.uint64)
    layer.set_codebooks(hist, hist)
    k = torch.zeros((2, 2, 16, 128), dtype=torch.float16, device="cuda")
    v = torch.zeros_like(k)
    k[1, 0, 3, 7] = float("inf")
    layer.fill_tails([0, 1], k, v, 16)
    layer.seal_full_pages()
    assert layer.device_status() & native.DEVSTAT_NONFINITE
    pid_bad = int(layer.h_page_table[1, 0])
    assert int(layer.page_dir[pid_bad * 2].item()) == 0          # not published
    pid_ok = int(layer.h_page_table[0, 0])
    assert int(layer.page_dir[pid_ok * 2].item()) != 0


LANES_CASES = [
    # hq, hkv, contexts, tails, window, min_pages_per_unit
    (32, 8, [128, 96], [7, 0], 0, 0),
    (8, 8, [80, 16], [1, 0], 0, 0),
    (4, 2, [64, 16, 40, 0], [0, 3, 5, 2], 0, 0),
    (8, 4, [330, 75, 16], [5, 0, 15], 0, 2),      # several chunks per sequence: split-KV + combine
    (4, 2, [160, 75], [5, 0], 50, 1),              # causal window cuts inside a page, one page per unit
    (12, 4, [100, 37], [0, 9], 0, 3),              # group of 3, ragged last page
]


@pytest.mark.parametrize("coder", list(CODERS))
@pytest.mark.parametrize("case", LANES_CASES, ids=lambda c: f"hq{c[0]}kv{c[1]}w{c[4]}u{c[5]}")
def test_lanes_kernel_matches_oracle(native, oracle, coder, case):
    """The tensor-core lane-per-block kernel (head_dim 128, 16-token pages, 64-symbol blocks)."""
    import torch
    hq, hkv, contexts, tails, window, ppu = case
    rng = np.random.default_rng(17)
    layer, host, kcb, vcb, tail_k, tail_v, stride = _build(native, oracle, rng, hq=hq, hkv=hkv, d=128, t=16, block=64,
                                                           coder=CODERS[coder], contexts=contexts, tails=tails)
    q = rng.standard_normal((len(contexts), hq, 128)).astype(np.float16)
    want = _oracle_attention(oracle, host, kcb, vcb, contexts, tails, tail_k, tail_v, q, hq, stride, window)
    got = layer.attention(torch.from_numpy(q).cuda(), causal_window=window, kernel=native.KERNEL_LANES,
                          min_pages_per_unit=ppu).cpu().numpy()
    assert layer.device_status() == 0
    ok, err = attention_close(got, want)
    assert ok, f"max abs error {err}"
    generic = layer.attention(torch.from_numpy(q).cuda(), causal_window=window, kernel=native.KERNEL_GENERIC,
                              min_pages_per_unit=ppu).cpu().numpy()
    assert attention_close(got, generic, rel=1e-3, abs_=5e-4)[0]


def test_lanes_kernel_mixed_coders_and_scales(native, oracle):
    """Pages whose streams fell back to fixed width (model mismatch), all-zero pages and wildly different page scales
    in one sequence."""
    import torch
    rng = np.random.default_rng(29)
    hq, hkv, d, t = 8, 2, 128, 16
    hist = hist_of(laplace_codes(rng, 1 << 16, 2.0).astype(np.int16) + 128)   # narrow model
    kcb = oracle.codebook_from_hist(hist)
    vcb = oracle.codebook_from_hist(hist)
    layer = _layer(native, kv_heads=hkv, query_heads=hq, coder=2, max_sequences=1, max_pages_per_sequence=8,
                   max_pages=16)
    layer.set_codebooks(hist, hist)
    host = HostCache(hkv, d, t, 64, 2, kcb, vcb)
    # (K spread, K scale, V scale): V scales differ by 4 orders of magnitude between neighbouring pages; K scales
    # stay where attention logits are O(10), as trained models have them
    for b, k_scale, v_scale in [(2.0, 0.01, 0.01), (60.0, 0.004, 0.01), (2.0, 0.02, 3.0), (0.0, 1.0, 1.0),
                                (60.0, 0.005, 1e-4), (2.0, 0.015, 0.5)]:
        if b:
            kc = laplace_codes(rng, (hkv, t, d), b).astype(np.float32)
            vc = laplace_codes(rng, (hkv, t, d), 2.0 if b > 10 else 60.0).astype(np.float32)
            kc[:, 0, 0] = 127.0   # pins absmax so that the codes keep their spread: narrow streams stay narrow
            vc[:, 0, 0] = 127.0
            k = (kc * k_scale).astype(np.float16).astype(np.float32)
            v = (vc * v_scale).astype(np.float16).astype(np.float32)
        else:
            k = np.zeros((hkv, t, d), np.float32)
            v = np.zeros((hkv, t, d), np.float32)
        host.seal_page(0, k, v)
    coders = {(int(r[4]), int(r[5])) for page in host.records[0] for r in page}
    assert (0, 2) in coders or (2, 0) in coders, coders      # mixed pages are present
    layer.import_records(0, host.records[0], host.tokens[0])
    q = (rng.standard_normal((1, hq, d)) * 0.3).astype(np.float16)
    arena, offsets, table, sealed = host.flat([0], 8)
    want = oracle.sealed_decode_attention(arena, offsets, table, sealed, q, hq, hkv, d, t, 64, 0, 1.0 / np.sqrt(d), kcb, vcb)
    for kernel in (native.KERNEL_GENERIC, native.KERNEL_LANES):
        got = layer.attention(torch.from_numpy(q).cuda(), kernel=kernel).cpu().numpy()
        ok, err = attention_close(got, want)
        assert ok, (kernel, err)
    # the same pages through the shared-prefix kernel (its mixed-coder, all-zero-page and scale handling)
    got = layer.attention(torch.from_numpy(q).cuda(), kernel=native.KERNEL_LANES, shared_prefix_pages=6).cpu().numpy()
    ok, err = attention_close(got, want)
    assert ok, ("prefix", err)
    assert layer.device_status() == 0


def test_bad_records_are_reported_not_faulted(native, oracle):
    """A directory entry that points at garbage raises the device status word; the launch completes."""
    import torch
    rng = np.random.default_rng(31)
    layer, host, kcb, vcb, *_ = _build(native, oracle, rng, hq=4, hkv=2, d=128, t=16, block=64, coder=2,
                                       contexts=[48], tails=[0])
    layer.arena[15] = 9            # version byte of the first record
    q = torch.zeros((1, 4, 128), dtype=torch.float16, device="cuda")
    for kernel in (native.KERNEL_GENERIC, native.KERNEL_LANES):
        layer.status.zero_()
        layer.attention(q, kernel=kernel)
        torch.cuda.synchronize()
        assert layer.device_status() & native.DEVSTAT_BAD_RECORD
    layer.status.zero_()
    layer.attention(q, kernel=native.KERNEL_LANES, shared_prefix_pages=3)   # the shared-prefix kernel skips it too
    torch.cuda.synchronize()
    assert layer.device_status() & native.DEVSTAT_BAD_RECORD


@pytest.mark.parametrize("coder", ["rans", "huffman"])
def test_block_offsets_past_their_part_are_reported(native, oracle, coder):
    """A record with a well-formed header whose block table sends one block past the end of its part (a bad producer,
    not transport damage): every kernel refuses the page with CF_B200_DEVSTAT_BAD_RECORD and the other pages still
    count. The bad offset chosen here still lies inside the record, so the read it would cause is in bounds with or
    without the check."""
    import torch
    rng = np.random.default_rng(32)
    layer, host, kcb, vcb, *_ = _build(native, oracle, rng, hq=4, hkv=2, d=128, t=16, block=64, coder=CODERS[coder],
                                       contexts=[48], tails=[0])
    q = torch.from_numpy(rng.standard_normal((1, 4, 128)).astype(np.float16)).cuda()
    good = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
    assert layer.device_status() == 0
    rec = host.records[0][1][0]                        # page 1 (page id 2), kv head 0
    k_bytes = 16 * int(rec[0] | rec[1] << 8)
    entry = int(layer.page_dir[2 * 2 + 0].item())
    base = (entry & 0xFFFFFFFFFF) * 16 + 16            # the K part in the arena
    if coder == "rans":                                # u32 state0[32] | u16 byte_off[32] | bytes
        at, bad = base + 128 + 2 * 5, k_bytes - 192 + 32
    else:                                              # u16 bit_off[32] | words
        at, bad = base + 2 * 5, (k_bytes - 64) * 8 + 256
    layer.arena[at] = bad & 0xFF
    layer.arena[at + 1] = bad >> 8
    if coder == "rans":                                # and a start state below 2^23 in page 0's V part, kv head 1
        entry0 = int(layer.page_dir[1 * 2 + 1].item())
        rec0 = host.records[0][0][1]
        v_base = (entry0 & 0xFFFFFFFFFF) * 16 + 16 + 16 * int(rec0[0] | rec0[1] << 8)
        layer.arena[v_base + 4 * 9 + 3] = 0            # state0[9] loses its top byte
    outs = []
    for kw in (dict(kernel=native.KERNEL_GENERIC), dict(kernel=native.KERNEL_LANES),
               dict(kernel=native.KERNEL_LANES, shared_prefix_pages=3)):
        layer.status.zero_()
        outs.append(layer.attention(q, **kw).cpu().numpy())
        assert layer.device_status() == native.DEVSTAT_BAD_RECORD, kw
    # the page is skipped whole for that kv head (query heads 0, 1); the other kv head's result is untouched
    if coder == "rans":
        assert not np.array_equal(outs[1][:, 2:], good[:, 2:]) and not np.array_equal(outs[1][:, :2], good[:, :2])
    else:
        assert np.array_equal(outs[1][:, 2:], good[:, 2:]) and not np.array_equal(outs[1][:, :2], good[:, :2])
    ok, err = attention_close(outs[0], outs[1])
    assert ok, err
    ok, err = attention_close(outs[2], outs[1])
    assert ok, err


@pytest.mark.parametrize("hq,hkv", [(32, 8), (8, 8), (16, 2), (6, 2)])
def test_dense_comparison_kernel_matches_oracle(native, oracle, hq, hkv):
    """The uncompressed binary16 paged-attention kernel against the oracle's dense attention on the same values."""
    import torch
    from chromofold_b200.cache import dense_attention, swizzle_dense_tiles
    rng = np.random.default_rng(41)
    contexts = [16 * 21, 16 * 3, 16 * 40]
    pages = [c // 16 for c in contexts]
    layer = _layer(native, kv_heads=hkv, query_heads=hq, max_sequences=3, max_pages_per_sequence=max(pages),
                   max_pages=sum(pages) + 2)
    pool_k = torch.zeros((sum(pages) + 2, hkv, 16, 128), dtype=torch.float16, device="cuda")
    pool_v = torch.zeros_like(pool_k)
    q = rng.standard_normal((3, hq, 128)).astype(np.float16)
    pid = 1
    want = []
    for s, n in enumerate(pages):
        k = rng.standard_normal((hkv, n * 16, 128)).astype(np.float16)
        v = rng.standard_normal((hkv, n * 16, 128)).astype(np.float16)
        tiles_k = torch.from_numpy(k.reshape(hkv, n, 16, 128).transpose(1, 0, 2, 3).copy()).cuda()
        tiles_v = torch.from_numpy(v.reshape(hkv, n, 16, 128).transpose(1, 0, 2, 3).copy()).cuda()
        pool_k[pid:pid + n] = swizzle_dense_tiles(tiles_k)
        pool_v[pid:pid + n] = swizzle_dense_tiles(tiles_v)
        layer.h_page_table[s, :n] = np.arange(pid, pid + n)
        pid += n
        rc, o = oracle.dense_attention(k.astype(np.float32), v.astype(np.float32), 0, q[s:s + 1].astype(np.float32),
                                       n * 16, 0, 1.0 / np.sqrt(128.0))
        assert rc == 0
        want.append(o[0])
    layer.page_table.copy_(torch.from_numpy(layer.h_page_table))
    layer.sealed_tokens.copy_(torch.tensor(contexts, dtype=torch.int32))
    out = torch.zeros((3, hq, 128), dtype=torch.float32, device="cuda")
    dense_attention(layer, pool_k, pool_v, torch.from_numpy(q).cuda(), out)
    ok, err = attention_close(out.cpu().numpy(), np.stack(want))
    assert ok, err


@pytest.mark.gpu
def test_decode_step_replays_from_a_cuda_graph(native, oracle):
    """The attention call allocates nothing, synchronises nothing and copies nothing between host and device, so a
    serving loop can capture a decode step (plan, attention, combine) once and replay it: the replay reads the current
    queries and page tables, and gives the eager result bit for bit."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    layer, info = build_sealed_layer(np.array([640, 1296, 48]), coder="rans", seed=21)
    q = torch.randn((3, 32, 128), device="cuda").half()
    out = torch.zeros((3, 32, 128), dtype=torch.float32, device="cuda")
    eager = layer.attention(q, out=out).clone()                  # also the first call: one-time kernel attributes are set
    torch.cuda.synchronize()
    out.zero_()
    graph = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph.capture_begin()
        layer.attention(q, out=out)
        graph.capture_end()
    torch.cuda.current_stream().wait_stream(side)
    assert float(out.abs().max()) == 0.0                          # captured, not run
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)
    q.copy_(torch.randn((3, 32, 128), device="cuda").half())     # new queries in the same buffer: the replay sees them
    graph.replay()
    torch.cuda.synchronize()
    again = out.clone()
    assert torch.equal(again, layer.attention(q).to(again.dtype)) and not torch.equal(again, eager)
    assert layer.device_status() == 0


@pytest.mark.gpu
def test_one_process_drives_two_devices(native, oracle):
    """Kernel attributes (the dynamic shared-memory opt-in) belong to a device: a process that works on a second GPU
    after the first must find its kernels configured there too. Same layer, same queries on both devices: same bits."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs in one process")
    results = []
    for index in (0, 1):
        device = torch.device("cuda", index)
        with torch.cuda.device(device):
            layer, info = build_sealed_layer(np.array([512, 2064, 96]), coder="rans", seed=33, device=device)
            g = torch.Generator(device=device)
            g.manual_seed(34)
            q = torch.randn((3, 32, 128), generator=g, device=device).half()
            outs = [layer.attention(q), layer.attention(q.float()), layer.attention(q, kernel=native.KERNEL_GENERIC),
                    layer.attention(q, shared_prefix_pages=0)]
            torch.cuda.synchronize(device)
            assert layer.device_status() == 0
            results.append([o.cpu().numpy() for o in outs])
    for a, b in zip(*results):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("prefix", [0, 8])
def test_a_wait_that_runs_out_is_reported_and_the_next_call_is_right(native, oracle, prefix):
    """The bounded waits on the page copies: with the test hook one record is armed on its barrier and never fetched, and
    the bound is lowered to 2000 polls. The warp that waits for it gives up, raises CF_B200_DEVSTAT_WAIT_EXPIRED and
    leaves; the launch ends by itself. With the hook off the very next call on the same store gives the right answer
    (prefix = 8: the same through the shared-prefix kernel, whose leaving path also has to free its tensor memory)."""
    import torch
    rng = np.random.default_rng(35)
    layer, host, kcb, vcb, tail_k, tail_v, stride = _build(native, oracle, rng, hq=4, hkv=2, d=128, t=16, block=64, coder=CODERS["rans4"],
                                                           contexts=[160, 160], tails=[0, 0], workspace_bytes=4 << 20)
    if prefix:
        layer.copy_sequence(0, 1)      # both entries now name the same ten pages
    q = torch.from_numpy(rng.standard_normal((2, 4, 128)).astype(np.float16)).cuda()
    kw = dict(kernel=native.KERNEL_LANES, shared_prefix_pages=prefix)
    good = layer.attention(q, **kw).cpu().numpy()
    assert layer.device_status() == 0
    lib = native.lib()
    try:
        assert lib.cf_b200_test_wait_expiry(3, 2000) == 0       # page id 3 = third page of sequence 0
        layer.attention(q, **kw)
        torch.cuda.synchronize()
        assert layer.device_status() & native.DEVSTAT_WAIT_EXPIRED
    finally:
        assert lib.cf_b200_test_wait_expiry(0, 0) == 0
    layer.status.zero_()
    again = layer.attention(q, **kw).cpu().numpy()
    assert layer.device_status() == 0 and np.array_equal(again, good)


def test_append_rows_entry_point_fills_the_tails_and_reports_a_full_one(native):
    """cf_b200_append_rows_async: one launch stores a token's K and V rows (binary16 or fp32 rows) at each listed slot's
    tail position and raises the count; a slot whose tail is full takes nothing and raises CF_B200_DEVSTAT_TAIL_FULL."""
    import torch
    layer = _layer(native, kv_heads=2, query_heads=4, max_sequences=4)
    rng = np.random.default_rng(71)
    want_k = np.zeros((4, 2, 16, 128), np.float16)
    want_v = np.zeros_like(want_k)
    counts = [0, 0, 0, 0]
    for step in range(16):
        slots = [0, 2, 3] if step % 2 == 0 else [2, 1]
        dtype = np.float16 if step % 3 else np.float32
        k = rng.standard_normal((len(slots), 2, 128)).astype(dtype)
        v = rng.standard_normal((len(slots), 2, 128)).astype(dtype)
        dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        if step % 5 == 4:            # bfloat16 rows: the values the tail must hold are the bf16-rounded ones
            dk, dv = dk.to(torch.bfloat16), dv.to(torch.bfloat16)
            k, v = dk.float().cpu().numpy(), dv.float().cpu().numpy()
        layer.append(slots, dk, dv)
        for i, s in enumerate(slots):
            want_k[s, :, counts[s]] = k[i].astype(np.float16)
            want_v[s, :, counts[s]] = v[i].astype(np.float16)
            counts[s] += 1
    assert layer.tail_tokens.cpu().tolist() == counts == [8, 8, 16, 8] and layer.device_status() == 0
    assert np.array_equal(layer.tail_k.cpu().numpy(), want_k) and np.array_equal(layer.tail_v.cpu().numpy(), want_v)
    with pytest.raises(ValueError):                 # the host mirror refuses before the device is asked
        layer.append([2], torch.zeros((1, 2, 128), dtype=torch.float16, device="cuda"), torch.zeros((1, 2, 128), dtype=torch.float16, device="cuda"))
    layer.h_tail[2] = 0                             # ask the device anyway: nothing is stored, the status bit is raised
    layer.append([2], torch.ones((1, 2, 128), dtype=torch.float16, device="cuda"), torch.ones((1, 2, 128), dtype=torch.float16, device="cuda"))
    torch.cuda.synchronize()
    assert layer.device_status() == native.DEVSTAT_TAIL_FULL
    assert layer.tail_tokens.cpu().tolist() == counts and np.array_equal(layer.tail_k.cpu().numpy(), want_k)
