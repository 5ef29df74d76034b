"""Randomised cases of the decode-attention path: geometry, coder, batch shape, context lengths (empty and ragged ones
included), shared prefixes, kv-head shards, unit sizes, causal windows, fp32 queries and query positions are drawn from
a seed, K and V rows with magnitudes that change from token to token by orders of magnitude, and the lane-per-block
kernels (with the shared-prefix kernel where the case has a prefix) are compared with the CPU oracle or, where the
oracle has no such option, with the any-geometry kernel, which computes in fp32 throughout."""
import numpy as np
import pytest

from helpers import oracle_from_layer

pytestmark = pytest.mark.gpu

GEOMETRIES = [(128, 64), (128, 64), (128, 128), (128, 256), (64, 64), (96, 64), (32, 64), (64, 128)]   # head_dim, block
HEADS = [(32, 8), (16, 8), (8, 8), (64, 8), (8, 2)]
CODERS = ["rans4", "huffman4", "rans", "huffman", "fixed8"]


def _close(actual, expected):
    """|a - e| <= 2e-4 * (largest |e| of the row + 0.5 % of the largest |e| of the case): far inside the 2e-3 bar, and
    scaled to the data because the V rows span six orders of magnitude. The second term is there for rows whose exact
    value is nearly zero next to the values the row is averaged from (a dominant token whose V quantised to zero):
    the kernels resolve softmax weights down to 2^-40 of the row maximum, the fp32 checkers further."""
    a, e = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    scale = np.abs(e).max(axis=-1, keepdims=True) + 5e-3 * np.abs(e).max() + 1e-30
    err = np.abs(a - e) / scale
    return bool(np.all(np.isfinite(a)) and err.max() <= 2e-4), float(err.max())


def _case(native, seed):
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    rng = np.random.default_rng(seed)
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    n = int(rng.integers(1, 13))
    head_dim, block = GEOMETRIES[int(rng.integers(0, len(GEOMETRIES)))]
    hq, hkv = HEADS[int(rng.integers(0, len(HEADS)))]
    coder = CODERS[int(rng.integers(0, len(CODERS)))]
    group = hq // hkv
    prefix_pages = int(rng.integers(1, 12)) if (head_dim == 128 and block == 64 and 128 % group == 0 and rng.random() < 0.5) else 0
    contexts = rng.integers(0, 300, n)
    if rng.random() < 0.3:
        contexts[int(rng.integers(0, n))] = 0
    pages = int(contexts.max()) // 16 + prefix_pages + 3
    layer, _ = build_sealed_layer(np.array([0] * n), query_heads=hq, kv_heads=hkv, head_dim=head_dim, block_size=block,
                                  coder=coder, seed=seed, extra_pages_per_sequence=pages, reserve_pages=n * pages + 8)
    hist = np.rint(1e6 * np.exp(-np.abs(np.arange(256) - 128) / float(rng.uniform(2, 40)))).astype(np.uint64) + 1
    layer.set_codebooks(hist, hist)
    wild = rng.random() < 0.6

    def rows(count):
        k = torch.randn((count, hkv, head_dim), generator=g, device="cuda")
        v = torch.randn((count, hkv, head_dim), generator=g, device="cuda")
        if wild:   # a new magnitude for every token
            k = k * float(10.0 ** rng.uniform(-2, 0.7))
            v = v * float(10.0 ** rng.uniform(-4, 2))
        return k.float(), v.float()

    for _ in range(16 * prefix_pages):       # the shared prefix: sealed on slot 0, then referenced by every other slot
        layer.append([0], *rows(1))
        layer.seal_full_pages()
    for s in range(1, n):
        if prefix_pages:
            layer.copy_sequence(0, s)
    for t in range(int(contexts.max())):
        slots = [s for s in range(n) if contexts[s] > t]
        layer.append(slots, *rows(len(slots)))
        layer.seal_full_pages()

    q = (torch.randn((n, hq, head_dim), generator=g, device="cuda") * float(10.0 ** rng.uniform(-1, 0.5))).half()
    options = {}
    if prefix_pages and rng.random() < 0.8:
        options["shared_prefix_pages"] = prefix_pages
    if rng.random() < 0.3:
        span = int(rng.integers(1, hkv + 1))
        options["kv_head_begin"], options["kv_head_span"] = int(rng.integers(0, hkv - span + 1)), span
    if rng.random() < 0.3:
        options["min_pages_per_unit"] = int(rng.integers(1, 9))
    if rng.random() < 0.25 and "shared_prefix_pages" not in options:
        options["causal_window"] = int(rng.integers(1, 200))
    positions = None
    if rng.random() < 0.25:   # query tokens somewhere inside what is cached (behind the shared prefix, if claimed)
        cached = (layer.h_sealed[:n] + layer.h_tail[:n]).astype(np.int64)
        low = 16 * prefix_pages if "shared_prefix_pages" in options else 0
        positions = torch.from_numpy(np.array([int(rng.integers(low, max(c, low) + 1)) for c in cached], np.int32)).cuda()
        options["query_positions"] = positions
    queries = q.float() if rng.random() < 0.3 else q

    out = torch.full((n, hq, head_dim), 7.0, dtype=torch.float32, device="cuda")
    layer.attention(queries, out=out, kernel=native.KERNEL_LANES, **options)
    assert layer.device_status() == 0
    got = out.cpu().numpy()
    if positions is None:
        want = oracle_from_layer(layer, q.cpu().numpy(), causal_window=options.get("causal_window", 0))
    else:
        plain = {k: v for k, v in options.items() if k in ("causal_window", "query_positions")}
        want = layer.attention(q, kernel=native.KERNEL_GENERIC, **plain).cpu().numpy()
        assert layer.device_status() == 0
    lo = options.get("kv_head_begin", 0) * group
    hi = lo + options.get("kv_head_span", hkv) * group
    ok, err = _close(got[:, lo:hi], want[:, lo:hi])
    what = dict(seed=seed, n=n, head_dim=head_dim, block=block, heads=(hq, hkv), coder=coder, prefix_pages=prefix_pages,
                wild=wild, options={k: v for k, v in options.items() if k != "query_positions"},
                positions=None if positions is None else positions.cpu().tolist(), contexts=contexts.tolist())
    assert ok, (err, what)
    assert np.all(got[:, :lo] == 7.0) and np.all(got[:, hi:] == 7.0), what    # the other heads' columns are not touched


@pytest.mark.parametrize("first", range(0, 96, 8))
def test_random_cases_against_the_fp32_checkers(native, oracle, first):
    for seed in range(first, first + 8):
        _case(native, 1000 + seed)


SEAL_GEOMETRIES = [(128, 64), (128, 64), (128, 128), (128, 256), (64, 64), (96, 64), (32, 64), (64, 128), (96, 128)]


def _rows_of_some_kind(rng, shape):
    """K or V rows [kv head][token][channel] of one of eight kinds, at a magnitude between 1e-9 and 1e5."""
    kind = int(rng.integers(0, 8))
    mag = float(10.0 ** rng.uniform(-9, 5))
    if kind == 0:
        x = rng.laplace(0, 1, shape) * mag
    elif kind == 1:
        x = rng.normal(0, 1, shape) * mag
    elif kind == 2:
        x = rng.uniform(-1, 1, shape) * mag
    elif kind == 3:   # a few outliers over a quiet floor
        x = rng.normal(0, 1, shape) * mag * 1e-3
        x.reshape(-1)[rng.integers(0, x.size, 5)] = rng.choice([-1, 1], 5) * mag
    elif kind == 4:
        x = np.zeros(shape)
    elif kind == 5:
        x = np.full(shape, mag) * rng.choice([-1, 1])
    elif kind == 6:   # on and around the quantiser's rounding boundaries
        scale = np.float32(np.float16(mag / 127)) if 0 < mag / 127 < 6e4 else np.float32(1.0)
        x = np.float64(scale) * (rng.integers(-127, 127, shape) + 0.5) * (1.0 + rng.integers(-3, 4, shape) * 2.0 ** -24)
        x.reshape(-1)[0] = 127.0 * float(scale)
    else:             # a magnitude per token
        x = rng.normal(0, 1, shape) * (10.0 ** rng.uniform(-6, 2, (shape[0], shape[1], 1)))
    return x.astype(np.float32)


@pytest.mark.parametrize("first", range(0, 120, 20))
def test_random_sealer_cases_are_byte_exact(native, oracle, first):
    """The GPU sealer (both kernels: compile-time geometry and any geometry) against the oracle's records, byte for byte:
    random geometry, coder, codebook, rows per page, fp32 or binary16 rows of the kinds above."""
    import ctypes as C
    import torch
    from chromofold_b200.cache import SealedKvLayer
    from helpers import hist_for_coder, laplace_codes
    for seed in range(2000 + first, 2000 + first + 20):
        rng = np.random.default_rng(seed)
        d, block = SEAL_GEOMETRIES[int(rng.integers(0, len(SEAL_GEOMETRIES)))]
        coder = int(rng.integers(0, 5))
        hkv, t, n = 2, 16, 4
        hist = hist_for_coder(laplace_codes(rng, 1 << 15, float(rng.uniform(1.5, 40))).astype(np.int16) + 128, coder)
        kcb, vcb = oracle.codebook_from_hist(hist), oracle.codebook_from_hist(hist[::-1].copy())
        layer = SealedKvLayer(kv_heads=hkv, query_heads=4, head_dim=d, page_tokens=t, block_size=block, coder=coder,
                              max_sequences=n, max_pages_per_sequence=4, max_pages=64, arena_bytes=2 << 20)
        layer.set_codebooks(hist, hist[::-1].copy())
        rows = [int(rng.integers(1, 17)) if rng.random() < 0.4 else 16 for _ in range(n)]
        k = np.stack([_rows_of_some_kind(rng, (hkv, t, d)) for _ in range(n)])
        v = np.stack([_rows_of_some_kind(rng, (hkv, t, d)) for _ in range(n)])
        half = rng.random() < 0.4
        if half:
            k = np.clip(k, -6e4, 6e4).astype(np.float16).astype(np.float32)
            v = np.clip(v, -6e4, 6e4).astype(np.float16).astype(np.float32)
            dk, dv = torch.from_numpy(k.astype(np.float16)).cuda(), torch.from_numpy(v.astype(np.float16)).cuda()
        else:
            dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        desc = layer._seal_desc(torch.arange(n, dtype=torch.int32, device="cuda"),
                                torch.arange(1, n + 1, dtype=torch.int32, device="cuda"),
                                torch.as_tensor(rows, dtype=torch.int32, device="cuda"))
        desc.tail_k, desc.tail_v, desc.tail_type = dk.data_ptr(), dv.data_ptr(), native.F16 if half else native.F32
        assert native.lib().cf_b200_seal_pages_async(C.byref(desc), None) == 0
        torch.cuda.synchronize()
        assert layer.device_status() == 0
        for s in range(n):
            for h in range(hkv):
                want = oracle.seal_record(k[s, h, :rows[s]], v[s, h, :rows[s]], rows[s], d, t, block, coder, 0, kcb, vcb)[0]
                got = layer.record_bytes(s + 1, h)
                assert got.size == want.size and np.array_equal(got, want), (seed, d, block, coder, rows, half, s, h)


@pytest.mark.parametrize("first", range(0, 60, 20))
def test_random_reference_descriptor_cases(native, oracle, first):
    """cf_kv_paged_attention_async on random descriptors of the reference's own fixed-width pages (its fixture encoder
    makes them): heads, head_dim (48 and 80 too), 4 or 8 bits, ragged page sizes, no page at all, fp32 tail, several
    query rows, causal window, per-token magnitudes. The answer must match fp64 softmax over the dequantised rows, and
    the reference's kernel (compiled from its sources) must return the same status on the same descriptor."""
    import ctypes as C
    import torch
    from compat_types import DevicePage, PagedAttentionDesc
    from test_gpu_compat import _dev, _softmax_attention
    ref_cpu, ref_cuda = oracle.ref_cpu(), oracle.ref_cuda()
    if ref_cpu is None or ref_cuda is None:
        pytest.skip("needs oracle/_ref (the reference's fixture encoder and kernels)")
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)
    for seed in range(first, first + 20):
        rng = np.random.default_rng(seed)
        hq, hkv = [(14, 2), (8, 8), (4, 2), (6, 2), (32, 8), (16, 2), (1, 1), (64, 8)][int(rng.integers(0, 8))]
        d = [32, 64, 96, 128, 128, 48, 80][int(rng.integers(0, 7))]
        bits = [4, 8][int(rng.integers(0, 2))]
        full = int(rng.choice([16, 32, 64]))
        sizes = [full if rng.random() < 0.7 else int(rng.integers(1, full + 1)) for _ in range(int(rng.integers(0, 9)))]
        wild = rng.random() < 0.5
        pages, keep, begin = [], [], 0
        dense_k = np.zeros((hkv, sum(sizes), d), np.float32)
        dense_v = np.zeros_like(dense_k)
        for tokens in sizes:
            for h in range(hkv):
                n = tokens * d
                k = rng.standard_normal(n).astype(np.float32)
                v = rng.standard_normal(n).astype(np.float32)
                if wild:
                    k = (k.reshape(tokens, d) * (10.0 ** rng.uniform(-2, 0.7, (tokens, 1)))).astype(np.float32).reshape(-1)
                    v = (v.reshape(tokens, d) * (10.0 ** rng.uniform(-4, 2, (tokens, 1)))).astype(np.float32).reshape(-1)
                words, blocks = (n * bits + 31) // 32, (n + 63) // 64
                kw, vw = np.zeros(words + 1, np.uint32), np.zeros(words + 1, np.uint32)
                ko, vo = np.zeros(blocks, np.int32), np.zeros(blocks, np.int32)
                lut = np.zeros(1 << bits, np.int32)
                ks, vs = np.zeros(d, np.float32), np.zeros(tokens, np.float32)
                dk, dv = np.zeros(n, np.float32), np.zeros(n, np.float32)
                assert ref_cpu.ref_fixture_encode(ptr(k), ptr(v), C.c_uint32(begin), C.c_uint32(tokens), C.c_uint32(d),
                                                  C.c_uint32(h), C.c_uint32(64), C.c_uint32(bits), ptr(kw), ptr(ko), ptr(vw),
                                                  ptr(vo), ptr(lut), ptr(ks), ptr(vs), ptr(dk), ptr(dv), None) == 0
                dense_k[h, begin:begin + tokens] = dk.reshape(tokens, d)
                dense_v[h, begin:begin + tokens] = dv.reshape(tokens, d)
                held = [_dev(x) for x in (kw, ko, lut, ks, vw, vo, lut, vs)]
                keep.append(held)
                pg = DevicePage()
                (pg.k_words, pg.k_block_offsets, pg.k_lut, pg.k_scales, pg.v_words, pg.v_block_offsets, pg.v_lut,
                 pg.v_scales) = [x.data_ptr() for x in held]
                pg.token_begin, pg.token_count, pg.head_dim, pg.block_size = begin, tokens, d, 64
                pg.k_max_code_length = pg.v_max_code_length = bits
                pg.zero_point, pg.kv_head, pg.fixed_code_length = 1 << (bits - 1), h, bits
                pages.append(pg)
            begin += tokens
        sealed = sum(sizes)
        tail = int(rng.integers(0, 12))
        if sealed + tail == 0:
            tail = 1
        nq = int(rng.integers(1, min(5, sealed + tail) + 1))
        window = int(rng.integers(1, sealed + tail + 5)) if rng.random() < 0.5 else 0
        tk = rng.standard_normal((max(tail, 1), hkv, d)).astype(np.float32)[:tail]
        tv = rng.standard_normal((max(tail, 1), hkv, d)).astype(np.float32)[:tail]
        q = (rng.standard_normal((nq, hq, d)) * 10.0 ** rng.uniform(-1, 0.5)).astype(np.float32)
        desc = PagedAttentionDesc()
        desc.struct_size, desc.abi_version = C.sizeof(desc), 0
        if pages:
            d_pages = _dev(np.frombuffer(bytes((DevicePage * len(pages))(*pages)), np.uint8).copy())
            desc.pages = d_pages.data_ptr()
        desc.page_count = len(pages)
        desc.kv_head_count, desc.query_head_count, desc.gqa_group_size = hkv, hq, hq // hkv
        if tail:
            d_tk, d_tv = _dev(tk), _dev(tv)
            desc.active_k, desc.active_v = d_tk.data_ptr(), d_tv.data_ptr()
        desc.active_token_begin, desc.active_token_count = sealed, tail
        d_q = _dev(q)
        desc.queries, desc.query_token_begin, desc.query_count = d_q.data_ptr(), sealed + tail - nq, nq
        desc.head_dim, desc.causal_window, desc.softmax_scale = d, window, 1.0 / np.sqrt(d)
        k_all = np.concatenate([dense_k, tk.transpose(1, 0, 2)], axis=1)
        v_all = np.concatenate([dense_v, tv.transpose(1, 0, 2)], axis=1)
        pos = [sealed + tail - nq + i for i in range(nq)]
        want = _softmax_attention(k_all, v_all, q, pos, [max(0, p + 1 - window) if window else 0 for p in pos],
                                  1.0 / np.sqrt(d), hq // hkv)
        answers = []
        for lib in (native.lib(), ref_cuda):
            out = torch.full((nq, hq, d), 3.0, dtype=torch.float32, device="cuda")
            desc.output = out.data_ptr()
            checked = lib.cf_kv_validate_paged_attention_desc(C.byref(desc))
            status = lib.cf_kv_paged_attention_async(C.byref(desc), None)
            torch.cuda.synchronize()
            answers.append((checked, status, out.cpu().numpy()))
        what = dict(seed=seed, heads=(hq, hkv), d=d, bits=bits, sizes=sizes, tail=tail, nq=nq, window=window, wild=wild)
        assert answers[0][:2] == answers[1][:2], what
        if answers[0][1] == 0:
            got = answers[0][2]
            assert np.isfinite(got).all() and np.abs(got - want).max() <= 2e-4 * (np.abs(want).max() + 1e-30), what


# ---- the multi-sequence cache ABI under random operations -------------------------------------------------------------
# A Python model holds, per sequence, the logical position of its first row and the rows of every layer; every operation
# the model allows must succeed, and attention must match the model's rows (sealed pages quantised as the sealer does).
def _multisequence_run(native, oracle, seed, steps):
    import ctypes as C
    import torch
    from compat_types import MsBatchItem, MultisequenceConfig, MultisequenceCounters
    from test_gpu_ms_resolver import _expected
    from test_gpu_mscache import _view
    INF, END = 1 << 40, 1 << 30   # removal takes 64-bit positions, copy and shift 32-bit ones
    rng = np.random.default_rng(seed)
    LAYERS = int(rng.integers(1, 3)); HKV = int(rng.choice([1, 2, 4])); G = int(rng.choice([1, 2, 4])); HQ = HKV * G
    D = int(rng.choice([128, 128, 64])); PAGE = 16
    lib = native.lib()
    lib.cf_multisequence_create.restype = C.c_void_p
    lib.cf_multisequence_last_error.restype = C.c_char_p
    lib.cf_sequence_speculation_begin.restype = C.c_uint64
    c = C.c_void_p(lib.cf_multisequence_create(C.byref(MultisequenceConfig(LAYERS, HKV, HQ, D, PAGE, G, 0, 1))))
    assert c.value
    err = lambda: lib.cf_multisequence_last_error(c)
    i64 = C.c_int64
    seqs = {}   # id -> dict(base=int, rows=[per layer [k, v]])
    next_id = 1
    log = []
    def item(seq, layer, q, out, position):
        it = MsBatchItem()
        it.sequence_id, it.layer = seq, layer
        it.query = _view(q, q.shape[0])
        it.output, it.output_type = out.data_ptr(), 3
        es = out.element_size()
        it.output_token_stride_bytes, it.output_head_stride_bytes, it.output_element_stride_bytes = out.stride(0) * es, out.stride(1) * es, es
        it.query_token_begin, it.softmax_scale, it.causal_window = position, 1.0 / np.sqrt(D), 0
        return it
    def append(seq, tokens):
        s = seqs[seq]
        dtype = [torch.float16, torch.float32, torch.bfloat16][int(rng.integers(0, 3))]
        for layer in range(LAYERS):
            k = torch.from_numpy(rng.standard_normal((tokens, HKV, D)).astype(np.float32) * 0.8).to(dtype).cuda()
            v = torch.from_numpy(rng.standard_normal((tokens, HKV, D)).astype(np.float32) * 0.8).to(dtype).cuda()
            begin = s["base"] + s["rows"][layer][0].shape[0]
            rc = lib.cf_sequence_append_async(c, i64(seq), layer, begin, C.byref(_view(k, tokens)), C.byref(_view(v, tokens)), None)
            assert rc == 0, ("append", seq, layer, tokens, begin, err(), log[-6:])
            s["rows"][layer] = [np.concatenate([s["rows"][layer][0], k.float().cpu().numpy()]), np.concatenate([s["rows"][layer][1], v.float().cpu().numpy()])]
    def count(seq): return seqs[seq]["rows"][0][0].shape[0]
    pending = []   # attention batches launched and not yet checked: (pairs, queries, outputs, rows captured at launch)
    def attend(pairs, defer=False):
        qs, outs, items, rows = [], [], (MsBatchItem * len(pairs))(), []
        for i, (seq, layer) in enumerate(pairs):
            nq = int(rng.integers(1, min(4, count(seq)) + 1)) if rng.random() < 0.3 else 1   # a short prefill item now and then
            q = torch.from_numpy(rng.standard_normal((nq, HQ, D)).astype(np.float32)).cuda()
            out = torch.zeros((nq, HQ, D), dtype=torch.float32, device="cuda")
            items[i] = item(seq, layer, q, out, seqs[seq]["base"] + count(seq) - nq)
            qs.append(q); outs.append(out); rows.append(tuple(seqs[seq]["rows"][layer]))
        rc = lib.cf_multisequence_attention_async(c, items, len(pairs), None)
        assert rc == 0, ("attend", pairs, err(), log[-6:])
        pending.append((pairs, qs, outs, rows, list(log[-8:])))
        if not defer: settle()
    def settle():
        torch.cuda.synchronize()
        for pairs, qs, outs, rows, at in pending:
            for (seq, layer), q, out, (k, v) in zip(pairs, qs, outs, rows):
                sealed = k.shape[0] // PAGE * PAGE
                nq = q.shape[0]
                want = _expected(oracle, k, v, sealed, 16, q.cpu().numpy(), list(range(k.shape[0] - nq, k.shape[0])), 1.0 / np.sqrt(D), G)
                got = out.cpu().numpy()
                assert np.allclose(got, want, rtol=2e-3, atol=1e-3), ("attention differs", seq, layer, float(np.abs(got - want).max()), at, log[-8:])
        pending.clear()
    for step in range(steps):
        ops = ["create", "append", "append", "append", "attend", "attend", "copy", "remove_suffix", "remove", "shift", "speculate", "reclaim"]
        op = ops[int(rng.integers(0, len(ops)))]
        live = [s for s in seqs]
        nonempty = [s for s in live if count(s) > 0]
        if op == "create" or not live:
            if len(live) >= 6: continue
            assert lib.cf_sequence_create(c, i64(next_id)) == 0, err()
            seqs[next_id] = dict(base=0, rows=[[np.zeros((0, HKV, D), np.float32)] * 2 for _ in range(LAYERS)])
            log.append(("create", next_id)); next_id += 1
        elif op == "append":
            seq = live[int(rng.integers(0, len(live)))]
            if count(seq) > 200: continue
            room = PAGE - count(seq) % PAGE
            for _ in range(int(rng.integers(1, 4))):
                room = PAGE - count(seq) % PAGE
                tokens = int(rng.integers(1, room + 1)) if rng.random() < 0.6 else room
                log.append(("append", seq, tokens)); append(seq, tokens)
        elif op == "attend" and nonempty:
            pairs = [(nonempty[int(rng.integers(0, len(nonempty)))], int(rng.integers(0, LAYERS))) for _ in range(int(rng.integers(1, 6)))]
            if rng.random() < 0.5: pairs = [(s, pairs[0][1]) for s, _ in pairs]   # one layer for the whole batch
            pairs = list(dict.fromkeys(pairs)) if rng.random() < 0.5 else pairs
            defer = rng.random() < 0.6
            log.append(("attend", pairs, "deferred" if defer else "")); attend(pairs, defer)
        elif op == "copy" and nonempty and len(live) < 6:
            src = nonempty[int(rng.integers(0, len(nonempty)))]
            s = seqs[src]; n = count(src); sealed = n // PAGE * PAGE
            kind = int(rng.integers(0, 4))
            if kind == 0: b, e = 0, END
            elif kind == 1: b, e = 0, s["base"] + int(rng.integers(0, sealed + 1))
            elif kind == 2: b, e = s["base"] + int(rng.integers(0, sealed + 1)), END
            else:
                x, y = sorted(int(v) for v in rng.integers(0, sealed + 1, 2)); b, e = s["base"] + x, s["base"] + y
            # model: pages wholly inside [b, e), active rows only when e reaches the end
            first = max(0, -(-(b - s["base"]) // PAGE))                 # first page index wholly at or after b
            last = min(sealed, (min(e, s["base"] + n) - s["base"]) // PAGE * PAGE) // PAGE   # one past the last whole page before e
            lo_row = first * PAGE
            hi_row = n if e >= s["base"] + n else last * PAGE
            if hi_row <= lo_row: continue
            rc = lib.cf_sequence_copy_async(c, i64(src), i64(next_id), C.c_uint32(b), C.c_uint32(e), None)
            log.append(("copy", src, next_id, b, e, "rows", lo_row, hi_row, "base", s["base"], "n", n))
            assert rc == 0, ("copy", err(), log[-6:])
            seqs[next_id] = dict(base=s["base"] + lo_row, rows=[[a[lo_row:hi_row].copy() for a in s["rows"][layer]] for layer in range(LAYERS)])
            next_id += 1
        elif op == "remove_suffix" and nonempty:
            seq = nonempty[int(rng.integers(0, len(nonempty)))]
            s = seqs[seq]; n = count(seq); sealed = n // PAGE * PAGE
            if sealed == 0: continue
            cut = int(rng.integers(1, sealed // PAGE + 1)) * PAGE   # keep at least one page
            rc = lib.cf_sequence_remove_async(c, i64(seq), i64(s["base"] + cut), i64(INF), None)
            log.append(("remove_suffix", seq, s["base"] + cut))
            assert rc == 0, ("remove suffix", err(), log[-6:])
            s["rows"] = [[a[:cut] for a in s["rows"][layer]] for layer in range(LAYERS)]
        elif op == "remove" and len(live) > 1:
            seq = live[int(rng.integers(0, len(live)))]
            assert lib.cf_sequence_remove_async(c, i64(seq), i64(-1), i64(-1), None) == 0, err()
            log.append(("remove", seq)); del seqs[seq]
        elif op == "shift" and nonempty:
            seq = nonempty[int(rng.integers(0, len(nonempty)))]
            s = seqs[seq]
            delta = int(rng.integers(-s["base"], 40)) if s["base"] else int(rng.integers(0, 40))
            rc = lib.cf_sequence_shift_async(c, i64(seq), C.c_uint32(0), C.c_uint32(END), C.c_int32(delta), None)
            log.append(("shift", seq, delta, "base", s["base"]))
            assert rc == 0, ("shift", err(), log[-6:])
            s["base"] += delta
        elif op == "speculate" and nonempty:
            seq = nonempty[int(rng.integers(0, len(nonempty)))]
            room = PAGE - count(seq) % PAGE
            if room < 3: continue
            k = int(rng.integers(1, room))   # does not fill the page
            spec = lib.cf_sequence_speculation_begin(c, i64(seq))
            before = [[a.copy() for a in seqs[seq]["rows"][layer]] for layer in range(LAYERS)]
            n0 = count(seq)
            append(seq, k)
            if rng.random() < 0.5:
                keep = int(rng.integers(0, k + 1))
                rc = lib.cf_sequence_speculation_commit(c, i64(seq), C.c_uint64(spec), keep, None)
                log.append(("spec commit", seq, k, keep))
                assert rc == 0, ("commit", err(), log[-6:])
                seqs[seq]["rows"] = [[a[:n0 + keep] for a in seqs[seq]["rows"][layer]] for layer in range(LAYERS)]
            else:
                rc = lib.cf_sequence_speculation_rollback(c, i64(seq), C.c_uint64(spec), None)
                log.append(("spec rollback", seq, k))
                assert rc == 0, ("rollback", err(), log[-6:])
                seqs[seq]["rows"] = before
        elif op == "reclaim":
            if rng.random() < 0.5: torch.cuda.synchronize()
            assert lib.cf_multisequence_reclaim_async(c, None) == 0 and lib.cf_multisequence_audit(c) == 0, (err(), log[-6:])
            log.append(("reclaim",))
        if len(pending) >= 3 or (pending and rng.random() < 0.3): settle()
    settle()
    k = MultisequenceCounters()
    lib.cf_multisequence_get_counters(c, C.byref(k))
    assert k.invariant_failures == 0, log[-6:]
    for seq in list(seqs):
        assert lib.cf_sequence_remove_async(c, i64(seq), i64(-1), i64(-1), None) == 0
    torch.cuda.synchronize()
    assert lib.cf_multisequence_reclaim_async(c, None) == 0 and lib.cf_multisequence_audit(c) == 0
    lib.cf_multisequence_get_counters(c, C.byref(k))
    assert k.active_sequences == 0 and k.pages_pending_reclamation == 0 and k.invariant_failures == 0, (k.active_sequences, k.pages_pending_reclamation)
    lib.cf_multisequence_destroy(c, None)
    return len(log)


@pytest.mark.parametrize("first", range(0, 24, 8))
def test_random_operations_on_the_multisequence_cache(native, oracle, first):
    """cf_sequence_create / append (fp16, bf16, fp32 rows) / copy over ranges / suffix and whole removal / shift /
    speculation commit and rollback / reclaim with audit / batched attention (decode items and short prefill items), in
    random order on up to six sequences.
    More than half of the attention batches are checked only after the operations that follow them (removals, reclaim,
    new pages that may take freed arena slots), against the rows the sequences had when the batch was launched."""
    for seed in range(3000 + first, 3000 + first + 8):
        assert _multisequence_run(native, oracle, seed, 100) > 0


# ---- the llama.cpp KV adapter ABI: pages in the reference's own format -------------------------------------------------
def _adapter_rows(rng, shape):
    """Rows [kv head][token][channel]: plain normal, one magnitude, a magnitude per token, per channel, zero channels and
    zero tokens, or many rounding ties."""
    kind = int(rng.integers(0, 6))
    x = rng.standard_normal(shape)
    if kind == 1: x *= 10.0 ** rng.uniform(-6, 4)
    elif kind == 2: x *= 10.0 ** rng.uniform(-5, 3, (shape[0], shape[1], 1))      # per token
    elif kind == 3: x *= 10.0 ** rng.uniform(-5, 3, (shape[0], 1, shape[2]))      # per channel
    elif kind == 4: x[:, :, rng.integers(0, shape[2], 3)] = 0.0; x[:, rng.integers(0, shape[1], 2), :] = 0.0
    elif kind == 5: x = np.rint(x * 3) * 0.5   # many ties
    return x.astype(np.float32)


def _adapter_case(native, oracle, seed):
    import ctypes as C
    import torch
    from compat_types import DevicePage, LlamaKvOptions, LlamaKvStats
    from test_gpu_compat import _dev, _read_device, _softmax_attention
    rng = np.random.default_rng(seed)
    ref = oracle.ref_cpu(); lib = native.lib()
    lib.cf_llama_kv_create.restype = C.c_void_p; lib.cf_llama_kv_last_error.restype = C.c_char_p
    hq, hkv = [(14, 2), (8, 8), (4, 2), (32, 8), (16, 2), (1, 1)][int(rng.integers(0, 6))]
    head_dim = int(rng.choice([32, 64, 96, 128, 128, 48, 80, 16]))
    page = int(rng.choice([16, 32, 64])); bits = int(rng.choice([4, 8])); layers = int(rng.integers(1, 3))
    tokens = int(rng.integers(1, 4 * page + 10))
    o = LlamaKvOptions()
    o.struct_size, o.backend = C.sizeof(o), 1
    o.layer_count, o.kv_head_count, o.query_head_count, o.head_dim, o.page_size, o.gqa_group_size = layers, hkv, hq, head_dim, page, hq // hkv
    o.kv_bits = bits if bits == 8 else int(rng.choice([0, 4, 5]))
    a = C.c_void_p(lib.cf_llama_kv_create(C.byref(o)))
    what = dict(seed=seed, heads=(hq, hkv), d=head_dim, page=page, bits=bits, layers=layers, tokens=tokens)
    if not a.value: return ("create refused",), what
    k = np.stack([_adapter_rows(rng, (hkv, tokens, head_dim)) for _ in range(layers)]); v = np.stack([_adapter_rows(rng, (hkv, tokens, head_dim)) for _ in range(layers)])
    p = lambda x: np.ascontiguousarray(x).ctypes.data_as(C.c_void_p)
    cuts = sorted(set([0, tokens] + [int(x) for x in rng.integers(0, tokens + 1, int(rng.integers(0, 4)))]))
    for layer in range(layers):
        for b, e in zip(cuts[:-1], cuts[1:]):
            for h in range(hkv):
                rc = lib.cf_llama_kv_append(a, layer, h, b, p(k[layer, h, b:e]), p(v[layer, h, b:e]), e - b, None)
                if rc != 0: return ("append", rc, lib.cf_llama_kv_last_error(a)), what
    full = tokens // page
    st = LlamaKvStats()
    assert lib.cf_llama_kv_get_stats(a, C.byref(st)) == 0
    if st.sealed_pages != layers * hkv * full or st.active_tokens != layers * hkv * (tokens - full * page):
        return ("stats", st.sealed_pages, st.active_tokens), what
    deq_k, deq_v = k.copy(), v.copy()
    n = page * head_dim; words, nb = (n * bits + 31) // 32, (n + 63) // 64
    for layer in range(layers):
        for index in range(hkv * full):
            pg = DevicePage()
            if lib.cf_b200_llama_kv_reference_page(a, layer, index, C.byref(pg)) != 0: return ("page lookup", layer, index), what
            h, begin = pg.kv_head, pg.token_begin
            kw, vw = np.zeros(words + 1, np.uint32), np.zeros(words + 1, np.uint32)
            ko, vo = np.zeros(nb, np.int32), np.zeros(nb, np.int32)
            lut = np.zeros(1 << bits, np.int32)
            ks, vs = np.zeros(head_dim, np.float32), np.zeros(page, np.float32)
            dk, dv = np.zeros(n, np.float32), np.zeros(n, np.float32)
            rk, rv = k[layer, h, begin:begin + page].ravel(), v[layer, h, begin:begin + page].ravel()
            assert ref.ref_fixture_encode(p(rk), p(rv), C.c_uint32(begin), C.c_uint32(page), C.c_uint32(head_dim), C.c_uint32(h),
                                          C.c_uint32(64), C.c_uint32(bits), p(kw), p(ko), p(vw), p(vo), p(lut), p(ks), p(vs), p(dk), p(dv), None) == 0
            checks = [("k words", _read_device(pg.k_words, words, np.uint32), kw[:words]), ("v words", _read_device(pg.v_words, words, np.uint32), vw[:words]),
                      ("k scales", _read_device(pg.k_scales, head_dim, np.float32).view(np.uint32), ks.view(np.uint32)),
                      ("v scales", _read_device(pg.v_scales, page, np.float32).view(np.uint32), vs.view(np.uint32)),
                      ("k offsets", _read_device(pg.k_block_offsets, nb, np.int32), ko)]
            for name, got, want in checks:
                if not np.array_equal(got, want):
                    i = int(np.argmax(got != want)); return (name, layer, index, i, int(got[i]), int(want[i])), what
            deq_k[layer, h, begin:begin + page] = dk.reshape(page, head_dim); deq_v[layer, h, begin:begin + page] = dv.reshape(page, head_dim)
    nq = int(rng.integers(1, min(4, tokens) + 1)); window = int(rng.integers(1, tokens + 4)) if rng.random() < 0.5 else 0
    q = rng.standard_normal((nq, hq, head_dim)).astype(np.float32)
    pos = [tokens - nq + i for i in range(nq)]
    d_q = _dev(q)
    for layer in range(layers):
        out = torch.zeros((nq, hq, head_dim), dtype=torch.float32, device="cuda")
        rc = lib.cf_llama_kv_attention(a, layer, C.c_void_p(d_q.data_ptr()), C.c_void_p(out.data_ptr()), nq, hq, hq // hkv,
                                       tokens - nq, C.c_float(1.0 / np.sqrt(head_dim)), window, None)
        if rc != 0: return ("attention rc", rc, lib.cf_llama_kv_last_error(a)), what
        torch.cuda.synchronize()
        want = _softmax_attention(deq_k[layer], deq_v[layer], q, pos, [max(0, x + 1 - window) if window else 0 for x in pos], 1.0 / np.sqrt(head_dim), hq // hkv)
        got = out.cpu().numpy()
        e = np.abs(got - want).max() / (np.abs(want).max() + 1e-30)
        if not np.isfinite(got).all() or e > 2e-4: return ("attention", layer, float(e)), what
    lib.cf_llama_kv_destroy(a)
    return None, what


@pytest.mark.parametrize("first", range(0, 60, 20))
def test_random_adapter_cases_store_the_references_own_pages(native, oracle, first, monkeypatch):
    """cf_llama_kv_* with the default page format on random shapes (heads, head_dim 16..128, page 16 / 32 / 64, int4 or
    int8, append chunking): every sealed page equals the reference encoder's (oracle/_ref) bit for bit — words, fp32
    scales, block offsets — and attention matches fp64 softmax over the reference's dequantised rows."""
    if oracle.ref_cpu() is None:
        pytest.skip("the reference's encoder was not built (oracle/_ref)")
    monkeypatch.delenv("CHROMOFOLD_B200_CODER", raising=False)
    for seed in range(4000 + first, 4000 + first + 20):
        bad, what = _adapter_case(native, oracle, seed)
        assert bad is None, (bad, what)


# ---- the flat-stream entry points of the reference's first ABI ----------------------------------------------------------
def _flat_rans_case(native, oracle, seed):
    import ctypes as C
    import torch
    from helpers import hist_of, laplace_codes
    from test_gpu_compat import _dev, _softmax_attention
    rng = np.random.default_rng(seed)
    block = int(rng.choice([64, 64, 64, 32, 100, 128, 256, 1024, 1, 7]))
    n = int(rng.choice([1, 63, 64, 65, 4096, 4097, 64 * 64, 64 * 64 + 1, 64 * 65, int(rng.integers(1, 300000))]))
    b = float(10.0 ** rng.uniform(-1.5, 1.8))
    sym = (laplace_codes(rng, n, b).astype(np.int16) + 128).astype(np.uint8)
    if rng.random() < 0.2: sym[:] = sym[0]
    hist = hist_of(sym) if rng.random() < 0.7 else hist_of((laplace_codes(rng, 4096, 20.0).astype(np.int16) + 128).astype(np.uint8)) + 1
    cb = oracle.codebook_from_hist(hist)
    data, off, st = oracle.rans_encode(sym, block, cb)
    args = [_dev(np.concatenate([data, np.zeros(8, np.uint8)])), _dev(off), _dev(st), _dev(cb.np("slot2sym")), _dev(cb.np("freq")), _dev(cb.np("cum"))]
    outs = []
    for lib in (native.lib(), oracle.ref_cuda()):
        out = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        rc = lib.cf_rans_decode_async(*[C.c_void_p(t.data_ptr()) for t in args], C.c_int(block), C.c_int(n), C.c_void_p(out.data_ptr()), None)
        torch.cuda.synchronize()
        outs.append((rc, out.cpu().numpy()))
    what = dict(kind="rans", seed=seed, block=block, n=n, b=b)
    if outs[0][0] != outs[1][0]: return ("rc", outs[0][0], outs[1][0]), what
    if outs[0][0] == 0 and not np.array_equal(outs[0][1], sym.astype(np.int32)): return ("symbols", int(np.argmax(outs[0][1] != sym)),), what
    if outs[0][0] == 0 and not np.array_equal(outs[0][1], outs[1][1]): return ("vs reference",), what
    return None, what


def _flat_fused_case(native, oracle, seed):
    import ctypes as C
    import torch
    from helpers import hist_of, laplace_codes
    from test_gpu_compat import _dev, _softmax_attention
    rng = np.random.default_rng(seed)
    seq = int(rng.integers(1, 400)); dim = int(rng.choice([16, 32, 40, 64, 80, 97, 128])); nq = int(rng.integers(1, seq + 1))
    nq = min(nq, 64); window = int(rng.integers(1, 513)); block = int(rng.choice([16, 32, 64, 100, 128]))
    ksym = (laplace_codes(rng, seq * dim, float(rng.uniform(1, 30))).astype(np.int16) + 128).astype(np.uint8)
    vsym = (laplace_codes(rng, seq * dim, float(rng.uniform(1, 30))).astype(np.int16) + 128).astype(np.uint8)
    kcb, vcb = oracle.codebook_from_hist(hist_of(ksym)), oracle.codebook_from_hist(hist_of(vsym))
    kw, kb = oracle.huff_encode(ksym, block, kcb); vw, vb = oracle.huff_encode(vsym, block, vcb)
    kscale = (rng.uniform(0.005, 0.02, dim) * 10.0 ** rng.uniform(-1, 1)).astype(np.float32)
    vscale = (rng.uniform(0.005, 0.02, seq) * 10.0 ** rng.uniform(-3, 2, seq)).astype(np.float32)
    q = rng.standard_normal((nq, dim)).astype(np.float32)
    sscale = 1.0 / np.sqrt(dim)
    kd = (ksym.astype(np.float32).reshape(seq, dim) - 128.0) * kscale[None, :]
    vd = (vsym.astype(np.float32).reshape(seq, dim) - 128.0) * vscale[:, None]
    positions = np.arange(nq); firsts = np.maximum(0, positions - window + 1)
    expect = _softmax_attention(kd[None], vd[None], q[:, None, :], positions, firsts, sscale, 1)[:, 0]
    pad = np.zeros(2, np.uint32)
    dev = [_dev(np.concatenate([kw, pad])), _dev(kb), _dev(kcb.np("lut")), _dev(np.concatenate([vw, pad])), _dev(vb), _dev(vcb.np("lut")), _dev(kscale), _dev(vscale), _dev(q)]
    p = [C.c_void_p(t.data_ptr()) for t in dev]
    res = []
    what = dict(kind="fused", seed=seed, seq=seq, dim=dim, nq=nq, window=window, block=block)
    for lib in (native.lib(), oracle.ref_cuda()):
        fused = torch.zeros((nq, dim), dtype=torch.float32, device="cuda"); dense = torch.zeros_like(fused)
        kdd = torch.zeros((seq, dim), dtype=torch.float32, device="cuda"); vdd = torch.zeros_like(kdd)
        tail = (C.c_int(seq), C.c_int(dim), C.c_int(nq), C.c_int(window), C.c_int(block), C.c_int(128), C.c_float(sscale), None)
        head = (p[0], p[1], p[2], C.c_int(12), p[3], p[4], p[5], C.c_int(12), p[6], p[7], p[8])
        rc1 = lib.cf_kv_attn_fused_async(*head, C.c_void_p(fused.data_ptr()), *tail)
        rc2 = lib.cf_kv_attn_dense_async(*head, C.c_void_p(kdd.data_ptr()), C.c_void_p(vdd.data_ptr()), C.c_void_p(dense.data_ptr()), *tail)
        torch.cuda.synchronize()
        res.append((rc1, rc2, fused.cpu().numpy(), dense.cpu().numpy(), kdd.cpu().numpy(), vdd.cpu().numpy()))
    if res[0][:2] != res[1][:2]: return ("rc", res[0][:2], res[1][:2]), what
    if res[0][0] != 0: return None, what
    if not np.array_equal(res[0][2], res[0][3]): return ("fused != dense",), what
    if not (np.array_equal(res[0][4], kd) and np.array_equal(res[0][5], vd)): return ("dequantised rows",), what
    scale = np.abs(expect).max() + 1e-30
    if np.abs(res[0][2] - expect).max() / scale > 2e-4: return ("vs fp64", float(np.abs(res[0][2] - expect).max() / scale), "ref", float(np.abs(res[1][2] - expect).max() / scale)), what
    return None, what


@pytest.mark.parametrize("first", range(0, 40, 20))
def test_random_flat_stream_cases(native, oracle, first):
    """cf_rans_decode_async and cf_kv_attn_fused_async / cf_kv_attn_dense_async on random sizes, block sizes (1 and 7
    included), codebooks that were not made from the stream, constant streams and per-token V scales over five orders:
    symbols exact, fused == dense bit for bit, the same status and the same symbols as the reference's kernels."""
    if oracle.ref_cuda() is None:
        pytest.skip("needs the reference's kernels (oracle/_ref)")
    for seed in range(5000 + first, 5000 + first + 20):
        for case in (_flat_rans_case, _flat_fused_case):
            bad, what = case(native, oracle, seed)
            assert bad is None, (bad, what)


# ---- the shared-prefix kernel at larger batch sizes ---------------------------------------------------------------------
def _prefix_case(native, seed):
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    rng = np.random.default_rng(seed)
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    n = int(rng.choice([1, 2, 7, 31, 32, 33, 64, 100, 129, 257, int(rng.integers(1, 300))]))
    hq, hkv = [(32, 8), (16, 8), (8, 8), (64, 8), (8, 2), (4, 1), (16, 1), (2, 2)][int(rng.integers(0, 8))]
    group = hq // hkv
    coder = ["rans4", "huffman4", "rans", "huffman", "fixed8"][int(rng.integers(0, 5))]
    pp = int(rng.choice([1, 2, 7, 8, 9, 16, 17, 40, int(rng.integers(1, 60))]))
    private = int(rng.integers(0, 40))
    layer, info = build_sealed_layer(np.array([16 * pp] + [0] * (n - 1)), query_heads=hq, kv_heads=hkv, coder=coder, seed=seed,
                                     extra_pages_per_sequence=private // 16 + 3, reserve_pages=n * (private // 16 + 2) + 8)
    for s in range(1, n): layer.copy_sequence(0, s)
    slots = list(range(n))
    ragged = rng.random() < 0.5
    for t in range(private):
        sl = [s for s in slots if (not ragged) or (s * 7 + 3) % (private + 1) > t] or [0]
        k = (torch.randn((len(sl), hkv, 128), generator=g, device="cuda") * 0.7).half()
        v = (torch.randn((len(sl), hkv, 128), generator=g, device="cuda") * 0.7).half()
        layer.append(sl, k, v); layer.seal_full_pages()
    q = (torch.randn((n, hq, 128), generator=g, device="cuda")).half()
    kw = {}
    if rng.random() < 0.4:
        span = int(rng.integers(1, hkv + 1)); kw["kv_head_begin"], kw["kv_head_span"] = int(rng.integers(0, hkv - span + 1)), span
    qq = q.float() if rng.random() < 0.3 else q
    claim = pp if rng.random() < 0.7 else int(rng.integers(1, pp + 1))
    a = torch.full((n, hq, 128), 7.0, dtype=torch.float32, device="cuda"); b = torch.full((n, hq, 128), 7.0, dtype=torch.float32, device="cuda")
    before = native.lib().cf_b200_shared_prefix_launches()
    layer.attention(qq, out=a, kernel=native.KERNEL_LANES, shared_prefix_pages=claim, **kw)
    used = native.lib().cf_b200_shared_prefix_launches() - before
    st = layer.device_status()
    layer.attention(qq, out=b, kernel=native.KERNEL_LANES, **kw)
    A, B = a.cpu().numpy().astype(np.float64), b.cpu().numpy().astype(np.float64)
    err = np.abs(A - B).max() / (np.abs(B).max() + 1e-30)
    what = dict(seed=seed, n=n, heads=(hq, hkv), coder=coder, prefix_pages=pp, claim=claim, private=private, ragged=ragged, kw=kw, used=int(used))
    if st != 0 or not np.isfinite(A).all() or err > 2e-5: return (st, float(err)), what
    if 128 % group == 0 and used != 1: return ("prefix kernel not used",), what
    return None, what


@pytest.mark.parametrize("first", range(0, 40, 20))
def test_random_shared_prefix_cases(native, first):
    """The shared-prefix kernel on batches of 1 to 300 sequences (one to several row tiles, the last one partly filled),
    1 to 60 shared pages (whole and ragged rounds), heads from 2 x 2 to 64 x 8, private tails of equal or ragged
    length, kv-head shards, fp32 queries, partial claims: equal to the per-sequence path to 2e-5 of the output's
    scale, and the kernel did run."""
    for seed in range(6000 + first, 6000 + first + 20):
        bad, what = _prefix_case(native, seed)
        assert bad is None, (bad, what)


# ---- longer contexts, larger query groups ---------------------------------------------------------------------------
def _long_case(native, seed):
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    rng = np.random.default_rng(seed)
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    n = int(rng.integers(1, 9))
    D, block = [(128, 64), (128, 64), (128, 128), (128, 256), (64, 64), (96, 64), (32, 64), (64, 128), (96, 128)][int(rng.integers(0, 9))]
    hq, hkv = [(32, 8), (64, 8), (8, 8), (128, 8), (16, 2), (12, 4), (40, 8)][int(rng.integers(0, 7))]
    coder = ["rans4", "huffman4", "rans", "huffman", "fixed8"][int(rng.integers(0, 5))]
    ctx = (rng.integers(0, 400, n) * 16)
    if rng.random() < 0.3: ctx[int(rng.integers(0, n))] = 0
    dist = ("laplace", float(rng.uniform(2, 30))) if rng.random() < 0.7 else ("geometric", float(rng.uniform(0.05, 0.7)))
    layer, info = build_sealed_layer(ctx, query_heads=hq, kv_heads=hkv, head_dim=D, block_size=block, coder=coder, dist=dist, seed=seed,
                                     extra_pages_per_sequence=3, reserve_pages=2 * n)
    if ctx.sum() == 0: layer.set_codebooks(np.ones(256, np.uint64), np.ones(256, np.uint64))
    tail = int(rng.integers(0, 16))
    for t in range(tail):
        sl = [s for s in range(n) if (s + t) % 3 != 0 or t < 2]
        k = (torch.randn((len(sl), hkv, D), generator=g, device="cuda") * 0.3).half(); v = (torch.randn((len(sl), hkv, D), generator=g, device="cuda") * 0.3).half()
        layer.append(sl, k, v)
    q = (torch.randn((n, hq, D), generator=g, device="cuda") * float(10.0 ** rng.uniform(-0.5, 0.5))).half()
    kw = {}
    if rng.random() < 0.4: kw["min_pages_per_unit"] = int(rng.choice([1, 2, 3, 5, 8, 16, 33, 64, 200]))
    if rng.random() < 0.3: kw["causal_window"] = int(rng.integers(1, 3000))
    if rng.random() < 0.3:
        span = int(rng.integers(1, hkv + 1)); kw["kv_head_begin"], kw["kv_head_span"] = int(rng.integers(0, hkv - span + 1)), span
    qq = q.float() if rng.random() < 0.3 else q
    out = torch.full((n, hq, D), 7.0, dtype=torch.float32, device="cuda")
    layer.attention(qq, out=out, kernel=native.KERNEL_LANES, **kw)
    st = layer.device_status()
    got = out.cpu().numpy()
    want = oracle_from_layer(layer, q.cpu().numpy(), causal_window=kw.get("causal_window", 0))
    group = hq // hkv
    lo = kw.get("kv_head_begin", 0) * group; hi = lo + kw.get("kv_head_span", hkv) * group
    a, e = got[:, lo:hi].astype(np.float64), want[:, lo:hi].astype(np.float64)
    err = np.abs(a - e).max() / (np.abs(e).max() + 1e-30)
    what = dict(seed=seed, n=n, D=D, block=block, heads=(hq, hkv), coder=coder, ctx=ctx.tolist(), tail=tail, kw=kw, dist=dist)
    untouched = np.all(got[:, :lo] == 7.0) and np.all(got[:, hi:] == 7.0)
    if st != 0 or not np.isfinite(a).all() or err > 1e-4 or not untouched: return (st, float(err), bool(untouched)), what
    return None, what


@pytest.mark.parametrize("first", range(0, 40, 20))
def test_random_long_context_cases(native, oracle, first):
    """Contexts of up to 6400 tokens (many chunks per sequence), groups of 1 to 16 query heads per kv head, every fast
    geometry and coder, Laplace and geometric codes, ragged tails, units from 1 page to whole sequences, windows, kv-head
    shards, fp32 queries, against the oracle. The bar is 1e-4 of the output's scale: the fp32 accumulation of the
    tensor cores drifts by about 1e-7 per page of a unit, which shows when a caller asks for units of hundreds of pages
    (2e-5 at 300); the library's own choice keeps units below 36 pages."""
    for seed in range(7000 + first, 7000 + first + 20):
        bad, what = _long_case(native, seed)
        assert bad is None, (bad, what)


# ---- transfer images ----------------------------------------------------------------------------------------------
def _transfer_case(native, seed):
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    rng = np.random.default_rng(seed)
    D, block = [(128, 64), (128, 128), (128, 256), (64, 64), (96, 64), (32, 64)][int(rng.integers(0, 6))]
    hq, hkv = [(32, 8), (8, 2), (4, 4), (16, 1)][int(rng.integers(0, 4))]
    coder = ["rans4", "huffman4", "rans", "huffman", "fixed8"][int(rng.integers(0, 5))]
    pages = int(rng.integers(1, 80)); other = int(rng.integers(0, 5)) * 16
    src, _ = build_sealed_layer(np.array([16 * pages, other]), query_heads=hq, kv_heads=hkv, head_dim=D, block_size=block, coder=coder, seed=seed,
                                dist=("laplace", float(rng.uniform(2, 40))))
    image = src.export_pages(0)
    what = dict(seed=seed, D=D, block=block, heads=(hq, hkv), coder=coder, pages=pages)
    if src.device_status() != 0: return ("export status", src.device_status()), what
    def fresh(seed2):
        pre = int(rng.integers(0, 4)) * 16
        dst, _ = build_sealed_layer(np.array([0, pre]), query_heads=hq, kv_heads=hkv, head_dim=D, block_size=block, coder=coder, seed=seed2,
                                    extra_pages_per_sequence=pages + 4, reserve_pages=pages + 8)
        dst.k_tables.copy_(src.k_tables); dst.v_tables.copy_(src.v_tables); dst.host_tables = src.host_tables; dst.codebook_id = src.codebook_id
        dst._codebooks_set = True
        return dst
    dst = fresh(seed + 1)
    if dst.import_pages(0, image) != pages or dst.device_status() != 0: return ("import", dst.device_status()), what
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    q = torch.randn((1, hq, D), generator=g, device="cuda").half()
    a = src.attention(q, slots=[0]).cpu().numpy(); b = dst.attention(q, slots=[0]).cpu().numpy()
    if not np.array_equal(a, b): return ("attention differs", float(np.abs(a - b).max())), what
    for h in range(hkv):
        for pg in (0, pages - 1):
            if not np.array_equal(src.record_bytes(int(src.h_page_table[0, pg]), h), dst.record_bytes(int(dst.h_page_table[0, pg]), h)): return ("record differs", pg, h), what
    # tampering: flip one to three bits somewhere in the payload
    header = native.TransferHeader.from_buffer_copy(image[:64])
    man_bytes = 16 * pages * hkv
    man = np.frombuffer(image[64:64 + man_bytes], dtype=[("off", "<u4"), ("len", "<u4"), ("sum", "<u8")])
    for trial in range(3):
        bad = bytearray(image)
        e = man[int(rng.integers(0, man.size))]
        for _ in range(int(rng.integers(1, 4))):
            at = 64 + man_bytes + 16 * int(e["off"]) + int(rng.integers(0, 16 * int(e["len"])))
            bad[at] ^= 1 << int(rng.integers(0, 8))
        if bytes(bad) == image: continue
        d2 = fresh(seed + 2 + trial)
        d2.import_pages(0, bytes(bad))
        if not (d2.device_status() & native.DEVSTAT_CHECKSUM): return ("tampering not caught", trial), what
    return None, what


@pytest.mark.parametrize("first", range(0, 30, 15))
def test_random_transfer_images(native, first):
    """Transfer images of 1 to 79 pages in every fast geometry and coder: the importing store holds the same record bytes
    and answers attention bit for bit like the exporting one; one to three flipped payload bits are always caught by the
    per-record checksum."""
    for seed in range(8000 + first, 8000 + first + 15):
        bad, what = _transfer_case(native, seed)
        assert bad is None, (bad, what)


# ---- the device dataplane ABI -----------------------------------------------------------------------------------------
def _record_tokens(page, d):
    """Tokens per record the stores behind the reference's device ABIs choose (engine_common.cuh)."""
    if d in (128, 96, 64, 32) and page % 16 == 0: return 16
    limit = 4096 // d
    for t in range(min(page, limit), 0, -1):
        if page % t == 0: return t
    return 1


def _dataplane_case(native, oracle, seed):
    import ctypes as C
    import torch
    from compat_types import DeviceKvConfig, DeviceKvCounters, TensorView
    from test_gpu_device_engine import _expected
    rng = np.random.default_rng(seed)
    lib = native.lib(); lib.cf_device_kv_create.restype = C.c_void_p; lib.cf_device_kv_last_error.restype = C.c_char_p
    layers = int(rng.integers(1, 3)); hkv = int(rng.choice([1, 2, 4, 8])); group = int(rng.choice([1, 2, 4, 7])); hq = hkv * group
    d = int(rng.choice([32, 64, 96, 128, 128, 48, 80])); page = int(rng.choice([16, 32, 64, 24]))
    p = C.c_void_p(lib.cf_device_kv_create(C.byref(DeviceKvConfig(layers, hkv, hq, d, page, group, 0))))
    what = dict(seed=seed, layers=layers, heads=(hq, hkv), d=d, page=page)
    if not p.value: return ("create refused",), what
    dtype = ["f16", "bf16", "f32"][int(rng.integers(0, 3))]
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dtype]; code = {"f16": 1, "bf16": 2, "f32": 3}[dtype]; width = 2 if dtype != "f32" else 4
    tokens = int(rng.integers(1, 5 * page)); base = int(rng.choice([0, 0, 1000, 17]))
    pad = int(rng.choice([0, 8]))
    what.update(dtype=dtype, tokens=tokens, base=base)
    ks, vs = [], []
    for layer in range(layers):
        k_src = torch.from_numpy((rng.standard_normal((tokens, hkv, d + pad)) * 10.0 ** rng.uniform(-2, 1)).astype(np.float32)).cuda().to(tdt)
        v_src = torch.from_numpy((rng.standard_normal((tokens, hkv, d + pad)) * 10.0 ** rng.uniform(-3, 2)).astype(np.float32)).cuda().to(tdt)
        ks.append(k_src); vs.append(v_src)
        def view(t, begin, count): return TensorView(t[begin:].data_ptr(), code, count, hkv, d, hkv * (d + pad) * width, (d + pad) * width, width, 0)
        at = 0
        while at < tokens:
            room = page - at % page
            count = min(tokens - at, int(rng.integers(1, room + 1)))
            rc = lib.cf_device_kv_append_async(p, layer, base + at, C.byref(view(k_src, at, count)), C.byref(view(v_src, at, count)), None)
            if rc != 0: return ("append", at, count, lib.cf_device_kv_last_error(p)), what
            at += count
            if at % page == 0 or rng.random() < 0.2:
                if lib.cf_device_kv_seal_full_pages_async(p, None) != 0: return ("seal", lib.cf_device_kv_last_error(p)), what
    sealed = tokens // page * page
    nq = int(rng.integers(1, min(4, tokens) + 1)); window = int(rng.integers(1, tokens + 3)) if rng.random() < 0.4 else 0
    scale = 1.0 / np.sqrt(d)
    q = rng.standard_normal((nq, hq, d)).astype(np.float32); dq = torch.from_numpy(q).cuda()
    for layer in range(layers):
        out = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda")
        rc = lib.cf_device_kv_attention_async(p, layer, C.c_void_p(dq.data_ptr()), C.c_void_p(out.data_ptr()), nq, base + tokens - nq, C.c_float(scale), window, None)
        if rc != 0: return ("attention rc", lib.cf_device_kv_last_error(p)), what
        torch.cuda.synchronize()
        k = ks[layer][:, :, :d].float().cpu().numpy(); v = vs[layer][:, :, :d].float().cpu().numpy()
        want = _expected(oracle, k, v, sealed, _record_tokens(page, d), q, [tokens - nq + i for i in range(nq)], window, scale, group)
        got = out.cpu().numpy()
        e = np.abs(got - want).max() / (np.abs(want).max() + 1e-30)
        if not np.isfinite(got).all() or e > 2e-4: return ("attention", layer, float(e)), what
    n = DeviceKvCounters(); lib.cf_device_kv_get_counters(p, C.byref(n))
    if n.dense_fallback_launches != 0: return ("dense fallback",), what
    lib.cf_device_kv_destroy(p, None)
    return None, what


@pytest.mark.parametrize("first", range(0, 40, 20))
def test_random_dataplane_cases(native, oracle, first):
    """cf_device_kv_* on random shapes (1-2 layers, 1-8 kv heads, groups of 1-7, head_dim 32..128 with 48 and 80, pages of
    16 / 24 / 32 / 64 tokens), fp16 / bf16 / fp32 strided rows appended in random pieces from position 0, 17 or 1000,
    sealing as pages fill, one to four query rows with or without a window: fp64 softmax over the engine's quantisation
    of the sealed rows, at the reference's 2e-4."""
    for seed in range(9000 + first, 9000 + first + 20):
        bad, what = _dataplane_case(native, oracle, seed)
        assert bad is None, (bad, what)


# ---- the batched decode runtime ABI -----------------------------------------------------------------------------------
def _runtime_int4_page(rng, tokens, token_begin, keep, HKV, D, BLOCK, wild):
    """One page as the reference's seal engine writes it (src/cuda/device_kv_seal_attention.cu:80-134)."""
    import torch
    from compat_types import PageDescriptor
    desc, dense = PageDescriptor(), []
    for name in ("key", "value"):
        x = rng.standard_normal((tokens, HKV, D)).astype(np.float32)
        if wild: x *= (10.0 ** rng.uniform(-3, 2, (tokens, 1, 1))).astype(np.float32)
        blocks = x.reshape(-1, BLOCK)
        scale = (np.abs(blocks).max(axis=1) / 7.0).astype(np.float32)
        scale[scale == 0] = 1.0
        q = np.clip(np.rint(blocks / scale[:, None]), -7, 7).astype(np.int32)
        dense.append((q.astype(np.float32) * scale[:, None]).reshape(tokens, HKV, D))
        nib = (q + 8).astype(np.uint8).reshape(-1)
        payload = (nib[0::2] | (nib[1::2] << 4)).astype(np.uint8)
        p, s = torch.from_numpy(payload).cuda(), torch.from_numpy(scale).cuda()
        keep += [p, s]
        setattr(desc, name + "_payload", p.data_ptr()); setattr(desc, name + "_scales", s.data_ptr()); setattr(desc, name + "_payload_bytes", payload.size)
    desc.token_begin, desc.token_count, desc.kv_head_count, desc.head_dim = token_begin, tokens, HKV, D
    desc.block_size, desc.blocks_per_page = BLOCK, tokens * HKV * D // BLOCK
    return desc, dense[0], dense[1]


def _runtime_case(native, seed):
    import ctypes as C
    import torch
    from compat_types import AttentionBatchItem, AttentionCounters, AttentionRuntimeConfig, PageDescriptor, TensorView
    rng = np.random.default_rng(seed)
    lib = native.lib(); lib.cf_attention_runtime_create.restype = C.c_void_p; lib.cf_attention_last_error.restype = C.c_char_p
    HKV = int(rng.choice([1, 2, 4, 8])); G = int(rng.choice([1, 2, 4, 7])); HQ = HKV * G
    D = int(rng.choice([32, 64, 96, 128, 80])); BLOCK = int(rng.choice([16, 32, 64])); PAGE = int(rng.choice([16, 32, 64]))
    if D % BLOCK and BLOCK % D: BLOCK = 16
    mode = int(rng.integers(0, 2)); layers = int(rng.integers(1, 4))
    cfg = AttentionRuntimeConfig()
    cfg.layer_count, cfg.query_head_count, cfg.kv_head_count, cfg.head_dim = layers, HQ, HKV, D
    cfg.page_size, cfg.block_size, cfg.gqa_group_size, cfg.mode = PAGE, BLOCK, G, mode
    rt = C.c_void_p(lib.cf_attention_runtime_create(C.byref(cfg)))
    what = dict(seed=seed, heads=(HQ, HKV), D=D, BLOCK=BLOCK, PAGE=PAGE, mode=mode, layers=layers)
    if not rt.value: return ("create refused",), what
    n = int(rng.integers(1, 7)); wild = rng.random() < 0.4
    keep, items, expected, outputs = [], (AttentionBatchItem * n)(), [], []
    scale = 1.0 / np.sqrt(D)
    cases = []
    for i in range(n):
        pages = int(rng.integers(0, 11)); tail = int(rng.integers(0, PAGE))
        if pages + tail == 0: tail = 1
        window = int(rng.integers(1, pages * PAGE + tail + 3)) if rng.random() < 0.4 else 0
        qdt = [torch.float32, torch.float16, torch.bfloat16][int(rng.integers(0, 3))]; odt = [torch.float32, torch.float16][int(rng.integers(0, 2))]
        cases.append((pages, tail, window, str(qdt), str(odt)))
        descs = (PageDescriptor * max(pages, 1))(); ks, vs = [], []
        for pg in range(pages):
            descs[pg], k, v = _runtime_int4_page(rng, PAGE, pg * PAGE, keep, HKV, D, BLOCK, wild); ks.append(k); vs.append(v)
        tk = rng.standard_normal((tail, HKV, D)).astype(np.float32); tv = rng.standard_normal((tail, HKV, D)).astype(np.float32)
        ks.append(tk); vs.append(tv)
        k_all, v_all = np.concatenate(ks), np.concatenate(vs)
        qpos = pages * PAGE + tail - 1
        q = torch.from_numpy(rng.standard_normal((HQ, D)).astype(np.float32)).to(qdt).cuda()
        out = torch.zeros((HQ, D), dtype=odt, device="cuda")
        d_desc = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
        d_tk, d_tv = torch.from_numpy(np.ascontiguousarray(tk)).cuda(), torch.from_numpy(np.ascontiguousarray(tv)).cuda()
        keep += [q, out, d_desc, d_tk, d_tv]
        it = items[i]
        it.sequence_id, it.layer = 100 + i, int(rng.integers(0, layers))
        esz = q.element_size()
        it.query = TensorView(q.data_ptr(), {torch.float16: 1, torch.bfloat16: 2, torch.float32: 3}[qdt], 1, HQ, D, HQ * D * esz, D * esz, esz, 0)
        it.output, it.output_type = out.data_ptr(), {torch.float16: 1, torch.float32: 3}[odt]
        osz = out.element_size()
        it.output_token_stride_bytes, it.output_head_stride_bytes, it.output_element_stride_bytes = HQ * D * osz, D * osz, osz
        it.query_token_begin, it.softmax_scale, it.causal_window = qpos, scale, window
        it.sealed_pages, it.sealed_page_count = (d_desc.data_ptr() if pages else None), pages
        it.active_keys, it.active_values = (d_tk.data_ptr() if tail else None), (d_tv.data_ptr() if tail else None)
        it.active_token_begin, it.active_token_count = pages * PAGE, tail
        first = 0 if window == 0 else max(0, qpos + 1 - window)
        qf = q.float().cpu().numpy(); exp = np.zeros((HQ, D))
        for h in range(HQ):
            kv = h // G
            s = (k_all[first:qpos + 1, kv].astype(np.float64) @ qf[h].astype(np.float64)) * scale
            w = np.exp(s - s.max()); exp[h] = (w[:, None] * v_all[first:qpos + 1, kv]).sum(0) / w.sum()
        expected.append(exp); outputs.append(out)
    what["cases"] = cases; what["wild"] = wild
    rc = lib.cf_attention_execute_async(rt, items, n, None)
    if rc != 0: return ("execute", lib.cf_attention_last_error(rt)), what
    torch.cuda.synchronize()
    for i, (out, exp) in enumerate(zip(outputs, expected)):
        got = out.float().cpu().numpy()
        tol = 2e-3 if out.dtype == torch.float16 else 2e-4
        e = np.abs(got - exp).max() / (np.abs(exp).max() + 1e-30)
        if not np.isfinite(got).all() or e > tol: return ("item", i, float(e)), what
    c = AttentionCounters(); lib.cf_attention_get_counters(rt, C.byref(c))
    if c.cuda_errors != 0: return ("cuda errors",), what
    lib.cf_attention_runtime_destroy(rt, None)
    return None, what


@pytest.mark.parametrize("first", range(0, 30, 15))
def test_random_batches_through_the_decode_runtime(native, first):
    """cf_attention_execute_async on random configurations (heads, head_dim 32..128 and 80, blocks of 16 / 32 / 64 values,
    pages of 16 / 32 / 64 tokens, both modes) and batches of one to six items (0-10 int4 pages, fp32 tails, windows,
    fp32 / fp16 / bf16 queries, fp32 / fp16 outputs, per-token magnitudes): fp64 softmax over the dequantised rows."""
    for seed in range(9500 + first, 9500 + first + 15):
        bad, what = _runtime_case(native, seed)
        assert bad is None, (bad, what)


# ---- the device sequence resolver ABI under random operations ----------------------------------------------------------
def _resolver_run(native, oracle, seed, steps):
    import ctypes as C
    import torch
    from compat_types import MsBatchItem, MsConfig, MsCounters, MsPublication, PageDescriptor, TensorView
    from test_gpu_ms_resolver import _expected, _int4_page
    rng = np.random.default_rng(seed)
    lib = native.lib(); lib.cf_ms_cuda_create.restype = C.c_void_p; lib.cf_ms_cuda_last_error.restype = C.c_char_p
    layers = int(rng.integers(1, 3)); hkv = int(rng.choice([1, 2, 4])); group = int(rng.choice([1, 2, 4])); hq = hkv * group
    d = int(rng.choice([64, 128, 32, 96])); page = int(rng.choice([16, 32, 64])); block = int(rng.choice([16, 32, 64]))
    r = C.c_void_p(lib.cf_ms_cuda_create(C.byref(MsConfig(layers, hkv, hq, d, page, group, 0))))
    assert r.value
    err = lambda: lib.cf_ms_cuda_last_error(r)
    tile = _record_tokens(page, d)
    keep = []
    seqs = {}   # id -> per layer dict(k, v sealed rows; closed (short last page); tk, tv tail rows)
    next_id = 1; log = []; scale = 1.0 / np.sqrt(d)
    def new_layer(): return dict(k=np.zeros((0, hkv, d), np.float32), v=np.zeros((0, hkv, d), np.float32), closed=False, tk=np.zeros((0, hkv, d), np.float32), tv=np.zeros((0, hkv, d), np.float32))
    def total(L): return L["k"].shape[0] + L["tk"].shape[0]
    for step in range(steps):
        op = ["create", "publish", "publish", "publish", "stage", "stage", "copy", "execute", "execute", "remove", "reclaim"][int(rng.integers(0, 11))]
        live = list(seqs)
        if op == "create" or not live:
            if len(live) >= 5: continue
            assert lib.cf_ms_cuda_sequence_create(r, C.c_int64(next_id)) == 0, err()
            seqs[next_id] = [new_layer() for _ in range(layers)]; log.append(("create", next_id)); next_id += 1
        elif op == "publish":
            s = live[int(rng.integers(0, len(live)))]; layer = int(rng.integers(0, layers)); L = seqs[s][layer]
            if L["closed"] or L["tk"].shape[0] or L["k"].shape[0] > 400: continue
            tokens = page if rng.random() < 0.8 else int(rng.integers(1, page + 1))
            if (tokens * hkv * d) % block: tokens = page
            (kp, ks, kd), (vp, vs, vd) = _int4_page(rng, tokens, hkv, d, block)
            t = [torch.from_numpy(x).cuda() for x in (kp, vp, ks, vs)]; keep.append(t)
            pub = MsPublication(); pub.sequence_id, pub.layer = s, layer
            pub.descriptor = PageDescriptor(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), L["k"].shape[0], tokens, hkv, d,
                                            block, ks.size, kp.size, vp.size, kp.size + vp.size + 8 * ks.size, 1)
            pub.resident_bytes, pub.seal_generation = kp.size + vp.size + 8 * ks.size, 1
            rc = lib.cf_ms_cuda_publish_page_async(r, C.byref(pub), None)
            log.append(("publish", s, layer, tokens))
            assert rc == 0, ("publish", err(), log[-6:])
            L["k"] = np.concatenate([L["k"], kd]); L["v"] = np.concatenate([L["v"], vd]); L["closed"] = tokens < page
        elif op == "stage":
            s = live[int(rng.integers(0, len(live)))]; layer = int(rng.integers(0, layers)); L = seqs[s][layer]
            count = int(rng.integers(1, page))
            tk = rng.standard_normal((count, hkv, d)).astype(np.float32); tv = rng.standard_normal((count, hkv, d)).astype(np.float32)
            dk, dv = torch.from_numpy(tk).cuda(), torch.from_numpy(tv).cuda(); keep.append((dk, dv))
            rc = lib.cf_ms_cuda_stage_active_async(r, C.c_int64(s), layer, L["k"].shape[0], C.c_void_p(dk.data_ptr()), C.c_void_p(dv.data_ptr()), count, None)
            log.append(("stage", s, layer, count))
            assert rc == 0, ("stage", err(), log[-6:])
            L["tk"], L["tv"] = tk, tv
        elif op == "copy" and len(live) < 5:
            src = live[int(rng.integers(0, len(live)))]
            rc = lib.cf_ms_cuda_copy_sequence_async(r, C.c_int64(src), C.c_int64(next_id), None)
            log.append(("copy", src, next_id)); assert rc == 0, ("copy", err(), log[-6:])
            seqs[next_id] = [dict(k=L["k"].copy(), v=L["v"].copy(), closed=L["closed"], tk=L["tk"].copy(), tv=L["tv"].copy()) for L in seqs[src]]
            next_id += 1
        elif op == "execute":
            cand = [(s, layer) for s in live for layer in range(layers) if total(seqs[s][layer]) > 0]
            if not cand: continue
            n = int(rng.integers(1, min(5, len(cand)) + 1))
            picks = [cand[i] for i in rng.choice(len(cand), n, replace=False)]
            items = (MsBatchItem * n)(); checks = []
            for i, (s, layer) in enumerate(picks):
                L = seqs[s][layer]; tot = total(L)
                nq = int(rng.integers(1, min(3, tot) + 1)); begin = tot - nq
                q = rng.standard_normal((nq, hq, d)).astype(np.float32)
                qd = torch.from_numpy(q).cuda(); od = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda"); keep.append((qd, od))
                items[i].sequence_id, items[i].layer = s, layer
                items[i].query = TensorView(qd.data_ptr(), 3, nq, hq, d, hq * d * 4, d * 4, 4, 0)
                items[i].output, items[i].output_type = od.data_ptr(), 3
                items[i].output_token_stride_bytes, items[i].output_head_stride_bytes, items[i].output_element_stride_bytes = hq * d * 4, d * 4, 4
                items[i].query_token_begin, items[i].softmax_scale, items[i].causal_window = begin, scale, 0
                checks.append((s, layer, q, [begin + j for j in range(nq)], od))
            rc = lib.cf_ms_cuda_execute_batch_async(r, items, n, None)
            log.append(("execute", picks)); assert rc == 0, ("execute", err(), log[-6:])
            torch.cuda.synchronize()
            for s, layer, q, pos, od in checks:
                L = seqs[s][layer]
                hk = np.concatenate([L["k"], L["tk"]]); hv = np.concatenate([L["v"], L["tv"]])
                want = _expected(oracle, hk, hv, L["k"].shape[0], tile, q, pos, scale, group)
                got = od.cpu().numpy()
                assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max()), ("attention", s, layer, float(np.abs(got - want).max()), log[-6:])
        elif op == "remove" and len(live) > 1:
            s = live[int(rng.integers(0, len(live)))]
            assert lib.cf_ms_cuda_sequence_remove_async(r, C.c_int64(s), None) == 0, err()
            log.append(("remove", s)); del seqs[s]
        elif op == "reclaim":
            assert lib.cf_ms_cuda_reclaim_async(r, None) == 0 and lib.cf_ms_cuda_audit(r) == 0, (err(), log[-6:])
            log.append(("reclaim",))
    for s in list(seqs): assert lib.cf_ms_cuda_sequence_remove_async(r, C.c_int64(s), None) == 0
    torch.cuda.synchronize()
    assert lib.cf_ms_cuda_reclaim_async(r, None) == 0 and lib.cf_ms_cuda_audit(r) == 0
    n = MsCounters(); lib.cf_ms_cuda_get_counters(r, C.byref(n))
    assert n.in_flight_page_references == 0 and n.pending_reclamation_bytes == 0 and n.dense_fallback_launches == 0, (n.in_flight_page_references, n.pending_reclamation_bytes)
    lib.cf_ms_cuda_destroy(r, None)
    return len(log)


@pytest.mark.parametrize("first", range(0, 12, 6))
def test_random_operations_on_the_sequence_resolver(native, oracle, first):
    """cf_ms_cuda_*: sequences created, int4 pages published (transcoded on the GPU; a short page closes its layer),
    tails staged, sequences copied and removed, batches of decode and short prefill items executed, reclaim with audit,
    in random order; attention against fp64 softmax over the model's rows with the sealed ones requantised as the
    store does."""
    for seed in range(9800 + first, 9800 + first + 6):
        assert _resolver_run(native, oracle, seed, 70) > 0


# ---- the seal engine ABI ----------------------------------------------------------------------------------------------
def _seal_engine_case(native, oracle, seed):
    import ctypes as C
    import torch
    from compat_types import DeviceSealConfig, DeviceSealCounters, TensorView
    from test_gpu_device_engine import _expected
    rng = np.random.default_rng(seed)
    lib = native.lib(); lib.cf_device_seal_create.restype = C.c_void_p; lib.cf_device_seal_last_error.restype = C.c_char_p
    layers = int(rng.integers(1, 3)); hkv = int(rng.choice([1, 2, 4, 8])); group = int(rng.choice([1, 2, 4, 7])); hq = hkv * group
    d = int(rng.choice([32, 64, 96, 128, 128, 80])); page = int(rng.choice([16, 32, 64]))
    e = C.c_void_p(lib.cf_device_seal_create(C.byref(DeviceSealConfig(layers, hkv, hq, d, page, group, 64, 0))))
    what = dict(seed=seed, layers=layers, heads=(hq, hkv), d=d, page=page)
    if not e.value: return ("create refused",), what
    err = lambda: lib.cf_device_seal_last_error(e)
    state, n = C.c_uint32(0), DeviceSealCounters()
    tile = _record_tokens(page, d)
    for layer in range(layers):
        pages = int(rng.integers(0, 6)); tail = int(rng.integers(0, page))
        if pages + tail == 0: tail = 1
        tokens = pages * page + tail
        k = (rng.standard_normal((tokens, hkv, d)) * 10.0 ** rng.uniform(-2, 1)).astype(np.float32); v = (rng.standard_normal((tokens, hkv, d)) * 10.0 ** rng.uniform(-3, 2)).astype(np.float32)
        dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
        def stage(begin, count, src_k=None): return lib.cf_device_seal_stage_active_page(e, layer, begin, C.c_void_p((src_k if src_k is not None else dk)[begin:].data_ptr()), C.c_void_p(dv[begin:].data_ptr()), count, None)
        for pg in range(pages):
            b = pg * page
            if rng.random() < 0.3:   # a partial stage first, then the whole page
                part = int(rng.integers(1, page))
                if stage(b, part) != 0: return ("partial stage", err()), what
                if lib.cf_device_seal_full_page_async(e, layer, None) != -1: return ("sealed a page that is not full",), what
            if rng.random() < 0.2:   # a NaN page is refused and stays staged
                bad = dk.clone(); bad[b + int(rng.integers(0, page)), int(rng.integers(0, hkv)), int(rng.integers(0, d))] = float("nan")
                if stage(b, page, bad) != 0: return ("stage nan", err()), what
                if lib.cf_device_seal_full_page_async(e, layer, None) != -1 or b"NaN" not in err(): return ("nan page not refused", err()), what
            if stage(b, page) != 0: return ("stage", err()), what
            lib.cf_device_seal_get_counters(e, C.byref(n)); before = (n.seal_successes, n.page_table_generation, n.descriptor_publications)
            for _ in range(int(rng.integers(0, 3))):
                fault = int(rng.choice([1, 2, 3, 4, 5, 6, 7, 9, 10]))
                lib.cf_device_seal_set_fault(e, fault)
                if lib.cf_device_seal_full_page_async(e, layer, None) != -1: return ("fault ignored", fault), what
                lib.cf_device_seal_get_state(e, layer, C.byref(state)); lib.cf_device_seal_get_counters(e, C.byref(n))
                if state.value != 1 or (n.seal_successes, n.page_table_generation, n.descriptor_publications) != before: return ("fault left traces", fault), what
            lib.cf_device_seal_set_fault(e, 0)
            if lib.cf_device_seal_full_page_async(e, layer, None) != 0: return ("seal", err()), what
        if tail and stage(pages * page, tail) != 0: return ("tail stage", err()), what
        for _ in range(2):
            nq = int(rng.integers(1, min(4, tokens) + 1)); window = int(rng.integers(1, tokens + 3)) if rng.random() < 0.4 else 0
            scale = 1.0 / np.sqrt(d)
            q = rng.standard_normal((nq, hq, d)).astype(np.float32); qf = torch.from_numpy(q).cuda()
            view = TensorView(qf.data_ptr(), 3, nq, hq, d, hq * d * 4, d * 4, 4, 0)
            out = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda")
            pos0 = int(rng.integers(nq - 1, tokens)) - (nq - 1)
            pos = [pos0 + i for i in range(nq)]
            rc = lib.cf_device_seal_attention_async(e, layer, C.byref(view), C.c_void_p(out.data_ptr()), 3, C.c_uint64(hq * d * 4), C.c_uint64(d * 4), C.c_uint64(4), pos[0], C.c_float(scale), window, None)
            if rc != 0: return ("attention rc", err(), pos, tokens), what
            torch.cuda.synchronize()
            want = _expected(oracle, k, v, pages * page, tile, q, pos, window, scale, group)
            got = out.cpu().numpy()
            er = np.abs(got - want).max() / (np.abs(want).max() + 1e-30)
            if not np.isfinite(got).all() or er > 2e-4: return ("attention", layer, float(er), pos, tokens, window), what
    lib.cf_device_seal_destroy(e, None)
    return None, what


@pytest.mark.parametrize("first", range(0, 30, 15))
def test_random_seal_engine_cases(native, oracle, first):
    """cf_device_seal_*: pages staged (sometimes partly first, sometimes with a NaN first, which must be refused and
    leave the page staged), sealed after zero to two injected faults at random fault points (each must abort without
    a trace in the counters or the state), a partial tail, and query rows at random positions with or without a
    window, against fp64 softmax over the engine's quantisation."""
    for seed in range(9900 + first, 9900 + first + 15):
        bad, what = _seal_engine_case(native, oracle, seed)
        assert bad is None, (bad, what)


# ---- the host sequence cache against the reference's own ---------------------------------------------------------------
def _cache_prototypes(lib):
    import ctypes as C
    lib.cf_multisequence_create.restype = C.c_void_p
    lib.cf_multisequence_last_error.restype = C.c_char_p
    lib.cf_sequence_speculation_begin.restype = C.c_uint64


def _cache_side_by_side(native, oracle, seed, steps):
    """The same random calls on this library's cache and on the reference's, compiled from its source; returns the first
    difference in a status (with the calls before it) or in the final counters, or None."""
    import ctypes as C
    import torch
    from compat_types import MultisequenceConfig, MultisequenceCounters, MULTISEQUENCE_COUNTER_NAMES
    from test_gpu_mscache import _view
    rng = np.random.default_rng(seed)
    mine, ref = native.lib(), oracle.ref_mscache()
    _cache_prototypes(mine); _cache_prototypes(ref)
    LAYERS = int(rng.integers(1, 3)); HKV = int(rng.choice([1, 2])); G = int(rng.choice([1, 4])); HQ = HKV * G; D = 128; PAGE = int(rng.choice([16, 32]))
    cfg = MultisequenceConfig(LAYERS, HKV, HQ, D, PAGE, G, 0, 1)
    a, b = C.c_void_p(mine.cf_multisequence_create(C.byref(cfg))), C.c_void_p(ref.cf_multisequence_create(C.byref(cfg)))
    assert a.value and b.value
    i64 = C.c_int64
    count = {}; begin = {}   # model of the active rows per sequence (the same in every layer)
    specs = {}               # sequence -> (id mine, id ref, baseline)
    log = []
    rows = torch.zeros((PAGE, HKV, D), dtype=torch.float16, device="cuda")
    def both(name, *args):
        ra, rb = getattr(mine, name)(a, *args), getattr(ref, name)(b, *args)
        return ra, rb
    for step in range(steps):
        ids = list(count) or [1]
        pick = lambda: int(ids[int(rng.integers(0, len(ids)))]) if rng.random() < 0.9 else int(rng.integers(1, 9))
        op = ["create", "append", "append", "append", "copy", "remove", "remove_range", "shift", "spec_begin", "spec_end", "reclaim"][int(rng.integers(0, 11))]
        if op == "create":
            s = int(rng.integers(1, 9)); ra, rb = both("cf_sequence_create", i64(s)); log.append((op, s, ra, rb))
            if ra == 0 and rb == 0 and s not in count: count[s] = 0; begin[s] = 0
        elif op == "append":
            s = pick(); n = int(rng.integers(1, PAGE + 2)); c = count.get(s, 0)
            if c + n == PAGE: n += 1            # an exactly full page: this library seals it, the reference's cache never does
            n = min(n, PAGE)
            if c + n == PAGE: continue
            where = begin.get(s, 0) + c if (c or rng.random() < 0.7) else int(rng.integers(0, 100))
            if rng.random() < 0.1: where += int(rng.integers(1, 5))      # a gap
            res = []
            for layer in range(LAYERS):
                kv = _view(rows, n)
                res.append((mine.cf_sequence_append_async(a, i64(s), layer, where, C.byref(kv), C.byref(kv), None),
                            ref.cf_sequence_append_async(b, i64(s), layer, where, C.byref(kv), C.byref(kv), None)))
            log.append((op, s, n, where, res))
            if any(x != y for x, y in res): return ("append", [l for l in log if len(l) > 1 and l[1] == s][-12:], "PAGE", PAGE)
            if res[0][0] == 0 and s in count:
                if c == 0: begin[s] = where
                count[s] = c + n
        elif op == "copy":
            s, t = pick(), int(rng.integers(1, 9))
            kind = int(rng.integers(0, 3))
            lo, hi = (0, 1 << 30) if kind == 0 else tuple(sorted(int(x) for x in rng.integers(0, 120, 2)))
            ra, rb = both("cf_sequence_copy_async", i64(s), i64(t), C.c_uint32(lo), C.c_uint32(hi), None); log.append((op, s, t, lo, hi, ra, rb))
            if ra != rb: return ("copy", log[-5:])
            if ra == 0:
                c, bg = count.get(s, 0), begin.get(s, 0)
                inside = c and bg >= lo and bg + c <= hi
                count[t] = c if inside else 0; begin[t] = bg if inside else 0
                specs.pop(t, None)
        elif op == "remove":
            s = pick(); ra, rb = both("cf_sequence_remove_async", i64(s), i64(-1), i64(-1), None); log.append((op, s, ra, rb))
            if ra != rb: return ("remove", log[-5:])
            if ra == 0: count.pop(s, None); begin.pop(s, None); specs.pop(s, None)
        elif op == "remove_range":
            s = pick(); c, bg = count.get(s, 0), begin.get(s, 0)
            if s in specs: continue     # the reference's rollback would then lengthen the tail again
            lo = bg + int(rng.integers(-2, c + 3)); hi = lo + int(rng.integers(0, c + 4)) if rng.random() < 0.5 else 1 << 40
            ra, rb = both("cf_sequence_remove_async", i64(s), i64(lo), i64(hi), None); log.append((op, s, lo, hi, "active", bg, c, ra, rb))
            if ra != rb: return ("remove_range", log[-5:])
            if ra == 0 and s in count:
                l2 = max(lo, 0)
                if l2 <= bg and hi >= bg + c: count[s] = 0
                elif bg <= l2 < bg + c and hi >= bg + c: count[s] = l2 - bg
        elif op == "shift":
            s = pick(); c, bg = count.get(s, 0), begin.get(s, 0)
            lo, hi = (0, 1 << 30) if rng.random() < 0.6 else tuple(sorted(int(x) for x in rng.integers(0, 120, 2)))
            delta = int(rng.integers(-40, 40))
            ra, rb = both("cf_sequence_shift_async", i64(s), C.c_uint32(lo), C.c_uint32(hi), C.c_int32(delta), None); log.append((op, s, lo, hi, delta, "active", bg, c, ra, rb))
            if ra != rb: return ("shift", log[-5:])
            if ra == 0 and s in count and c and bg >= lo and bg + c <= hi: begin[s] = bg + delta
        elif op == "spec_begin":
            s = pick(); ia, ib = mine.cf_sequence_speculation_begin(a, i64(s)), ref.cf_sequence_speculation_begin(b, i64(s)); log.append((op, s, ia, ib))
            if (ia == 0) != (ib == 0): return ("spec_begin", log[-5:])
            if ia: specs[s] = (ia, ib, count.get(s, 0))
        elif op == "spec_end" and specs:
            s = list(specs)[int(rng.integers(0, len(specs)))]; ia, ib, base = specs[s]
            if rng.random() < 0.15: ia, ib = ia + 7, ib + 7      # a wrong id
            if rng.random() < 0.5:
                keep = int(rng.integers(0, max(count.get(s, 0) - base, 0) + 2))
                ra, rb = mine.cf_sequence_speculation_commit(a, i64(s), C.c_uint64(ia), keep, None), ref.cf_sequence_speculation_commit(b, i64(s), C.c_uint64(ib), keep, None)
                log.append(("commit", s, keep, "count", count.get(s), "base", base, ra, rb))
                if ra != rb: return ("commit", log[-5:])
                if ra == 0: count[s] = base + keep; specs.pop(s)
            else:
                ra, rb = mine.cf_sequence_speculation_rollback(a, i64(s), C.c_uint64(ia), None), ref.cf_sequence_speculation_rollback(b, i64(s), C.c_uint64(ib), None)
                log.append(("rollback", s, "count", count.get(s), "base", base, ra, rb))
                if ra != rb: return ("rollback", log[-5:])
                if ra == 0: count[s] = base; specs.pop(s)
        elif op == "reclaim":
            ra, rb = both("cf_multisequence_reclaim_async", None); ra2, rb2 = mine.cf_multisequence_audit(a), ref.cf_multisequence_audit(b)
            if (ra, ra2) != (rb, rb2): return ("reclaim/audit", ra, rb, ra2, rb2, log[-5:])
    ka, kb = MultisequenceCounters(), MultisequenceCounters()
    mine.cf_multisequence_get_counters(a, C.byref(ka)); ref.cf_multisequence_get_counters(b, C.byref(kb))
    diff = {n: (int(getattr(ka, n)), int(getattr(kb, n))) for n in MULTISEQUENCE_COUNTER_NAMES if getattr(ka, n) != getattr(kb, n)}
    mine.cf_multisequence_destroy(a, None); ref.cf_multisequence_destroy(b, None)
    return ("counters", diff) if diff else None


@pytest.mark.parametrize("first", range(0, 40, 20))
def test_sequence_cache_calls_answer_like_the_references_own_cache(native, oracle, first):
    """cf_sequence_create / append / copy / remove (whole and ranges) / shift / speculation begin, commit, rollback /
    reclaim / audit with valid and invalid arguments (unknown ids, gaps, ranges that cut the tail, empty ranges, wrong
    speculation ids), the same calls on the reference's own host cache (src/multisequence_cache.cpp compiled into
    oracle/_ref): every call returns the same status and the counter blocks are equal at the end. The runs stay where
    the two can be compared: the reference's cache never seals a page, so no tail is filled exactly, and no rows are
    removed while a speculation is open (its rollback would then lengthen the tail again)."""
    if oracle.ref_mscache() is None:
        pytest.skip("needs the reference's host cache (oracle/_ref)")
    for seed in range(first, first + 20):
        bad = _cache_side_by_side(native, oracle, seed, 120)
        assert bad is None, (seed, bad)


# ---- the decode runtime beside the reference's own --------------------------------------------------------------------
def _runtime_int4_page_pair(rng, tokens, token_begin, keep, HKV, D, BLOCK, wild):
    """One page twice: nibbles as the reference's seal engine writes them (value + 8, device_kv_seal_attention.cu:101) and
    the same values as two's-complement nibbles, which is how the reference's decode kernel reads a nibble
    (production_attention.cu:39-44)."""
    import torch
    from compat_types import PageDescriptor
    desc, desc2, dense = PageDescriptor(), PageDescriptor(), []
    for name in ("key", "value"):
        x = rng.standard_normal((tokens, HKV, D)).astype(np.float32)
        if wild: x *= (10.0 ** rng.uniform(-3, 2, (tokens, 1, 1))).astype(np.float32)
        blocks = x.reshape(-1, BLOCK)
        scale = (np.abs(blocks).max(axis=1) / 7.0).astype(np.float32)
        scale[scale == 0] = 1.0
        q = np.clip(np.rint(blocks / scale[:, None]), -7, 7).astype(np.int32)
        dense.append((q.astype(np.float32) * scale[:, None]).reshape(tokens, HKV, D))
        nib = (q + 8).astype(np.uint8).reshape(-1)
        payload = (nib[0::2] | (nib[1::2] << 4)).astype(np.uint8)
        twos = (q & 0xF).astype(np.uint8).reshape(-1)                    # the same values as two's-complement nibbles
        payload2 = (twos[0::2] | (twos[1::2] << 4)).astype(np.uint8)
        p, s, p2 = torch.from_numpy(payload).cuda(), torch.from_numpy(scale).cuda(), torch.from_numpy(payload2).cuda()
        keep += [p, s, p2]
        setattr(desc, name + "_payload", p.data_ptr()); setattr(desc, name + "_scales", s.data_ptr()); setattr(desc, name + "_payload_bytes", payload.size)
        setattr(desc2, name + "_payload", p2.data_ptr()); setattr(desc2, name + "_scales", s.data_ptr()); setattr(desc2, name + "_payload_bytes", payload.size)
    for x in (desc, desc2):
        x.token_begin, x.token_count, x.kv_head_count, x.head_dim = token_begin, tokens, HKV, D
        x.block_size, x.blocks_per_page = BLOCK, tokens * HKV * D // BLOCK
    return (desc, desc2), dense[0], dense[1]


def _runtime_side_by_side(native, oracle, seed):
    import ctypes as C
    import torch
    from compat_types import AttentionBatchItem, AttentionCounters, AttentionRuntimeConfig, PageDescriptor, TensorView
    rng = np.random.default_rng(seed)
    lib = native.lib(); lib.cf_attention_runtime_create.restype = C.c_void_p; lib.cf_attention_last_error.restype = C.c_char_p
    ref = oracle.ref_device(); ref.cf_attention_runtime_create.restype = C.c_void_p
    HKV = int(rng.choice([1, 2, 4, 8])); G = int(rng.choice([1, 2, 4, 7])); HQ = HKV * G
    D = int(rng.choice([32, 64, 96, 128, 80])); BLOCK = int(rng.choice([16, 32, 64])); PAGE = int(rng.choice([16, 32, 64]))
    if D % BLOCK and BLOCK % D: BLOCK = 16
    mode = 1; layers = int(rng.integers(1, 4))
    cfg = AttentionRuntimeConfig()
    cfg.layer_count, cfg.query_head_count, cfg.kv_head_count, cfg.head_dim = layers, HQ, HKV, D
    cfg.page_size, cfg.block_size, cfg.gqa_group_size, cfg.mode = PAGE, BLOCK, G, mode
    rt = C.c_void_p(lib.cf_attention_runtime_create(C.byref(cfg)))
    what = dict(seed=seed, heads=(HQ, HKV), D=D, BLOCK=BLOCK, PAGE=PAGE, mode=mode, layers=layers)
    if not rt.value: return ("create refused",), what
    n = int(rng.integers(1, 7)); wild = rng.random() < 0.4
    keep, items, expected, outputs = [], (AttentionBatchItem * n)(), [], []
    ref_pages = []
    scale = 1.0 / np.sqrt(D)
    cases = []
    for i in range(n):
        pages = int(rng.integers(0, 11)); tail = int(rng.integers(0, PAGE))
        if pages + tail == 0: tail = 1
        window = 0
        qdt = [torch.float32, torch.float16, torch.bfloat16][int(rng.integers(0, 3))]; odt = [torch.float32, torch.float16][int(rng.integers(0, 2))]
        cases.append((pages, tail, window, str(qdt), str(odt)))
        descs = (PageDescriptor * max(pages, 1))(); descs2 = (PageDescriptor * max(pages, 1))(); ks, vs = [], []
        for pg in range(pages):
            (descs[pg], descs2[pg]), k, v = _runtime_int4_page_pair(rng, PAGE, pg * PAGE, keep, HKV, D, BLOCK, wild); ks.append(k); vs.append(v)
        tk = rng.standard_normal((tail, HKV, D)).astype(np.float32); tv = rng.standard_normal((tail, HKV, D)).astype(np.float32)
        ks.append(tk); vs.append(tv)
        k_all, v_all = np.concatenate(ks), np.concatenate(vs)
        qpos = pages * PAGE + tail - 1
        q = torch.from_numpy(rng.standard_normal((HQ, D)).astype(np.float32)).to(qdt).cuda()
        out = torch.zeros((HQ, D), dtype=odt, device="cuda")
        d_desc = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
        d_desc2 = torch.from_numpy(np.frombuffer(bytes(descs2), dtype=np.uint8).copy()).cuda(); keep.append(d_desc2); ref_pages.append(d_desc2.data_ptr() if pages else None)
        d_tk, d_tv = torch.from_numpy(np.ascontiguousarray(tk)).cuda(), torch.from_numpy(np.ascontiguousarray(tv)).cuda()
        keep += [q, out, d_desc, d_tk, d_tv]
        it = items[i]
        it.sequence_id, it.layer = 100 + i, int(rng.integers(0, layers))
        esz = q.element_size()
        it.query = TensorView(q.data_ptr(), {torch.float16: 1, torch.bfloat16: 2, torch.float32: 3}[qdt], 1, HQ, D, HQ * D * esz, D * esz, esz, 0)
        it.output, it.output_type = out.data_ptr(), {torch.float16: 1, torch.float32: 3}[odt]
        osz = out.element_size()
        it.output_token_stride_bytes, it.output_head_stride_bytes, it.output_element_stride_bytes = HQ * D * osz, D * osz, osz
        it.query_token_begin, it.softmax_scale, it.causal_window = qpos, scale, window
        it.sealed_pages, it.sealed_page_count = (d_desc.data_ptr() if pages else None), pages
        it.active_keys, it.active_values = (d_tk.data_ptr() if tail else None), (d_tv.data_ptr() if tail else None)
        it.active_token_begin, it.active_token_count = pages * PAGE, tail
        first = 0 if window == 0 else max(0, qpos + 1 - window)
        qf = q.float().cpu().numpy(); exp = np.zeros((HQ, D))
        for h in range(HQ):
            kv = h // G
            s = (k_all[first:qpos + 1, kv].astype(np.float64) @ qf[h].astype(np.float64)) * scale
            w = np.exp(s - s.max()); exp[h] = (w[:, None] * v_all[first:qpos + 1, kv]).sum(0) / w.sum()
        expected.append(exp); outputs.append(out)
    what["cases"] = cases; what["wild"] = wild
    rc = lib.cf_attention_execute_async(rt, items, n, None)
    if rc != 0: return ("execute", lib.cf_attention_last_error(rt)), what
    torch.cuda.synchronize()
    mine_out = [o.float().cpu().numpy().copy() for o in outputs]
    for o in outputs: o.zero_()
    rt2 = C.c_void_p(ref.cf_attention_runtime_create(C.byref(cfg)))
    if not rt2.value: return ("reference create refused",), what
    if D % BLOCK: return None, what      # the reference's kernel indexes scales per head; only whole blocks per head compare
    items2 = (AttentionBatchItem * n)()
    for i in range(n):
        C.memmove(C.byref(items2[i]), C.byref(items[i]), C.sizeof(AttentionBatchItem)); items2[i].sealed_pages = ref_pages[i]
    rc2 = ref.cf_attention_execute_async(rt2, items2, n, None)
    torch.cuda.synchronize()
    if rc2 != 0: return ("reference execute", rc2), what
    for i, (a, o) in enumerate(zip(mine_out, outputs)):
        r = o.float().cpu().numpy()
        tol = 2e-3 if o.dtype == torch.float16 else 2e-5
        e = np.abs(a - r).max() / (np.abs(r).max() + 1e-30)
        if e > tol: return ("differs from the reference kernel", i, float(e)), what
    ref.cf_attention_runtime_destroy(rt2, None)
    for o, a in zip(outputs, mine_out): o.copy_(torch.from_numpy(a).to(o.dtype))
    for i, (out, exp) in enumerate(zip(outputs, expected)):
        got = out.float().cpu().numpy()
        tol = 2e-3 if out.dtype == torch.float16 else 2e-4
        e = np.abs(got - exp).max() / (np.abs(exp).max() + 1e-30)
        if not np.isfinite(got).all() or e > tol: return ("item", i, float(e)), what
    c = AttentionCounters(); lib.cf_attention_get_counters(rt, C.byref(c))
    if c.cuda_errors != 0: return ("cuda errors",), what
    lib.cf_attention_runtime_destroy(rt, None)
    return None, what


@pytest.mark.parametrize("first", range(0, 30, 15))
def test_decode_runtime_beside_the_references_own_kernel(native, oracle, first):
    """cf_attention_execute_async here and in the reference (src/cuda/production_attention.cu compiled into oracle/_ref) on
    the same random batches, no window, query at the last token. The reference's kernel reads a nibble as two's
    complement while its seal engine writes value + 8; it is therefore given the same values re-encoded, and the two
    libraries must then agree to 2e-5 of the output's scale (2e-3 for fp16 outputs). This library reads the pages the
    way the seal engine writes them."""
    if oracle.ref_device() is None:
        pytest.skip("needs the reference's decode runtime (oracle/_ref)")
    for seed in range(9600 + first, 9600 + first + 15):
        bad, what = _runtime_side_by_side(native, oracle, seed)
        assert bad is None, (bad, what)


# ---- the seal engine beside the reference's own -----------------------------------------------------------------------
SEAL_COUNTERS_COMPARED = ("seal_attempts", "seal_successes", "seal_failures", "invalid_pages_rejected", "values_quantized", "descriptor_publications",
        "page_table_generation", "compressed_attention_launches", "sealed_pages_consumed", "cuda_errors")


def _seal_engine_side_by_side(native, oracle, seed):
    import ctypes as C
    import torch
    from compat_types import DeviceSealConfig, DeviceSealCounters
    rng = np.random.default_rng(seed)
    libs = [native.lib(), oracle.ref_device()]
    for l in libs: l.cf_device_seal_create.restype = C.c_void_p; l.cf_device_seal_last_error.restype = C.c_char_p
    layers = int(rng.integers(1, 3)); hkv = int(rng.choice([1, 2, 4])); group = int(rng.choice([1, 2, 4])); hq = hkv * group
    d = int(rng.choice([64, 128])); page = int(rng.choice([16, 32, 64])); block = int(rng.choice([32, 64]))
    cfg = DeviceSealConfig(layers, hkv, hq, d, page, group, block, 0)
    es = [C.c_void_p(l.cf_device_seal_create(C.byref(cfg))) for l in libs]
    what = dict(seed=seed, layers=layers, heads=(hq, hkv), d=d, page=page, block=block)
    if not es[0].value or not es[1].value: return ("create", bool(es[0].value), bool(es[1].value)), what
    log = []
    def both(name, *args):
        r = tuple(getattr(l, name)(e, *args) for l, e in zip(libs, es)); log.append((name, r)); return r
    def states(layer):
        out = []
        for l, e in zip(libs, es):
            st = C.c_uint32(99); l.cf_device_seal_get_state(e, layer, C.byref(st)); out.append(st.value)
        return tuple(out)
    sealed = [0] * layers
    base = {}
    rows = {}
    for step in range(int(rng.integers(10, 40))):
        layer = int(rng.integers(0, layers + 1))    # one past the last: an invalid layer
        op = ["stage", "stage", "seal", "seal", "fault", "attend", "stage_bad", "clear"][int(rng.integers(0, 8))]
        if op in ("stage", "stage_bad"):
            count = page if rng.random() < 0.6 else int(rng.integers(0, page + 2))
            have = sealed[min(layer, layers - 1)]
            begin = base.get(min(layer, layers - 1), 0) + have if (op == "stage" or have or rng.random() < 0.5) else int(rng.integers(0, 200))
            if not have: base[min(layer, layers - 1)] = begin
            k = rng.standard_normal((max(count, 1), hkv, d)).astype(np.float32); v = rng.standard_normal((max(count, 1), hkv, d)).astype(np.float32)
            if rng.random() < 0.1: k[int(rng.integers(0, max(count, 1))), 0, 0] = np.nan
            dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(); rows[step] = (dk, dv)
            r = both("cf_device_seal_stage_active_page", layer, begin, C.c_void_p(dk.data_ptr()), C.c_void_p(dv.data_ptr()), count, None)
            log[-1] = log[-1] + (("layer", layer, "begin", begin, "count", count, "sealed", sealed),)
        elif op == "seal":
            r = both("cf_device_seal_full_page_async", layer, None)
            if r == (0, 0) and layer < layers: sealed[layer] += page
        elif op == "fault":
            fv = int(rng.integers(0, 12)); r = both("cf_device_seal_set_fault", fv); log[-1] = log[-1] + (fv,)
        elif op == "clear":
            if rng.random() < 0.7: continue
            r = both("cf_device_seal_clear_async", None); sealed = [0] * layers; base = {}
        else:
            continue
        torch.cuda.synchronize()
        if r[0] != r[1]: return ("status", log[-6:]), what
        if layer < layers and states(layer)[0] != states(layer)[1]: return ("state", states(layer), log[-6:]), what
    ka, kb = DeviceSealCounters(), DeviceSealCounters()
    libs[0].cf_device_seal_get_counters(es[0], C.byref(ka)); libs[1].cf_device_seal_get_counters(es[1], C.byref(kb))
    diff = {n: (int(getattr(ka, n)), int(getattr(kb, n))) for n in SEAL_COUNTERS_COMPARED if getattr(ka, n) != getattr(kb, n)}
    for l, e in zip(libs, es): l.cf_device_seal_destroy(e, None)
    return (("counters", diff, log[-4:]), what) if diff else (None, what)


@pytest.mark.parametrize("first", range(0, 40, 20))
def test_seal_engine_answers_like_the_references_own(native, oracle, first):
    """cf_device_seal_* here and in the reference (src/cuda/device_kv_seal_attention.cu compiled into oracle/_ref): random
    stage / seal / set_fault / clear calls, valid and invalid (layers that do not exist, zero or too many rows, NaN
    pages, every fault point, faults left armed). Every call returns the same status, the layer is in the same state
    after it, and ten counters that mean the same in both are equal at the end. Staging stays where the two can be
    compared: a layer that has sealed pages is staged at its next position (this library's history is contiguous)."""
    if oracle.ref_device() is None:
        pytest.skip("needs the reference's seal engine (oracle/_ref)")
    for seed in range(first, first + 20):
        bad, what = _seal_engine_side_by_side(native, oracle, seed)
        assert bad is None, (bad, what)


# ---- the sequence resolver beside the reference's own -----------------------------------------------------------------
def _resolver_counters_compared():
    from compat_types import MsCounters
    return [n for n, _ in MsCounters._fields_ if n not in ("descriptor_table_rebuilds", "sequence_attention_launches", "descriptor_tables_built")]


def _resolver_side_by_side(native, oracle, seed, steps):
    import ctypes as C
    import torch
    from compat_types import MsBatchItem, MsConfig, MsCounters, MsPublication, PageDescriptor, TensorView
    from test_gpu_ms_resolver import _int4_page
    NAMES = _resolver_counters_compared()
    rng = np.random.default_rng(seed)
    libs = [native.lib(), oracle.ref_device()]
    for l in libs: l.cf_ms_cuda_create.restype = C.c_void_p; l.cf_ms_cuda_last_error.restype = C.c_char_p
    layers = int(rng.integers(1, 3)); hkv = int(rng.choice([1, 2, 4])); group = int(rng.choice([1, 2, 4])); hq = hkv * group
    d = int(rng.choice([64, 128])); page = int(rng.choice([16, 32, 64])); block = int(rng.choice([16, 32, 64]))
    cfg = MsConfig(layers, hkv, hq, d, page, group, 0)
    rs = [C.c_void_p(l.cf_ms_cuda_create(C.byref(cfg))) for l in libs]
    what = dict(seed=seed, layers=layers, heads=(hq, hkv), d=d, page=page, block=block)
    if not rs[0].value or not rs[1].value: return ("create", bool(rs[0].value), bool(rs[1].value)), what
    keep = []; log = []
    def both(name, *args):
        r = tuple(getattr(l, name)(x, *args) for l, x in zip(libs, rs)); log.append((name, r)); return r
    seqs = {}   # id -> per layer dict(sealed tokens, closed, tail rows, dense rows k / v, cancelled flag at sequence level)
    cancelled = set(); next_id = 1; scale = 1.0 / np.sqrt(d)
    def new_layer(): return dict(k=np.zeros((0, hkv, d), np.float32), v=np.zeros((0, hkv, d), np.float32), closed=False, tk=np.zeros((0, hkv, d), np.float32), tv=np.zeros((0, hkv, d), np.float32))
    for step in range(steps):
        live = list(seqs)
        def pick():     # a live sequence, or now and then an id that may not exist; never a cancelled one, whose history the
            while True:  # model no longer follows (this library would refuse a page that does not continue it)
                s = int(live[int(rng.integers(0, len(live)))]) if live and rng.random() < 0.9 else int(rng.integers(1, 12))
                if s not in cancelled: return s
        op = ["create", "publish", "publish", "publish", "stage", "stage", "copy", "execute", "execute", "remove", "reclaim", "cancel", "audit"][int(rng.integers(0, 13))]
        if op == "create":
            s = int(rng.integers(1, 12))
            if s in cancelled: continue
            r = both("cf_ms_cuda_sequence_create", C.c_int64(s)); log[-1] += (s,)
            if r == (0, 0): seqs[s] = [new_layer() for _ in range(layers)]
        elif op == "publish":
            s = pick(); layer = int(rng.integers(0, layers + 1)); L = seqs[s][layer] if s in seqs and layer < layers else None
            if L is not None and (L["closed"] or L["tk"].shape[0] or L["k"].shape[0] > 300): continue
            tokens = page if rng.random() < 0.8 else int(rng.integers(1, page + 1))
            if (tokens * hkv * d) % block: tokens = page
            (kp, ks, kd), (vp, vs, vd) = _int4_page(rng, tokens, hkv, d, block)
            t = [torch.from_numpy(x).cuda() for x in (kp, vp, ks, vs)]; keep.append(t)
            pub = MsPublication(); pub.sequence_id, pub.layer = s, layer
            begin = L["k"].shape[0] if L is not None else 0
            pub.descriptor = PageDescriptor(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), begin, tokens, hkv, d, block, ks.size, kp.size, vp.size, kp.size + vp.size + 8 * ks.size, 1)
            if rng.random() < 0.05: pub.descriptor.key_scales = None
            pub.resident_bytes, pub.seal_generation = kp.size + vp.size + 8 * ks.size, 1
            r = both("cf_ms_cuda_publish_page_async", C.byref(pub), None); log[-1] += (s, layer, tokens)
            if r == (0, 0) and L is not None:
                L["k"] = np.concatenate([L["k"], kd]); L["v"] = np.concatenate([L["v"], vd]); L["closed"] = tokens < page
        elif op == "stage":
            s = pick(); layer = int(rng.integers(0, layers + 1)); L = seqs[s][layer] if s in seqs and layer < layers else None
            count = int(rng.integers(0, page + 2))
            tk = rng.standard_normal((max(count, 1), hkv, d)).astype(np.float32); tv = rng.standard_normal((max(count, 1), hkv, d)).astype(np.float32)
            dk, dv = torch.from_numpy(tk).cuda(), torch.from_numpy(tv).cuda(); keep.append((dk, dv))
            begin = L["k"].shape[0] if L is not None else 0
            r = both("cf_ms_cuda_stage_active_async", C.c_int64(s), layer, begin, C.c_void_p(dk.data_ptr()), C.c_void_p(dv.data_ptr()), count, None); log[-1] += (s, layer, count)
            if r == (0, 0) and L is not None: L["tk"], L["tv"] = tk[:count], tv[:count]
        elif op == "copy":
            src = pick(); dst = next_id + 100; next_id += 1
            r = both("cf_ms_cuda_copy_sequence_async", C.c_int64(src), C.c_int64(dst), None); log[-1] += (src, dst)
            if r == (0, 0) and src in seqs: seqs[dst] = [dict(k=L["k"].copy(), v=L["v"].copy(), closed=L["closed"], tk=L["tk"].copy(), tv=L["tv"].copy()) for L in seqs[src]]
        elif op == "execute":
            cand = [(s, layer) for s in live for layer in range(layers) if seqs[s][layer]["k"].shape[0] + seqs[s][layer]["tk"].shape[0] > 0]
            if not cand: continue
            n = int(rng.integers(1, min(4, len(cand)) + 1)); picks = [cand[i] for i in rng.choice(len(cand), n, replace=False)]
            if rng.random() < 0.1: picks[0] = (int(rng.integers(20, 30)), 0)      # an unknown sequence
            outs = []
            for lib, x in zip(libs, rs):
                rng2 = np.random.default_rng(seed * 1000 + step)
                items = (MsBatchItem * n)(); ods = []
                for i, (s, layer) in enumerate(picks):
                    L = seqs[s][layer] if s in seqs else None
                    tot = (L["k"].shape[0] + L["tk"].shape[0]) if L is not None else 1
                    nq = int(rng2.integers(1, min(3, tot) + 1)); begin = tot - nq
                    q = rng2.standard_normal((nq, hq, d)).astype(np.float32)
                    qd = torch.from_numpy(q).cuda(); od = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda"); keep.append((qd, od)); ods.append(od)
                    items[i].sequence_id, items[i].layer = s, layer
                    items[i].query = TensorView(qd.data_ptr(), 3, nq, hq, d, hq * d * 4, d * 4, 4, 0)
                    items[i].output, items[i].output_type = od.data_ptr(), 3
                    items[i].output_token_stride_bytes, items[i].output_head_stride_bytes, items[i].output_element_stride_bytes = hq * d * 4, d * 4, 4
                    items[i].query_token_begin, items[i].softmax_scale, items[i].causal_window = begin, scale, 0
                rc = lib.cf_ms_cuda_execute_batch_async(x, items, n, None); torch.cuda.synchronize()
                outs.append((rc, [o.cpu().numpy() for o in ods]))
            log.append(("execute", (outs[0][0], outs[1][0]), picks))
            if outs[0][0] != outs[1][0]: return ("status", log[-6:]), what
            if outs[0][0] == 0:
                for a, b in zip(outs[0][1], outs[1][1]):
                    e = np.abs(a - b).max() / (np.abs(b).max() + 1e-30)
                    if not np.isfinite(a).all() or e > 5e-2: return ("attention", float(e), log[-3:]), what
            continue
        elif op == "remove":
            s = pick(); r = both("cf_ms_cuda_sequence_remove_async", C.c_int64(s), None); log[-1] += (s,)
            if r == (0, 0): seqs.pop(s, None)
        elif op == "cancel":
            if rng.random() < 0.7: continue
            s = pick(); r = both("cf_ms_cuda_cancel_sequence_async", C.c_int64(s), None); log[-1] += (s,)
            if r == (0, 0): seqs.pop(s, None); cancelled.add(s)      # not dispatchable any more: leave it alone
        elif op == "reclaim":
            torch.cuda.synchronize(); r = both("cf_ms_cuda_reclaim_async", None)
        else:
            r = both("cf_ms_cuda_audit")
        if r[0] != r[1]: return ("status", log[-6:], libs[0].cf_ms_cuda_last_error(rs[0]), libs[1].cf_ms_cuda_last_error(rs[1])), what
    ka, kb = MsCounters(), MsCounters()
    libs[0].cf_ms_cuda_get_counters(rs[0], C.byref(ka)); libs[1].cf_ms_cuda_get_counters(rs[1], C.byref(kb))
    diff = {n: (int(getattr(ka, n)), int(getattr(kb, n))) for n in NAMES if getattr(ka, n) != getattr(kb, n)}
    for l, x in zip(libs, rs): l.cf_ms_cuda_destroy(x, None)
    return (("counters", diff), what) if diff else (None, what)


@pytest.mark.parametrize("first", range(0, 20, 10))
def test_sequence_resolver_answers_like_the_references_own(native, oracle, first):
    """cf_ms_cuda_* here and in the reference (src/cuda/multisequence_cuda_resolver.cu compiled into oracle/_ref): random
    create / publish / stage / copy / execute / remove / cancel / reclaim / audit calls, valid and invalid (unknown
    sequences, layers that do not exist, incomplete descriptors, zero or too many rows). Every call returns the same
    status; every counter but the three that describe the reference's descriptor tables and its launch per item is
    equal at the end; attention agrees to 5 % of the output's scale (the reference reads the int4 pages as they are,
    this library its int8 transcoding of them). Pages are published in order, which is what this library takes."""
    if oracle.ref_device() is None:
        pytest.skip("needs the reference's resolver (oracle/_ref)")
    for seed in range(first, first + 10):
        bad, what = _resolver_side_by_side(native, oracle, seed, 70)
        assert bad is None, (bad, what)


# ---- the llama-server runtime beside the reference's own --------------------------------------------------------------
def _server_side_by_side(native, oracle, seed, steps):
    import ctypes as C
    import torch
    from compat_types import LlamaServerBatch, LlamaServerConfig, LlamaServerStats, MsBatchItem, TensorView
    rng = np.random.default_rng(seed)
    libs = [native.lib(), oracle.ref_device()]
    for l in libs: l.cf_llama_server_runtime_create.restype = C.c_void_p; l.cf_llama_server_last_error.restype = C.c_char_p
    LAYERS = int(rng.integers(1, 3)); HKV = int(rng.choice([1, 2])); G = int(rng.choice([1, 4])); HQ = HKV * G; D = int(rng.choice([64, 128])); PAGE = int(rng.choice([16, 32]))
    cfg = LlamaServerConfig(LAYERS, HQ, HKV, D, PAGE, 64, 4096, G, 0, 1, None, b"76f46ad2", b"0" * 64)
    rs = [C.c_void_p(l.cf_llama_server_runtime_create(C.byref(cfg))) for l in libs]
    what = dict(seed=seed, layers=LAYERS, heads=(HQ, HKV), d=D, page=PAGE)
    if not rs[0].value or not rs[1].value: return ("create", bool(rs[0].value), bool(rs[1].value)), what
    i64 = C.c_int64; log = []; keep = []
    def both(name, *args):
        r = tuple(getattr(l, name)(x, *args) for l, x in zip(libs, rs)); log.append((name, r) + tuple(a.value if hasattr(a, "value") else a for a in args[:3])); return r
    rows = {}     # (sequence, layer) -> (k, v) staged rows
    live = set(); cancelled = set(); shut = False; scale = 1.0 / np.sqrt(D)
    for step in range(steps):
        ids = sorted(live) or [1]
        pick = lambda: int(ids[int(rng.integers(0, len(ids)))]) if rng.random() < 0.9 else int(rng.integers(1, 9))
        op = ["slot", "slot", "append", "append", "append", "execute", "execute", "copy", "reset", "cancel", "remove_range", "shift", "shutdown"][int(rng.integers(0, 13))]
        if op == "slot":
            s = int(rng.integers(1, 9)); r = both("cf_llama_server_slot_create", i64(s))
            if r == (0, 0): live.add(s)
        elif op == "append":
            s = pick(); layer = int(rng.integers(0, LAYERS + 1)); n = int(rng.integers(0, PAGE + 1))
            if n == PAGE: n -= 1          # a full page is sealed here and stays staged in the reference
            if (s, layer) in rows or s in cancelled: continue     # the reference restages, this library appends: one append per layer
            k = rng.standard_normal((max(n, 1), HKV, D)).astype(np.float32); v = rng.standard_normal((max(n, 1), HKV, D)).astype(np.float32)
            dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda(); keep.append((dk, dv))
            r = both("cf_llama_server_append_layer_async", i64(s), layer, 0, C.c_void_p(dk.data_ptr()), C.c_void_p(dv.data_ptr()), n, None)
            if r == (0, 0): rows[(s, layer)] = (k[:n], v[:n])
        elif op == "execute":
            cand = [key for key in rows if key[0] in live and key[0] not in cancelled]
            if not cand and rng.random() < 0.8: continue
            picks = [cand[i] for i in rng.choice(len(cand), int(rng.integers(1, min(3, len(cand)) + 1)), replace=False)] if cand else [(int(rng.integers(1, 9)), 0)]
            if rng.random() < 0.1: picks.append((int(rng.integers(20, 30)), 0))
            outs = []
            for lib, x in zip(libs, rs):
                rng2 = np.random.default_rng(seed * 977 + step)
                items = (MsBatchItem * len(picks))(); ods = []
                for i, (s, layer) in enumerate(picks):
                    tot = rows[(s, layer)][0].shape[0] if (s, layer) in rows else 1
                    q = rng2.standard_normal((1, HQ, D)).astype(np.float32); qd = torch.from_numpy(q).cuda(); od = torch.zeros((1, HQ, D), dtype=torch.float32, device="cuda"); keep.append((qd, od)); ods.append(od)
                    items[i].sequence_id, items[i].layer = s, layer
                    items[i].query = TensorView(qd.data_ptr(), 3, 1, HQ, D, HQ * D * 4, D * 4, 4, 0)
                    items[i].output, items[i].output_type = od.data_ptr(), 3
                    items[i].output_token_stride_bytes, items[i].output_head_stride_bytes, items[i].output_element_stride_bytes = HQ * D * 4, D * 4, 4
                    items[i].query_token_begin, items[i].softmax_scale, items[i].causal_window = tot - 1, scale, 0
                batch = LlamaServerBatch(None, 0, C.cast(items, C.c_void_p), len(picks))
                rc = lib.cf_llama_server_execute_batch_async(x, C.byref(batch), None); torch.cuda.synchronize()
                outs.append((rc, [o.cpu().numpy() for o in ods]))
            log.append(("execute", (outs[0][0], outs[1][0]), picks))
            if outs[0][0] != outs[1][0]: return ("status", log[-6:], libs[0].cf_llama_server_last_error(rs[0]), libs[1].cf_llama_server_last_error(rs[1])), what
            if outs[0][0] == 0:
                for a, b in zip(outs[0][1], outs[1][1]):
                    e = np.abs(a - b).max() / (np.abs(b).max() + 1e-30)
                    if not np.isfinite(a).all() or e > 2e-5: return ("attention", float(e), log[-3:]), what     # only unsealed fp32 rows here: the same numbers
            continue
        elif op == "copy":
            s = pick(); t = int(rng.integers(30, 60))
            r = both("cf_llama_server_sequence_copy_async", i64(s), i64(t), C.c_uint32(0), C.c_uint32(1 << 30), None)
            if r == (0, 0):
                live.add(t)
                for layer in range(LAYERS):
                    if (s, layer) in rows: rows[(t, layer)] = rows[(s, layer)]
                if s in cancelled: cancelled.add(t) if False else None
        elif op == "reset":
            s = pick(); r = both("cf_llama_server_slot_reset_async", i64(s), None)
            if r == (0, 0):
                live.discard(s); cancelled.discard(s)
                for layer in range(LAYERS): rows.pop((s, layer), None)
        elif op == "cancel":
            if rng.random() < 0.6: continue
            s = pick(); r = both("cf_llama_server_cancel_async", i64(s), None)
            if r == (0, 0): cancelled.add(s)
        elif op == "remove_range":
            s = pick()
            if any((s, layer) in rows for layer in range(LAYERS)): continue    # host bookkeeping only in the reference: rows stay staged there
            lo = int(rng.integers(0, 40)); r = both("cf_llama_server_sequence_remove_async", i64(s), i64(lo), i64(lo + int(rng.integers(0, 40))), None)
        elif op == "shift":
            s = pick()
            if any((s, layer) in rows for layer in range(LAYERS)): continue
            r = both("cf_llama_server_sequence_shift_async", i64(s), C.c_uint32(0), C.c_uint32(1 << 30), C.c_int32(int(rng.integers(0, 30))), None)
        else:
            if rng.random() < 0.85: continue
            r = both("cf_llama_server_shutdown_async", None); shut = True; live.clear(); rows.clear()
        if r[0] != r[1]: return ("status", log[-6:], libs[0].cf_llama_server_last_error(rs[0]), libs[1].cf_llama_server_last_error(rs[1])), what
    if not shut:
        r = both("cf_llama_server_shutdown_async", None)
        if r[0] != r[1]: return ("shutdown", r), what
    sa, sb = LlamaServerStats(), LlamaServerStats()
    libs[0].cf_llama_server_get_stats(rs[0], C.byref(sa)); libs[1].cf_llama_server_get_stats(rs[1], C.byref(sb))
    diff = {n: (int(getattr(sa, n)), int(getattr(sb, n))) for n, _ in LlamaServerStats._fields_ if getattr(sa, n) != getattr(sb, n)}
    for l, x in zip(libs, rs): l.cf_llama_server_runtime_destroy(x, None)
    return (("stats", diff), what) if diff else (None, what)


@pytest.mark.parametrize("first", range(0, 16, 8))
def test_llama_server_runtime_answers_like_the_references_own(native, oracle, first):
    """cf_llama_server_* here and in the reference (src/llama_server_runtime.cpp over its host cache and resolver, compiled
    into oracle/_ref): slots created, reset and cancelled, layers appended, sequences copied, ranges removed and shifted,
    batches executed (unknown sequences too), shutdown. Same status for every call, equal statistics, and the same
    attention to 2e-5 (the rows stay unsealed fp32 in both). The runs stay where the two mean the same: one append of
    less than a page per layer (the reference restages a tail where this library appends to it and seals full pages),
    ranges removed or shifted only on sequences without rows (host bookkeeping only in the reference)."""
    if oracle.ref_device() is None:
        pytest.skip("needs the reference's llama-server runtime (oracle/_ref)")
    for seed in range(first, first + 8):
        bad, what = _server_side_by_side(native, oracle, seed, 60)
        assert bad is None, (bad, what)


# ---- the tensor-view validator and the dataplane's appends beside the reference's own ---------------------------------
def _random_tensor_views(rng, n):
    """Tensor views with every field drawn from a few values, most of them invalid one way or another."""
    from compat_types import TensorView
    out = []
    for _ in range(n):
        t = int(rng.choice([0, 1, 2, 3, 4, 7])); tok = int(rng.choice([0, 1, 5, 64])); h = int(rng.choice([0, 1, 2, 8])); d = int(rng.choice([0, 1, 64, 128, 129]))
        es = int(rng.choice([0, 1, 2, 4, 8])); hs = int(rng.choice([0, es * d, es * d + 16, 3])); ts = int(rng.choice([0, hs * h, hs * h + 32, 5]))
        data = int(rng.choice([0, 0x7f0000001000, 0x7f0000001001, 0x7f0000001002, 0x7f0000001004]))
        out.append(TensorView(data, t, tok, h, d, ts, hs, es, int(rng.choice([0, 0, 1]))))
    return out


def _dataplane_side_by_side(native, oracle, seed):
    import ctypes as C
    import torch
    from compat_types import DeviceKvConfig, TensorView
    rng = np.random.default_rng(seed)
    libs = [native.lib(), oracle.ref_device()]
    for v in _random_tensor_views(rng, 400):
        a, b = libs[0].cf_device_tensor_validate(C.byref(v)), libs[1].cf_device_tensor_validate(C.byref(v))
        if a != b: return ("validate", a, b, [getattr(v, n) for n, _ in TensorView._fields_]), seed
    for l in libs: l.cf_device_kv_create.restype = C.c_void_p
    layers = int(rng.integers(1, 3)); hkv = int(rng.choice([1, 2, 4])); group = int(rng.choice([1, 4])); hq = hkv * group; d = int(rng.choice([64, 128])); page = int(rng.choice([16, 32]))
    cfg = DeviceKvConfig(layers, hkv, hq, d, page, group, 0)
    ps = [C.c_void_p(l.cf_device_kv_create(C.byref(cfg))) for l in libs]
    if bool(ps[0].value) != bool(ps[1].value): return ("create",), seed
    rows = torch.zeros((page, hkv, d), dtype=torch.float32, device="cuda")
    count = [0] * layers; begin = [0] * layers; log = []
    for step in range(40):
        layer = int(rng.integers(0, layers + 1)); L = min(layer, layers - 1)
        n = int(rng.integers(0, page + 2)); c = count[L]
        if c + n == page: n += 1       # an exactly full page: the reference's seal is a stub that fails, this library seals
        n = min(n, page)
        if c + n == page: continue
        where = begin[L] + c if (c or rng.random() < 0.6) else int(rng.integers(0, 90))
        if rng.random() < 0.1: where += int(rng.integers(1, 4))
        hv = hkv if rng.random() < 0.9 else hkv + 1
        view = TensorView(rows.data_ptr(), 3, n, hv, d, hv * d * 4, d * 4, 4, 0)
        r = tuple(l.cf_device_kv_append_async(p, layer, where, C.byref(view), C.byref(view), None) for l, p in zip(libs, ps))
        log.append((layer, where, n, hv, "count", c, r))
        if r[0] != r[1]: return ("append", log[-5:]), seed
        if r == (0, 0) and layer < layers:
            if c == 0: begin[L] = where
            count[L] = c + n
    for l, p in zip(libs, ps): l.cf_device_kv_destroy(p, None)
    return None, seed


@pytest.mark.parametrize("first", range(0, 20, 10))
def test_tensor_validator_and_dataplane_appends_answer_like_the_references_own(native, oracle, first):
    """cf_device_tensor_validate on 400 random views per run and cf_device_kv_append_async on random appends (layers that
    do not exist, gaps, page-boundary crossings, wrong head counts, a first append anywhere), here and in the reference
    (src/cuda/device_kv_dataplane.cu in oracle/_ref): the same answer for every call. No page is filled exactly: the
    reference's seal is a stub that fails, this library seals."""
    if oracle.ref_device() is None:
        pytest.skip("needs the reference's dataplane (oracle/_ref)")
    for seed in range(first, first + 10):
        bad, what = _dataplane_side_by_side(native, oracle, seed)
        assert bad is None, (bad, what)


# ---- the llama KV adapter beside the reference's own, end to end -------------------------------------------------------
def _adapter_side_by_side(native, oracle, seed):
    import ctypes as C
    import torch
    from compat_types import LlamaKvOptions, LlamaKvStats
    from test_gpu_compat import _dev
    rng = np.random.default_rng(seed)
    libs = [native.lib(), oracle.ref_adapter()]
    for l in libs: l.cf_llama_kv_create.restype = C.c_void_p; l.cf_llama_kv_last_error.restype = C.c_char_p
    hq, hkv = [(14, 2), (8, 8), (4, 2), (32, 8), (16, 2), (1, 1)][int(rng.integers(0, 6))]
    head_dim = int(rng.choice([32, 64, 96, 128, 128])); page = int(rng.choice([16, 32, 64])); layers = int(rng.integers(1, 3))
    o = LlamaKvOptions(); o.struct_size, o.backend = C.sizeof(o), 1
    o.layer_count, o.kv_head_count, o.query_head_count, o.head_dim, o.page_size, o.gqa_group_size = layers, hkv, hq, head_dim, page, hq // hkv
    o.kv_bits = int(rng.choice([0, 4, 8, 8]))
    if rng.random() < 0.1: o.gqa_group_size += 1
    what = dict(seed=seed, heads=(hq, hkv), d=head_dim, page=page, layers=layers, bits=int(o.kv_bits))
    v = tuple(l.cf_llama_kv_options_validate(C.byref(o)) for l in libs)
    if v[0] != v[1]: return ("validate", v), what
    hs = [C.c_void_p(l.cf_llama_kv_create(C.byref(o))) for l in libs]
    if bool(hs[0].value) != bool(hs[1].value): return ("create", bool(hs[0].value), bool(hs[1].value)), what
    if not hs[0].value: return None, what
    log = []
    def both(name, *args):
        r = tuple(getattr(l, name)(h, *args) for l, h in zip(libs, hs)); log.append((name, r)); return r
    p = lambda x: np.ascontiguousarray(x).ctypes.data_as(C.c_void_p)
    tokens = int(rng.integers(1, 4 * page + 10))
    k = rng.standard_normal((layers, hkv, tokens, head_dim)).astype(np.float32) * float(10.0 ** rng.uniform(-2, 1))
    vv = rng.standard_normal((layers, hkv, tokens, head_dim)).astype(np.float32) * float(10.0 ** rng.uniform(-3, 2))
    cuts = sorted(set([0, tokens] + [int(x) for x in rng.integers(0, tokens + 1, int(rng.integers(0, 4)))]))
    for layer in range(layers):
        for b, e in zip(cuts[:-1], cuts[1:]):
            for h in range(hkv):
                begin = b if (rng.random() < 0.95 or b % page == 0) else b + 3       # now and then a gap inside a page: both must refuse
                r = both("cf_llama_kv_append", layer, h, begin, p(k[layer, h, b:e]), p(vv[layer, h, b:e]), e - b, None); log[-1] += (layer, h, begin, e - b)
                if r[0] != r[1]: return ("append", log[-4:], libs[0].cf_llama_kv_last_error(hs[0]), libs[1].cf_llama_kv_last_error(hs[1])), what
                if r[0] != 0:    # the gap was refused: append the piece where it belongs
                    r = both("cf_llama_kv_append", layer, h, b, p(k[layer, h, b:e]), p(vv[layer, h, b:e]), e - b, None)
                    if r[0] != r[1]: return ("append after refusal", r), what
                    if r[0] != 0:      # both refuse alike (a head that took rows at the wrong place keeps them): end of this run
                        for l, h in zip(libs, hs): l.cf_llama_kv_destroy(h)
                        return None, what
    def stats():
        out = []
        for l, h in zip(libs, hs):
            st = LlamaKvStats(); rc = l.cf_llama_kv_get_stats(h, C.byref(st)); out.append((rc,) + tuple(int(getattr(st, n)) for n in ("appended_tokens", "sealed_tokens", "sealed_pages", "active_tokens")))
        return out
    s = stats()
    if s[0] != s[1]: return ("stats", s), what
    for rounds in range(2):
        nq = int(rng.integers(1, min(4, tokens) + 1)); window = int(rng.integers(1, tokens + 4)) if rng.random() < 0.5 else 0
        q = rng.standard_normal((nq, hq, head_dim)).astype(np.float32); d_q = _dev(q)
        layer = int(rng.integers(0, layers + 1)); outs = []
        for l, h in zip(libs, hs):
            out = torch.zeros((nq, hq, head_dim), dtype=torch.float32, device="cuda")
            rc = l.cf_llama_kv_attention(h, layer, C.c_void_p(d_q.data_ptr()), C.c_void_p(out.data_ptr()), nq, hq, hq // hkv, tokens - nq, C.c_float(1.0 / np.sqrt(head_dim)), window, None)
            torch.cuda.synchronize(); host = np.zeros((nq, hq, head_dim), np.float32)
            rc2 = l.cf_llama_kv_attention_host(h, layer, p(q), p(host), nq, hq, hq // hkv, tokens - nq, C.c_float(1.0 / np.sqrt(head_dim)), window, None)
            outs.append((rc, rc2, out.cpu().numpy(), host))
        if (outs[0][0], outs[0][1]) != (outs[1][0], outs[1][1]): return ("attention status", outs[0][:2], outs[1][:2], layer, libs[1].cf_llama_kv_last_error(hs[1]), dict(nq=nq, window=window, tokens=tokens, cuts=cuts)), what
        if outs[0][0] == 0:
            for j in (2, 3):
                e = np.abs(outs[0][j] - outs[1][j]).max() / (np.abs(outs[1][j]).max() + 1e-30)
                if not np.isfinite(outs[0][j]).all() or e > 2e-4: return ("attention", j, float(e)), what
        if rounds == 0 and rng.random() < 0.5:
            r = both("cf_llama_kv_flush", None)
            if r[0] != r[1]: return ("flush", r), what
            s = stats()
            if s[0] != s[1]: return ("stats after flush", s), what
    for name, args in (("cf_llama_kv_seq_cp", (0, 1)), ("cf_llama_kv_seq_cp", (0, 0)), ("cf_llama_kv_seq_shift", (0, 0)), ("cf_llama_kv_seq_shift", (0, 1)), ("cf_llama_kv_seq_rm", (1,)), ("cf_llama_kv_seq_rm", (0,))):
        if rng.random() < 0.5: continue
        r = both(name, *args)
        if r[0] != r[1]: return (name, args, r), what
    s = stats()
    if s[0] != s[1]: return ("stats at the end", s), what
    for l, h in zip(libs, hs): l.cf_llama_kv_destroy(h)
    return None, what


@pytest.mark.parametrize("first", range(0, 24, 12))
def test_llama_kv_adapter_answers_like_the_references_own(native, oracle, first, monkeypatch):
    """cf_llama_kv_* here and in the reference, end to end (its adapter over its CompressedKvCache, quantiser and
    paged-attention kernel, compiled into oracle/_ref): options (valid or not), appends in random pieces with a gap now
    and then, statistics, device and host attention on one to three query rows with or without a window (layers that do
    not exist too), flush, the sequence calls. Same status for every call, equal statistics, outputs equal to 2e-4 of
    their scale. Gaps are tried inside a page only: at a page boundary the reference takes any position for the next
    rows, this library only the next one."""
    if oracle.ref_adapter() is None:
        pytest.skip("needs the reference's adapter (oracle/_ref)")
    monkeypatch.delenv("CHROMOFOLD_B200_CODER", raising=False)
    for seed in range(first, first + 12):
        bad, what = _adapter_side_by_side(native, oracle, seed)
        assert bad is None, (bad, what)


# ---- the multi-GPU admission runtime and the delta fetch beside the reference's own -----------------------------------
def _multigpu_runtime_side_by_side(native, oracle, seed):
    import ctypes as C
    import torch
    from compat_types import MultigpuCounters, MultigpuDeviceConfig, MultigpuPageView, MultigpuRuntimeConfig, MultigpuShard
    rng = np.random.default_rng(seed)
    libs = [native.lib(), oracle.ref_device()]
    for l in libs: l.cf_multigpu_cuda_create.restype = C.c_void_p; l.cf_multigpu_cuda_last_error.restype = C.c_char_p
    ndev = int(rng.integers(1, 5))
    ords = [int(x) for x in rng.choice(6, ndev, replace=rng.random() < 0.1)]
    if rng.random() < 0.8 and 0 not in ords: ords[0] = 0
    devs = (MultigpuDeviceConfig * ndev)(*[MultigpuDeviceConfig(o if rng.random() < 0.95 else -1, int(rng.choice([0, 1 << 30])) if rng.random() < 0.1 else 1 << 30, 0) for o in ords])
    cfg = MultigpuRuntimeConfig(C.cast(devs, C.c_void_p), ndev, int(rng.integers(1, 4)), int(rng.integers(1, 5)), int(rng.integers(0, 2)), int(rng.integers(0, 2)), int(rng.integers(0, 3)))
    hs = [C.c_void_p(l.cf_multigpu_cuda_create(C.byref(cfg))) for l in libs]
    what = dict(seed=seed, ords=ords, tp=cfg.tensor_parallel_size, layers=cfg.layer_count)
    if bool(hs[0].value) != bool(hs[1].value): return ("create", bool(hs[0].value), bool(hs[1].value)), what
    if not hs[0].value: return None, what
    buf = torch.zeros(4096, dtype=torch.uint8, device="cuda"); ptr = buf.data_ptr()
    log = []
    for step in range(int(rng.integers(3, 20))):
        op = ["execute", "execute", "execute", "migrate", "inject", "shutdown"][int(rng.integers(0, 6))]
        if op == "execute":
            n = int(rng.integers(1, 4)); shards = (MultigpuShard * n)(); keep = []
            for i in range(n):
                npages = int(rng.integers(0, 4)) if rng.random() < 0.15 else int(rng.integers(1, 4))
                dim = int(rng.choice([64, 128]))
                pages = (MultigpuPageView * max(npages, 1))()
                for j in range(npages):
                    pages[j] = MultigpuPageView(ptr if rng.random() < 0.95 else None, ptr, ptr, ptr, 1024, 1024, int(rng.choice([4, 4, 4, 8, 1, 0, 9])), int(rng.choice([4, 4, 8, 2])),
                                                int(rng.choice([16, 16, 0])), 2, dim if rng.random() < 0.95 else dim + 1, 32, 0, 1)
                keep.append(pages)
                shards[i] = MultigpuShard(int(rng.integers(1, 9)), int(rng.integers(0, cfg.layer_count + 1)) if rng.random() < 0.2 else 0, 0, int(rng.integers(0, 3)) if rng.random() < 0.1 else 4,
                                          0 if rng.random() < 0.9 else int(rng.choice([7, -1])), ptr if rng.random() < 0.95 else None, ptr, 3, 3, dim, npages, C.cast(pages, C.c_void_p))
            r = tuple(l.cf_multigpu_cuda_execute_async(h, shards, n, None) for l, h in zip(libs, hs))
        elif op == "migrate":
            pages = (MultigpuPageView * 2)(); src = int(rng.choice([0, 1])); dst = int(rng.choice([0, 1, 2]))
            for j in range(2): pages[j] = MultigpuPageView(ptr, ptr if rng.random() < 0.9 else None, ptr, ptr, 64, 64, 4, 4, 16, 2, 64, 32, src if rng.random() < 0.9 else 5, 1)
            count = int(rng.integers(0, 3))
            r = tuple(l.cf_multigpu_cuda_migrate_sequence_async(h, C.c_uint64(3), src, dst, pages, count, None) for l, h in zip(libs, hs))
        elif op == "inject":
            if rng.random() < 0.7: continue
            o = int(rng.choice(ords + [9])); r = tuple(l.cf_multigpu_cuda_inject_device_failure(h, o) for l, h in zip(libs, hs))
        else:
            if rng.random() < 0.8: continue
            r = tuple(l.cf_multigpu_cuda_shutdown(h) for l, h in zip(libs, hs))
        log.append((op, r))
        if r[0] != r[1]: return ("status", log[-5:], libs[0].cf_multigpu_cuda_last_error(hs[0]), libs[1].cf_multigpu_cuda_last_error(hs[1])), what
    ka, kb = MultigpuCounters(), MultigpuCounters()
    libs[0].cf_multigpu_cuda_get_counters(hs[0], C.byref(ka)); libs[1].cf_multigpu_cuda_get_counters(hs[1], C.byref(kb))
    diff = {n: (int(getattr(ka, n)), int(getattr(kb, n))) for n, _ in MultigpuCounters._fields_ if getattr(ka, n) != getattr(kb, n)}
    for l, h in zip(libs, hs): l.cf_multigpu_cuda_destroy(h)
    return (("counters", diff, log[-4:]), what) if diff else (None, what)


def _delta_fetch_side_by_side(native, oracle, seed):
    """A random reference/delta cluster (sorted override positions per member, some past the base's end) and random
    queries, through cf_delta_fetch_async here and in the reference (src/cuda/delta_apply.cu): the same tokens."""
    import ctypes as C
    import torch
    rng = np.random.default_rng(seed)
    nbase, members = int(rng.integers(1, 5000)), int(rng.integers(1, 200))
    base = rng.integers(0, 50000, nbase).astype(np.int32)
    lens = rng.integers(0, min(nbase, 60) + 1, members).astype(np.int32)
    if rng.random() < 0.3:
        lens[:] = 0
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]]).astype(np.int32)
    dpos = np.concatenate([np.sort(rng.choice(nbase + 50, int(n), replace=False)) for n in lens] + [np.zeros(1)]).astype(np.int32)
    dval = rng.integers(0, 50000, dpos.size).astype(np.int32)
    count = int(rng.integers(1, 20000))
    leaf = rng.integers(0, members, count).astype(np.int32)
    pos = rng.integers(0, nbase + 100, count).astype(np.int32)
    dev = [torch.from_numpy(x).cuda() for x in (base, dpos, dval, starts, lens, leaf, pos)]
    outs = []
    for lib in (native.lib(), oracle.ref_device()):
        lib.cf_delta_fetch_async.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 7 + [C.c_size_t, C.c_void_p]
        out = torch.full((count,), -7, dtype=torch.int32, device="cuda")
        rc = lib.cf_delta_fetch_async(dev[0].data_ptr(), nbase, dev[1].data_ptr(), dev[2].data_ptr(), dev[3].data_ptr(), dev[4].data_ptr(),
                                      dev[5].data_ptr(), dev[6].data_ptr(), out.data_ptr(), count, None)
        torch.cuda.synchronize()
        outs.append((rc, out.cpu().numpy()))
    if outs[0][0] != outs[1][0] or not np.array_equal(outs[0][1], outs[1][1]):
        return ("delta fetch", outs[0][0], outs[1][0], int((outs[0][1] != outs[1][1]).sum())), dict(seed=seed, nbase=nbase, members=members)
    return None, None


@pytest.mark.parametrize("first", range(0, 60, 30))
def test_multigpu_runtime_and_delta_fetch_answer_like_the_references_own(native, oracle, first):
    """cf_multigpu_cuda_* (create with valid and invalid device lists, execute with valid and invalid shards and pages,
    migrate, injected device failures, shutdown; local pages on device 0, so that neither side needs a second GPU) and
    cf_delta_fetch_async, here and in the reference (oracle/_ref): same status for every call, equal counters, the same
    fetched tokens."""
    if oracle.ref_device() is None:
        pytest.skip("needs the reference's sources compiled (oracle/_ref)")
    for seed in range(first, first + 30):
        bad, what = _multigpu_runtime_side_by_side(native, oracle, seed)
        assert bad is None, (bad, what)
        bad, what = _delta_fetch_side_by_side(native, oracle, seed)
        assert bad is None, (bad, what)
