"""The benchmark configurations as parity cases (seeded synthetic inputs with their shapes and distributions), through
the C ABI, against the CPU oracle reading the same sealed bytes. Config 2 runs at its full size."""
import numpy as np
import pytest

from helpers import attention_close, oracle_from_layer

pytestmark = pytest.mark.gpu


def _q(n, hq, seed):
    import torch
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return torch.randn((n, hq, 128), generator=g, device="cuda", dtype=torch.float32).half()


def test_config1_plumbing_single_sequence_mha(native, oracle):
    """1 sequence, 8 = 8 heads, head_dim 128, 4096 tokens, K/V fp16 N(0,1) quantised with per-page-per-head fp16 absmax
    scales, rANS pages. Codes decoded on the GPU equal the CPU quantiser's codes; outputs match the oracle."""
    import torch
    from chromofold_b200.cache import SealedKvLayer
    rng = np.random.default_rng(1)
    layer = SealedKvLayer(kv_heads=8, query_heads=8, max_sequences=1, max_pages_per_sequence=258, max_pages=260,
                          arena_bytes=260 * 8 * 4200, coder=native.CODER_RANS)
    k = rng.standard_normal((256, 8, 16, 128)).astype(np.float16)
    v = rng.standard_normal((256, 8, 16, 128)).astype(np.float16)
    rc, bits, codes = oracle.quantize_stream(k[0, 0].astype(np.float32))
    hist = np.bincount(codes.astype(np.int64) + 128, minlength=256).astype(np.uint64) + 1
    layer.set_codebooks(hist, hist)
    layer.seal_tiles([0] * 256, torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda())
    assert layer.device_status() == 0
    ks, vs = layer.decode_pages([1, 100, 256])
    for i, p in enumerate((0, 99, 255)):
        for h in (0, 7):
            rc, bits, codes = oracle.quantize_stream(k[p, h].astype(np.float32))
            assert np.array_equal(ks[i, h].cpu().numpy(), (codes.astype(np.int16) + 128).astype(np.uint8))
            rc, bits, codes = oracle.quantize_stream(v[p, h].astype(np.float32))
            assert np.array_equal(vs[i, h].cpu().numpy().reshape(128, 16).T.ravel(), (codes.astype(np.int16) + 128).astype(np.uint8))
    q = _q(1, 8, 2)
    want = oracle_from_layer(layer, q.cpu().numpy())
    for kernel in (native.KERNEL_LANES, native.KERNEL_GENERIC):
        ok, err = attention_close(layer.attention(q, kernel=kernel).cpu().numpy(), want)
        assert ok, (kernel, err)
    # N(0,1) scaled by absmax/127 has H0 ~ 7.2 bits: entropy coding buys little, as the reference found
    assert 0.80 < layer.sealed_bytes() / (4096 * 8 * 2 * 128) < 1.01


def test_config2_llama8b_full_size(native, oracle):
    """64 sequences, contexts U[2048, 32768], 32/8 heads, Laplace(b=12) codes, rANS pages — the benchmark workload at
    full size (1.8 GB of sealed pages); every sequence checked against the oracle."""
    from chromofold_b200.workloads import build_sealed_layer, uniform_contexts
    contexts = uniform_contexts(64, 2048, 32768, 16, 3)
    layer, info = build_sealed_layer(contexts, coder="rans", dist=("laplace", 12.0), seed=4)
    assert 5.9 < info["h0_bits_k"] < 6.2 and 1650 < info["bytes_per_seq_token"] < 1850
    q = _q(64, 32, 5)
    got = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
    assert layer.device_status() == 0
    want = oracle_from_layer(layer, q.cpu().numpy())
    ok, err = attention_close(got, want)
    assert ok, err


@pytest.mark.parametrize("p", [0.05, 0.1, 0.2, 0.4, 0.7])
def test_config3_coder_crossover(native, oracle, p):
    """Two-sided geometric codes at five entropies, each sealed with rANS and with Huffman: parity for both, and both
    stay below the fixed-width size."""
    from chromofold_b200.workloads import build_sealed_layer
    sizes = {}
    for coder in ("rans", "huffman"):
        layer, info = build_sealed_layer(np.array([512, 1024, 256]), coder=coder, dist=("geometric", p), seed=6)
        q = _q(3, 32, 7)
        got = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
        ok, err = attention_close(got, oracle_from_layer(layer, q.cpu().numpy()))
        assert ok and layer.device_status() == 0, (coder, err)
        sizes[coder] = info["bytes_per_seq_token"]
    assert sizes["rans"] < 2056 and sizes["huffman"] < 2056
    if p >= 0.4:
        assert sizes["huffman"] < sizes["rans"] * 1.25    # block-64 state overhead keeps rANS from winning big


def test_config4_gqa8_kv_head_sharding(native, oracle):
    """70B shape (64 query / 8 kv heads): kv heads sharded 1, 2, 4 and 8 ways, each shard a separate launch over its
    kv_head_begin / kv_head_span; the union of the shards' head blocks equals the unsharded result."""
    import torch
    from chromofold_b200.scheduler import shard_kv_heads
    from chromofold_b200.workloads import build_sealed_layer
    layer, _ = build_sealed_layer(np.array([2048, 1536]), query_heads=64, kv_heads=8, coder="rans", seed=8)
    q = _q(2, 64, 9)
    want = oracle_from_layer(layer, q.cpu().numpy())
    whole = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
    ok, err = attention_close(whole, want)
    assert ok, err
    for ways in (2, 4, 8):
        merged = torch.zeros((2, 64, 128), device="cuda")
        for begin, span in shard_kv_heads(8, ways):
            part = layer.attention(q, kernel=native.KERNEL_LANES, kv_head_begin=begin, kv_head_span=span)
            merged[:, begin * 8:(begin + span) * 8] = part[:, begin * 8:(begin + span) * 8]
        assert np.array_equal(merged.cpu().numpy(), whole)       # sharding changes nothing, bit for bit
    assert layer.device_status() == 0


def test_config5_shared_prefix_with_gpu_sealed_suffixes(native, oracle):
    """Sequences sharing one sealed prefix (one copy of its pages, referenced from every page table) plus private
    suffixes that grow by one token per step and are sealed on the GPU whenever 16 tokens have accumulated."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    n, prefix = 12, 1024
    layer, info = build_sealed_layer(np.array([prefix] + [0] * (n - 1)), coder="rans", seed=10, extra_pages_per_sequence=8)
    bytes_one_copy = layer.sealed_bytes()
    for s in range(1, n):
        layer.copy_sequence(0, s)
    assert layer.sealed_bytes() == bytes_one_copy                # sharing copies no page
    g = torch.Generator(device="cuda")
    g.manual_seed(11)
    slots = list(range(n))
    for step in range(37):
        k = (torch.randn((n, 8, 128), generator=g, device="cuda") * 0.7).half()
        v = (torch.randn((n, 8, 128), generator=g, device="cuda") * 0.7).half()
        layer.append(slots, k, v)
        if step in (4, 15, 36):
            q = _q(n, 32, 100 + step)
            got = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
            ok, err = attention_close(got, oracle_from_layer(layer, q.cpu().numpy()))
            assert ok, (step, err)
            assert not np.allclose(got[0], got[1])               # private suffixes differ
        layer.seal_full_pages()
    assert layer.device_status() == 0
    assert int(layer.h_sealed[3]) == prefix + 32 and int(layer.h_tail[3]) == 5
    assert np.array_equal(layer.h_page_table[0, :prefix // 16], layer.h_page_table[7, :prefix // 16])
    assert layer.h_page_table[0, prefix // 16] != layer.h_page_table[7, prefix // 16]


@pytest.mark.parametrize("coder", ["rans", "huffman", "fixed8", "rans4", "huffman4"])
@pytest.mark.parametrize("heads", [(32, 8), (64, 8), (8, 8)], ids=str)
def test_shared_prefix_is_decoded_once_for_all_sequences(native, oracle, coder, heads):
    """The shared-prefix kernel: with the hint the sealed prefix pages are decoded once per 128 query rows and
    contracted with every sequence's queries on the tensor cores; results must equal the per-sequence path within
    the attention tolerance and the oracle's."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    hq, hkv = heads
    n, prefix = 21, 1616                      # 101 shared pages: not a multiple of the 8-page round
    layer, info = build_sealed_layer(np.array([prefix] + [0] * (n - 1)), query_heads=hq, kv_heads=hkv, coder=coder,
                                     seed=70, extra_pages_per_sequence=8, reserve_pages=4 * n)
    for s in range(1, n):
        layer.copy_sequence(0, s)
    g = torch.Generator(device="cuda")
    g.manual_seed(71)
    slots = list(range(n))
    for step in range(21):                    # one sealed private page and a 5-token tail per sequence
        k = (torch.randn((n, hkv, 128), generator=g, device="cuda") * 0.7).half()
        v = (torch.randn((n, hkv, 128), generator=g, device="cuda") * 0.7).half()
        layer.append(slots, k, v)
        layer.seal_full_pages()
    q = _q(n, hq, 72)
    plain = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
    shared = layer.attention(q, kernel=native.KERNEL_LANES, shared_prefix_pages=prefix // 16).cpu().numpy()
    assert layer.device_status() == 0
    ok, err = attention_close(shared, plain)
    assert ok, err
    ok, err = attention_close(shared, oracle_from_layer(layer, q.cpu().numpy()))
    assert ok, err
    # a shorter claim is fine too (the rest of the prefix is then handled per sequence)
    part = layer.attention(q, kernel=native.KERNEL_LANES, shared_prefix_pages=40).cpu().numpy()
    ok, err = attention_close(part, plain)
    assert ok, err
    # a subset of the sequences, in another order
    some = [5, 0, 17, 9]
    sub = layer.attention(q[:4].contiguous(), slots=some, kernel=native.KERNEL_LANES, shared_prefix_pages=prefix // 16).cpu().numpy()
    ref = layer.attention(q[:4].contiguous(), slots=some, kernel=native.KERNEL_LANES).cpu().numpy()
    ok, err = attention_close(sub, ref)
    assert ok, err
    assert layer.device_status() == 0


@pytest.mark.parametrize("coder", ["rans", "huffman"])
def test_shared_prefix_with_several_units_per_cta(native, oracle, coder):
    """More units than SMs: 16 chunks x 8 kv heads x 3 row tiles (the last one 64 rows) = 384 units, so that a CTA of the
    shared-prefix kernel walks through several units (new Q rows in tensor memory, O started afresh, decoders running
    ahead across the unit boundary). Checked against the per-sequence path on every row and against the oracle on a
    few sequences."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    n, prefix = 80, 5136                       # 321 shared pages: the last chunk's last round holds a single page
    layer, info = build_sealed_layer(np.array([prefix] + [0] * (n - 1)), coder=coder, seed=90, extra_pages_per_sequence=4,
                                     reserve_pages=2 * n)
    for s in range(1, n):
        layer.copy_sequence(0, s)
    g = torch.Generator(device="cuda")
    g.manual_seed(91)
    slots = list(range(n))
    for step in range(19):                     # one sealed private page and a 3-token tail per sequence
        k = (torch.randn((n, 8, 128), generator=g, device="cuda") * 0.7).half()
        v = (torch.randn((n, 8, 128), generator=g, device="cuda") * 0.7).half()
        layer.append(slots, k, v)
        layer.seal_full_pages()
    q = _q(n, 32, 92)
    plain = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
    shared = layer.attention(q, kernel=native.KERNEL_LANES, shared_prefix_pages=prefix // 16).cpu().numpy()
    assert layer.device_status() == 0
    ok, err = attention_close(shared, plain)
    assert ok, err
    some = [0, 37, 79]
    want = oracle_from_layer(layer, q.cpu().numpy()[some], slots=some)
    ok, err = attention_close(shared[some], want)
    assert ok, err
    again = layer.attention(q, kernel=native.KERNEL_LANES, shared_prefix_pages=prefix // 16).cpu().numpy()
    assert np.array_equal(again, shared)       # the static unit split makes the result repeatable bit for bit


def test_shared_prefix_under_kv_head_sharding_and_fp32_queries(native, oracle):
    """The hint combined with the other launch options: a kv-head shard (each rank of a head-sharded deployment passes
    kv_head_begin / kv_head_span) writes its heads' columns of the unsharded result (to fp32 rounding: how the prefix is
    cut over the CTAs depends on the number of heads, and with it the order the partials merge in); fp32 queries give the
    fp16-query result within tolerance whichever kernel serves them."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    n, prefix = 40, 2048
    layer, info = build_sealed_layer(np.array([prefix] + [0] * (n - 1)), coder="rans", seed=95, extra_pages_per_sequence=4,
                                     reserve_pages=2 * n)
    for s in range(1, n):
        layer.copy_sequence(0, s)
    g = torch.Generator(device="cuda")
    g.manual_seed(96)
    for step in range(5):                       # a private tail of 5 tokens per sequence
        k = (torch.randn((n, 8, 128), generator=g, device="cuda") * 0.7).half()
        v = (torch.randn((n, 8, 128), generator=g, device="cuda") * 0.7).half()
        layer.append(list(range(n)), k, v)
    q = _q(n, 32, 97)
    pages = prefix // 16
    full = layer.attention(q, kernel=native.KERNEL_LANES, shared_prefix_pages=pages).cpu().numpy()
    ok, err = attention_close(full, layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy())
    assert ok, err
    group = 4
    for begin, span in ((0, 2), (2, 2), (4, 4)):
        out = torch.full((n, 32, 128), 7.0, dtype=torch.float32, device="cuda")
        layer.attention(q, out=out, kernel=native.KERNEL_LANES, shared_prefix_pages=pages, kv_head_begin=begin, kv_head_span=span)
        got = out.cpu().numpy()
        lo, hi = begin * group, (begin + span) * group
        assert np.allclose(got[:, lo:hi], full[:, lo:hi], rtol=1e-5, atol=2e-6)
        assert np.all(got[:, :lo] == 7.0) and np.all(got[:, hi:] == 7.0)      # other heads' columns untouched
    f32 = layer.attention(q.float(), shared_prefix_pages=pages).cpu().numpy()
    ok, err = attention_close(f32, full)
    assert ok, err
    # queries that binary16 cannot hold: both kernels split them into binary16 + residue, the results must agree tightly
    g.manual_seed(98)
    q32 = torch.randn((n, 32, 128), generator=g, device="cuda") * 1.7
    with_hint = layer.attention(q32, shared_prefix_pages=pages).cpu().numpy()
    without = layer.attention(q32).cpu().numpy()
    generic = layer.attention(q32, kernel=native.KERNEL_GENERIC).cpu().numpy()
    assert np.abs(with_hint - generic).max() <= 2e-5 and np.abs(without - generic).max() <= 2e-5
    rounded = layer.attention(q32.half()).cpu().numpy()
    assert np.abs(rounded - generic).max() > 2e-5           # rounding the queries to binary16 would have shown
    assert layer.device_status() == 0


def test_shared_prefix_claim_that_does_not_hold_falls_back(native, oracle):
    """A claim the page tables do not bear out is refused by the plan kernel: the status word says so and the
    result is the per-sequence one."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    layer, info = build_sealed_layer(np.array([512, 512, 512]), coder="rans", seed=73)   # three unrelated sequences
    q = _q(3, 32, 74)
    plain = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
    claimed = layer.attention(q, kernel=native.KERNEL_LANES, shared_prefix_pages=16).cpu().numpy()
    assert np.array_equal(claimed, plain)
    assert layer.device_status() == 0x20


def test_prefill_query_tokens_share_the_sealed_history(native, oracle):
    """Multi-query (prefill) attention over sealed pages: several entries name the same slot at consecutive query
    positions (src/cuda/paged_kv_attention.cu:67-69). With the shared-prefix hint the slot's sealed pages are decoded
    once for all the query tokens; the result equals the per-entry path, and the last position equals a decode step."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    # the empty slots only make the layer's workspace large enough for eleven entries
    layer, info = build_sealed_layer(np.array([2048, 1024] + [0] * 10), coder="rans", seed=80, extra_pages_per_sequence=4)
    g = torch.Generator(device="cuda")
    g.manual_seed(81)
    for step in range(11):                     # an unsealed tail of 11 tokens on both sequences
        k = (torch.randn((2, 8, 128), generator=g, device="cuda") * 0.7).half()
        v = (torch.randn((2, 8, 128), generator=g, device="cuda") * 0.7).half()
        layer.append([0, 1], k, v)
    n = 11
    q = _q(n, 32, 82)
    slots = [0] * n
    positions = torch.arange(2048, 2048 + n, dtype=torch.int32, device="cuda")   # token j of the tail asks as itself
    per_entry = layer.attention(q, slots=slots, kernel=native.KERNEL_LANES, query_positions=positions).cpu().numpy()
    shared = layer.attention(q, slots=slots, kernel=native.KERNEL_LANES, query_positions=positions,
                             shared_prefix_pages=2048 // 16).cpu().numpy()
    assert layer.device_status() == 0
    ok, err = attention_close(shared, per_entry)
    assert ok, err
    assert not np.allclose(shared[0], shared[5])
    # the last query token sees every cached token except none after it: position 2058 = sealed + tail - 1
    decode = layer.attention(q[n - 1:].contiguous(), slots=[0], kernel=native.KERNEL_LANES,
                             query_positions=positions[n - 1:].contiguous()).cpu().numpy()
    ok, err = attention_close(shared[n - 1:], decode)
    assert ok, err
    # a position inside the shared pages makes the claim false for that entry: refused, per-entry result
    early = positions.clone()
    early[3] = 1000
    a = layer.attention(q, slots=slots, kernel=native.KERNEL_LANES, query_positions=early, shared_prefix_pages=128).cpu().numpy()
    b = layer.attention(q, slots=slots, kernel=native.KERNEL_LANES, query_positions=early).cpu().numpy()
    assert np.array_equal(a, b) and layer.device_status() == 0x20


@pytest.mark.parametrize("coder", ["rans", "huffman", "fixed8", "rans4", "huffman4"])
def test_decode_probe_folds_exactly_the_symbols_of_every_page(native, oracle, coder):
    """CF_B200_KERNEL_DECODE_PROBE runs the lanes kernel's fetch + entropy decode without attention and leaves, per
    (chunk, kv head), the XOR of every 4-symbol word it decoded: it must equal the XOR over the symbols the decode
    probe kernel (and the oracle, which that kernel is checked against) recovers from the same pages."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    layer, info = build_sealed_layer(np.array([160, 64]), coder=coder, seed=85)
    q = _q(2, 32, 86)
    layer.attention(q, kernel=native.KERNEL_DECODE_PROBE, stages=native.STAGE_PLAN | native.STAGE_ATTENTION,
                    min_pages_per_unit=16)
    torch.cuda.synchronize()
    assert layer.device_status() == 0
    ws = layer.workspace
    base = (-ws.data_ptr()) % 256
    raw = ws[base:].cpu().numpy()
    header = raw[:64].view(np.uint32)
    chunks, pages_per_unit = int(header[0]), int(header[1])
    assert chunks == 2 and pages_per_unit >= 10                       # one chunk per sequence here
    partials_offset = (64 + 4 * 3 + 255) // 256 * 256
    stride = 130                                                      # floats per (chunk, query head)
    partials = raw[partials_offset:partials_offset + chunks * 32 * stride * 4].view(np.uint32).reshape(chunks, 32, stride)
    for seq, pages in ((0, 10), (1, 4)):
        ks, vs = layer.decode_pages(layer.h_page_table[seq, :pages])
        ks, vs = ks.cpu().numpy(), vs.cpu().numpy()
        for head in range(8):
            want = (np.bitwise_xor.reduce(np.ascontiguousarray(ks[:, head]).view("<u4").ravel()) ^
                    np.bitwise_xor.reduce(np.ascontiguousarray(vs[:, head]).view("<u4").ravel()))
            assert int(partials[seq, head * 4, 0]) == int(want), (seq, head)


@pytest.mark.parametrize("kernel", ["lanes", "generic"])
def test_row_map_serves_a_subset_of_a_batch_in_place(native, kernel):
    """cf_b200_sealed_attention_desc.row_map: two calls, each over half of the batch's sequences with the rows of the
    shared query / output tensors they stand for, give exactly what one call over the whole batch gives (and leave the
    other half's rows alone). Tails included, so the combine kernel's query reads are covered too."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    contexts = np.array([16 * 40, 16 * 3, 16 * 77, 16 * 12, 16 * 150, 16 * 1])
    layer, _ = build_sealed_layer(contexts, query_heads=8, kv_heads=2, coder="rans4", seed=61)
    g = torch.Generator(device="cuda")
    g.manual_seed(62)
    tails = torch.randn((6, 2, 16, 128), generator=g, device="cuda", dtype=torch.float32).half()
    layer.fill_tails(list(range(6)), tails, tails.flip(0).contiguous(), 7)
    q = torch.randn((6, 8, 128), generator=g, device="cuda", dtype=torch.float32).half()
    k = native.KERNEL_LANES if kernel == "lanes" else native.KERNEL_GENERIC
    want = layer.attention(q, kernel=k, min_pages_per_unit=4)
    out = torch.full((6, 8, 128), 7.0, dtype=torch.float32, device="cuda")
    first, second = [4, 0, 3], [5, 2, 1]
    layer.attention(q, slots=first, out=out, kernel=k, min_pages_per_unit=4,
                    row_map=torch.as_tensor(first, dtype=torch.int32, device="cuda"))
    assert torch.equal(out[first], want[first]) and bool((out[second] == 7.0).all())
    layer.attention(q, slots=second, out=out, kernel=k, min_pages_per_unit=4,
                    row_map=torch.as_tensor(second, dtype=torch.int32, device="cuda"))
    assert torch.equal(out, want) and layer.device_status() == 0


def test_a_batch_of_three_thousand_short_sequences(native):
    """More batch entries than the plan kernel keeps in shared memory (2048) and fewer chunks than eight per entry: the
    plan kernel's uncached, thread-per-sequence paths. Lanes kernel against the any-geometry kernel and the oracle."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    contexts = np.array([16 * (1 + i % 5) for i in range(3000)])
    layer, _ = build_sealed_layer(contexts, query_heads=8, kv_heads=2, coder="rans4", seed=81)
    g = torch.Generator(device="cuda")
    g.manual_seed(82)
    q = torch.randn((3000, 8, 128), generator=g, device="cuda", dtype=torch.float32).half()
    fast = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
    slow = layer.attention(q, kernel=native.KERNEL_GENERIC).cpu().numpy()
    assert layer.device_status() == 0
    ok, err = attention_close(fast, slow, rel=1e-3, abs_=5e-4)
    assert ok, err
    ok, err = attention_close(fast, oracle_from_layer(layer, q.cpu().numpy()))
    assert ok, err


def test_shared_prefix_whose_first_page_has_a_tiny_v_scale(native, oracle):
    """The shared-prefix kernel keeps O in units of a V scale and lets each page's scale ride on its binary16 weights.
    A unit whose first page holds almost-zero V rows (scale 2^-24) followed by ordinary pages (scale ~ 0.02) must not
    push those weights past the binary16 range: the result has to equal the per-sequence path's."""
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    n, pages = 8, 24
    layer, info = build_sealed_layer(np.array([0] * n), coder="rans4", seed=120, extra_pages_per_sequence=pages + 2,
                                     reserve_pages=2 * n)
    layer.set_codebooks(np.ones(256, np.uint64), np.ones(256, np.uint64))   # nothing was sealed yet to calibrate on
    g = torch.Generator(device="cuda")
    g.manual_seed(121)
    for t in range(16 * pages):
        k = (torch.randn((1, 8, 128), generator=g, device="cuda") * 0.7).float()
        v = (torch.randn((1, 8, 128), generator=g, device="cuda") * (1e-7 if t < 16 else 0.7)).float()
        layer.append([0], k, v)
        layer.seal_full_pages()
    for s in range(1, n):
        layer.copy_sequence(0, s)
    q = _q(n, 32, 122)
    plain = layer.attention(q, kernel=native.KERNEL_LANES).cpu().numpy()
    shared = layer.attention(q, kernel=native.KERNEL_LANES, shared_prefix_pages=pages).cpu().numpy()
    assert layer.device_status() == 0
    assert np.all(np.isfinite(shared))
    ok, err = attention_close(shared, plain)
    assert ok, err
    ok, err = attention_close(shared, oracle_from_layer(layer, q.cpu().numpy()))
    assert ok, err
