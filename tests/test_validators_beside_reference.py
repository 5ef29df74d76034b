"""The validators and the host-only states of the reference-side ABIs, run beside the reference's own code on the CPU
(its sources compiled into oracle/_ref by oracle/Makefile; no CUDA call is made by either side in these calls): random
arguments, most of them invalid one way or another, must get the same answer from both."""
import ctypes as C

import numpy as np
import pytest

from compat_types import (LlamaGraphCounters, LlamaGraphOptions, LlamaKvOptions, LlamaModelTopology,
                          LlamaRuntimeCounters, LlamaRuntimeOptions, TensorView)


def _kv_options(rng):
    o = LlamaKvOptions()
    o.struct_size = C.sizeof(o) if rng.random() < 0.9 else int(rng.integers(0, 100))
    o.backend = int(rng.choice([0, 1, 1, 1, 2, 7]))
    hkv = int(rng.choice([0, 1, 2, 8]))
    group = int(rng.choice([0, 1, 4, 7, 16, 17, 32]))
    o.layer_count, o.kv_head_count = int(rng.choice([0, 1, 32])), hkv
    o.query_head_count = hkv * group if rng.random() < 0.85 else int(rng.integers(0, 70))
    o.head_dim, o.page_size = int(rng.choice([0, 16, 64, 96, 128, 129, 256])), int(rng.choice([0, 1, 16, 32, 64, 100]))
    o.gqa_group_size, o.kv_bits = group, int(rng.choice([0, 4, 8, 16]))
    return o


def test_option_and_view_validators_answer_like_the_references_own(native, oracle):
    adapter, device = oracle.ref_adapter(), oracle.ref_device()
    if adapter is None or device is None:
        pytest.skip("needs the reference's sources compiled (oracle/_ref)")
    mine = native.lib()
    rng = np.random.default_rng(77)
    for _ in range(4000):
        o = _kv_options(rng)
        assert mine.cf_llama_kv_options_validate(C.byref(o)) == adapter.cf_llama_kv_options_validate(C.byref(o)), \
            [getattr(o, n) for n, _ in LlamaKvOptions._fields_]
        r = LlamaRuntimeOptions()
        r.struct_size = C.sizeof(r) if rng.random() < 0.9 else int(rng.integers(0, 200))
        r.kv = _kv_options(rng)
        r.causal_window, r.require_cuda = int(rng.choice([0, 1, 4096])), int(rng.integers(0, 3))
        r.allow_dense_fallback, r.emit_stats = int(rng.integers(0, 3)), int(rng.integers(0, 2))
        assert mine.cf_llama_runtime_options_validate(C.byref(r)) == adapter.cf_llama_runtime_options_validate(C.byref(r)), \
            ([getattr(r.kv, n) for n, _ in LlamaKvOptions._fields_], r.struct_size, r.causal_window, r.require_cuda,
             r.allow_dense_fallback)
        g = LlamaGraphOptions(C.sizeof(LlamaGraphOptions) if rng.random() < 0.9 else int(rng.integers(0, 64)),
                              int(rng.choice([0, 1, 2, 9])), int(rng.choice([0, 16, 32, 100])), int(rng.choice([0, 1, 512])),
                              int(rng.integers(0, 2)), None if rng.random() < 0.5 else b"evidence.json")
        assert mine.cf_llama_graph_options_validate(C.byref(g)) == adapter.cf_llama_graph_options_validate(C.byref(g)), \
            (g.struct_size, g.backend, g.page_size, g.window)
        hkv = int(rng.choice([0, 1, 2, 8]))
        t = LlamaModelTopology(C.sizeof(LlamaModelTopology) if rng.random() < 0.9 else int(rng.integers(0, 64)),
                               int(rng.choice([0, 1, 32])), hkv * int(rng.choice([0, 1, 4, 16, 17])) if rng.random() < 0.85 else 7,
                               hkv, int(rng.choice([0, 64, 128, 129, 256])), int(rng.choice([0, 1, 4096])),
                               int(rng.integers(0, 2)), int(rng.integers(0, 2)), int(rng.integers(0, 2)))
        assert mine.cf_llama_model_topology_validate(C.byref(t)) == adapter.cf_llama_model_topology_validate(C.byref(t)), \
            [getattr(t, n) for n, _ in LlamaModelTopology._fields_]
        v = TensorView(int(rng.choice([0, 0x7f0000001000, 0x7f0000001001, 0x7f0000001002])), int(rng.choice([0, 1, 2, 3, 4])),
                       int(rng.choice([0, 1, 64])), int(rng.choice([0, 1, 8])), int(rng.choice([0, 64, 128, 129])),
                       int(rng.choice([0, 5, 1024, 4096])), int(rng.choice([0, 3, 128, 512])), int(rng.choice([0, 1, 2, 4, 8])),
                       int(rng.choice([0, 1])))
        assert mine.cf_device_tensor_validate(C.byref(v)) == device.cf_device_tensor_validate(C.byref(v)), \
            [getattr(v, n) for n, _ in TensorView._fields_]
    assert mine.cf_llama_kv_options_validate(None) == adapter.cf_llama_kv_options_validate(None)
    assert mine.cf_device_tensor_validate(None) == device.cf_device_tensor_validate(None)


def test_dense_backend_states_count_like_the_references_own(native, oracle):
    """The graph state and the runtime bridge on the DENSE backend hold no GPU state: create, the record calls and the
    counters must behave the same here and in the reference, call by call."""
    adapter = oracle.ref_adapter()
    if adapter is None:
        pytest.skip("needs the reference's sources compiled (oracle/_ref)")
    libs = [native.lib(), adapter]
    for l in libs:
        l.cf_llama_graph_create.restype = C.c_void_p
        l.cf_llama_runtime_create.restype = C.c_void_p
    rng = np.random.default_rng(78)
    for _ in range(200):
        g = LlamaGraphOptions(C.sizeof(LlamaGraphOptions), 0, int(rng.choice([16, 32])), int(rng.choice([0, 512])), 0, None)
        hkv = int(rng.choice([1, 2, 8]))
        t = LlamaModelTopology(C.sizeof(LlamaModelTopology), int(rng.choice([1, 4])), hkv * int(rng.choice([1, 4])), hkv,
                               int(rng.choice([64, 128])), 4096, int(rng.integers(0, 2)), int(rng.integers(0, 2)), int(rng.integers(0, 2)))
        states = [C.c_void_p(l.cf_llama_graph_create(C.byref(g), C.byref(t))) for l in libs]
        assert bool(states[0].value) == bool(states[1].value), [getattr(t, n) for n, _ in LlamaModelTopology._fields_]
        if not states[0].value:
            continue
        for _ in range(int(rng.integers(1, 12))):
            if rng.random() < 0.5:
                a, b = int(rng.integers(0, 1 << 20)), int(rng.integers(0, 1 << 10))
                r = [l.cf_llama_graph_record_attention(s, C.c_uint64(a), C.c_uint64(b)) for l, s in zip(libs, states)]
            else:
                r = [l.cf_llama_graph_record_dense_dispatch(s) for l, s in zip(libs, states)]
            assert r[0] == r[1]
        counters = [LlamaGraphCounters(), LlamaGraphCounters()]
        for l, s, c in zip(libs, states, counters):
            assert l.cf_llama_graph_get_counters(s, C.byref(c)) == 0
        assert bytes(counters[0]) == bytes(counters[1])
        for l, s in zip(libs, states):
            l.cf_llama_graph_destroy(s)


def _random_page(rng, fake):
    """A page view that is valid about half the time: every field goes wrong with a few per cent probability."""
    from compat_types import PageView
    p = PageView()
    odd = lambda good, bad: int(rng.choice(good)) if rng.random() < 0.96 else int(rng.choice(bad))
    tokens, dim = odd([1, 4, 16, 64], [0, 4096]), odd([8, 64, 128], [0, 129, 256])
    p.struct_size = odd([C.sizeof(PageView)], [0, 4, 300])
    p.abi_version, p.flags = odd([0], [1, 9]), odd([1, 3], [0, 2])   # bit 0: sealed
    p.layer, p.kv_head = int(rng.integers(0, 4)), int(rng.integers(0, 4))
    p.token_begin = odd([0, 4, 100], [0xFFFFFFFE, 0xFFFFFFFF])
    p.token_count, p.head_dim = tokens, dim
    p.block_size, p.zero_point = odd([1, 32, 64], [0]), int(rng.choice([8, 128]))
    values = tokens * dim
    blocks = (values + max(p.block_size, 1) - 1) // max(p.block_size, 1)
    ptr = lambda: fake if rng.random() < 0.98 else None
    big = lambda n: n if rng.random() < 0.97 else int(rng.choice([0, 1, 0x7FFFFFFFFFFFFFFF]))
    p.k_words, p.k_word_count = ptr(), big(max(values // 8, 1))
    p.v_words, p.v_word_count = ptr(), big(max(values // 8, 1))
    p.k_block_offsets, p.k_block_count = ptr(), big(blocks if rng.random() < 0.97 else max(blocks - 1, 0))
    p.v_block_offsets, p.v_block_count = ptr(), big(blocks)
    p.k_lut, p.k_lut_count, p.v_lut, p.v_lut_count = ptr(), big(16), ptr(), big(16)
    p.k_scales, p.k_scale_count = ptr(), big(dim if rng.random() < 0.97 else dim + 1)
    p.v_scales, p.v_scale_count = ptr(), big(tokens if rng.random() < 0.97 else tokens + 1)
    return p


def test_host_runtime_answers_like_the_references_own(native, oracle):
    """cf_kv_validate_page / cf_kv_page_resident_bytes / cf_kv_validate_layout / cf_kv_cache_memory_stats on random
    page views and layouts, and the online-softmax state (init, accumulate, merge, finalize) on random scores with -inf
    and equal maxima among them: the same status and the same bytes as the reference's src/runtime/kv_runtime.cpp
    (oracle/_ref)."""
    from compat_types import CacheLayout, MemoryStats, PageView, SoftmaxState
    ref = oracle.ref_cpu()
    if ref is None:
        pytest.skip("needs the reference's sources compiled (oracle/_ref)")
    mine = native.lib()
    rng = np.random.default_rng(79)
    fake = 0x7f0000002000
    for _ in range(3000):
        p = _random_page(rng, fake)
        assert mine.cf_kv_validate_page(C.byref(p)) == ref.cf_kv_validate_page(C.byref(p)), [getattr(p, n) for n, _ in PageView._fields_]
        a, b = C.c_uint64(7), C.c_uint64(7)
        ra, rb = mine.cf_kv_page_resident_bytes(C.byref(p), C.byref(a)), ref.cf_kv_page_resident_bytes(C.byref(p), C.byref(b))
        assert (ra, a.value if ra == 0 else 0) == (rb, b.value if rb == 0 else 0), [getattr(p, n) for n, _ in PageView._fields_]
    for _ in range(1500):
        count = int(rng.integers(0, 5))
        pages = (PageView * max(count, 1))()
        begin = 0
        for i in range(count):   # mostly a well-formed run of pages, sometimes not
            q = _random_page(rng, fake) if rng.random() < 0.15 else _random_page(np.random.default_rng(1), fake)
            if rng.random() < 0.85:
                q.struct_size, q.abi_version, q.flags, q.token_count, q.head_dim, q.block_size = C.sizeof(PageView), 0, 1, 4, 8, 32
                q.token_begin = begin if rng.random() < 0.9 else begin + 1
                q.layer, q.kv_head = 0, 0
                for name, n in (("k_word", 4), ("v_word", 4), ("k_block", 1), ("v_block", 1), ("k_lut", 16), ("v_lut", 16), ("k_scale", 8), ("v_scale", 4)):
                    setattr(q, name + "s" if not name.endswith("lut") else name, fake)
                    setattr(q, name + "_count", n)
                q.k_block_offsets = q.v_block_offsets = fake
                begin += 4
            pages[i] = q
        lay = CacheLayout()
        lay.struct_size = C.sizeof(CacheLayout) if rng.random() < 0.9 else 8
        lay.abi_version = int(rng.choice([0, 0, 0, 3]))
        lay.layer_count, lay.kv_head_count, lay.head_dim = int(rng.choice([0, 1, 2])), int(rng.choice([0, 1, 2])), int(rng.choice([0, 8, 8, 16]))
        lay.page_capacity_tokens = int(rng.choice([0, 4, 4, 8]))
        lay.active_token_begin = begin if rng.random() < 0.8 else int(rng.integers(0, 40))
        lay.active_token_count, lay.active_element_bytes = int(rng.choice([0, 2, 4, 5])), int(rng.choice([0, 2, 4, 4, 3]))
        lay.pages, lay.page_count = (pages if rng.random() < 0.95 else None), count
        lay.active_k_bytes = lay.active_v_bytes = int(lay.active_token_count) * 8 * int(lay.active_element_bytes) if rng.random() < 0.85 else 7
        assert mine.cf_kv_validate_layout(C.byref(lay)) == ref.cf_kv_validate_layout(C.byref(lay))
        sa, sb = MemoryStats(), MemoryStats()
        ra, rb = mine.cf_kv_cache_memory_stats(C.byref(lay), C.byref(sa)), ref.cf_kv_cache_memory_stats(C.byref(lay), C.byref(sb))
        assert ra == rb and (ra != 0 or bytes(sa) == bytes(sb))
    for _ in range(300):
        dim = int(rng.choice([1, 3, 64, 128]))
        outs = []
        seeds = int(rng.integers(0, 1 << 30))
        for lib in (mine, ref):
            r = np.random.default_rng(seeds)
            states, buffers, log = [], [], []
            for s in range(2):
                buf = (C.c_double * dim)()
                st = SoftmaxState()
                log.append(lib.cf_online_softmax_init(C.byref(st), buf, dim if r.random() < 0.95 else 0))
                states.append(st)
                buffers.append(buf)
                for _ in range(int(r.integers(0, 12))):
                    score = float(r.choice([r.normal(0, 5), r.normal(0, 5), -np.inf, 3.0, 3.0, np.nan, np.inf]))
                    value = r.standard_normal(dim).astype(np.float32)
                    log.append(lib.cf_online_softmax_accumulate(C.byref(st), C.c_double(score), value.ctypes.data_as(C.c_void_p)))
            log.append(lib.cf_online_softmax_merge(C.byref(states[0]), C.byref(states[1])))
            out = np.full(dim, 9.0, np.float32)
            log.append(lib.cf_online_softmax_finalize(C.byref(states[0]), out.ctypes.data_as(C.c_void_p)))
            outs.append((log, out.tobytes(), states[0].max_score, states[0].exp_sum, states[0].initialized))
        assert outs[0][0] == outs[1][0]
        assert outs[0][1] == outs[1][1]
        same = lambda x, y: x == y or (x != x and y != y)
        assert same(outs[0][2], outs[1][2]) and same(outs[0][3], outs[1][3]) and outs[0][4] == outs[1][4]


def test_dense_runtime_bridge_behaves_like_the_references_own(native, oracle, tmp_path):
    """cf_llama_runtime_* on the dense backend (no adapter, no GPU): random record / append / error calls give the same
    status and the same last_error text, the snapshots are equal byte for byte, and the evidence files written by
    cf_llama_runtime_write_json are the same JSON documents."""
    import json
    from compat_types import LlamaRuntimeSnapshot, LlamaTensorView
    ref = oracle.ref_adapter()
    if ref is None:
        pytest.skip("needs the reference's sources compiled (oracle/_ref)")
    libs = [native.lib(), ref]
    for l in libs:
        l.cf_llama_runtime_create.restype = C.c_void_p
        l.cf_llama_runtime_last_error.restype = C.c_char_p
    rng = np.random.default_rng(80)
    rows = np.zeros((1, 2, 64), np.float32)
    view = LlamaTensorView(rows.ctypes.data, 2 * 64 * 4, 64 * 4, 4, 1, 2, 64, 0)
    for run in range(40):
        o = LlamaRuntimeOptions()
        o.struct_size = C.sizeof(o)
        o.kv.struct_size, o.kv.backend = C.sizeof(o.kv), 0          # dense
        o.kv.layer_count, o.kv.kv_head_count, o.kv.query_head_count = 2, 2, 8
        o.kv.head_dim, o.kv.page_size, o.kv.gqa_group_size, o.kv.kv_bits = 64, 32, 4, 8
        o.causal_window, o.require_cuda, o.allow_dense_fallback, o.emit_stats = int(rng.choice([0, 512])), 0, 1, int(rng.integers(0, 2))
        hs = [C.c_void_p(l.cf_llama_runtime_create(C.byref(o))) for l in libs]
        assert bool(hs[0].value) == bool(hs[1].value)
        if not hs[0].value:
            continue
        for _ in range(int(rng.integers(1, 15))):
            op = int(rng.integers(0, 4))
            if op == 0:
                r = [l.cf_llama_runtime_record_dense_fallback(h) for l, h in zip(libs, hs)]
            elif op == 1:
                a, b = int(rng.integers(0, 1 << 20)), int(rng.integers(0, 1 << 10))
                r = [l.cf_llama_runtime_record_compressed_launch(h, C.c_uint64(a), C.c_uint64(b)) for l, h in zip(libs, hs)]
            elif op == 2:
                r = [l.cf_llama_runtime_append(h, 0, 0, C.byref(view), C.byref(view), None) for l, h in zip(libs, hs)]
            else:
                r = [l.cf_llama_runtime_record_cuda_error(h) for l, h in zip(libs, hs)]
            assert r[0] == r[1]
            assert libs[0].cf_llama_runtime_last_error(hs[0]) == libs[1].cf_llama_runtime_last_error(hs[1])
        snaps = [LlamaRuntimeSnapshot(), LlamaRuntimeSnapshot()]
        for l, h, s in zip(libs, hs, snaps):
            assert l.cf_llama_runtime_snapshot_get(h, C.byref(s)) == 0
        assert bytes(snaps[0]) == bytes(snaps[1])
        docs = []
        for i, (l, h) in enumerate(zip(libs, hs)):
            path = str(tmp_path / f"evidence_{run}_{i}.json").encode()
            assert l.cf_llama_runtime_write_json(h, path) == 0
            docs.append(json.load(open(path)))
        assert docs[0] == docs[1]
        for l, h in zip(libs, hs):
            l.cf_llama_runtime_destroy(h)


class _ReferenceLibraries:
    """Looks a symbol up in the reference's own libraries (oracle/_ref), whichever holds it."""

    def __init__(self, oracle):
        self.libs = [oracle.ref_cpu(), oracle.ref_device(), oracle.ref_adapter(), oracle.ref_mscache()]

    def __getattr__(self, name):
        for lib in self.libs:
            try:
                return getattr(lib, name)
            except AttributeError:
                continue
        raise AttributeError(name)


@pytest.mark.parametrize("name", [
    "test_page_validation_and_exact_byte_accounting", "test_layout_validation_and_memory_stats",
    "test_online_softmax_matches_reference_golden", "test_adapter_options_and_null_handles",
    "test_device_engine_contracts_without_a_gpu", "test_sequence_resolver_contract_without_a_gpu",
    "test_multisequence_cache_and_server_contracts_without_a_gpu"])
def test_hand_written_host_contract_cases_hold_for_the_reference_itself(native, oracle, name):
    """The host-contract cases of tests/test_compat_host.py were written from reading the reference; here the very same
    test functions run against the reference's own code instead of this library, so that what they expect is what the
    reference does. (Two of that file's tests are left out: the multi-GPU runtime's execute calls cudaSetDevice in the
    reference, which needs a GPU, and the decode runtime's test looks for this library's own wording of an error that
    the reference does not detect before launching.)"""
    import types
    import test_compat_host
    if any(lib is None for lib in (oracle.ref_cpu(), oracle.ref_device(), oracle.ref_adapter(), oracle.ref_mscache())):
        pytest.skip("needs the reference's sources compiled (oracle/_ref)")
    reference = _ReferenceLibraries(oracle)
    stand_in = types.SimpleNamespace(**{k: getattr(native, k) for k in dir(native) if not k.startswith("__")})
    stand_in.lib = lambda: reference
    getattr(test_compat_host, name)(stand_in)


@pytest.mark.parametrize("name", [
    "test_graph_contract_validation", "test_dense_graph_state_counts_and_never_owns_a_runtime",
    "test_runtime_bridge_options_and_dense_runtime", "test_forwarding_bridges_refuse_bad_options_without_a_gpu"])
def test_hand_written_bridge_cases_hold_for_the_reference_itself(native, oracle, name, tmp_path):
    """The same for the CPU cases of tests/test_compat_bridges.py: the llama.cpp-side bridges of the reference
    (integrations/llama.cpp/*.cpp, compiled into oracle/_ref) must pass the very tests written for this library's."""
    import inspect
    import types
    import test_compat_bridges
    if any(lib is None for lib in (oracle.ref_device(), oracle.ref_adapter(), oracle.ref_msbridge())):
        pytest.skip("needs the reference's sources compiled (oracle/_ref)")
    reference = _ReferenceLibraries(oracle)
    stand_in = types.SimpleNamespace(**{k: getattr(native, k) for k in dir(native) if not k.startswith("__")})
    stand_in.lib = lambda: reference
    stand_in.ms_bridge_lib = oracle.ref_msbridge
    function = getattr(test_compat_bridges, name)
    if "tmp_path" in inspect.signature(function).parameters:
        function(stand_in, tmp_path)
    else:
        function(stand_in)
