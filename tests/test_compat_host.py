"""Host-side functions of the reference ABI re-implemented by this library (compat_kv.h, compat_adapter.h): the cases
of the reference's tests/kv_runtime_test.cpp and tests/llama_kv_adapter_seam.cpp, plus the golden vectors made from the
reference's own cf_online_softmax_* (tests/golden/online_softmax.npz). No GPU is touched."""
import ctypes as C
import os

import numpy as np

from compat_types import CacheLayout, LlamaKvOptions, MemoryStats, PageView, SoftmaxState

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
FAKE = [0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 0x6000, 0x7000, 0x8000]   # never dereferenced (kv_runtime_test.cpp:12-17)


def _page(token_begin=0, tokens=4, dim=8, layer=0, head=0):
    p = PageView()
    p.struct_size, p.abi_version, p.flags = C.sizeof(PageView), 0, 0x3
    p.layer, p.kv_head, p.token_begin, p.token_count, p.head_dim, p.block_size, p.zero_point = layer, head, token_begin, tokens, dim, 64, 8
    p.k_words, p.k_word_count, p.v_words, p.v_word_count = FAKE[0], 5, FAKE[1], 6
    p.k_block_offsets, p.k_block_count, p.v_block_offsets, p.v_block_count = FAKE[2], 1, FAKE[3], 1
    p.k_lut, p.k_lut_count, p.v_lut, p.v_lut_count = FAKE[4], 16, FAKE[5], 16
    p.k_scales, p.k_scale_count, p.v_scales, p.v_scale_count = FAKE[6], dim, FAKE[7], tokens
    return p


def test_page_validation_and_exact_byte_accounting(native):
    lib = native.lib()
    p = _page()
    assert lib.cf_kv_validate_page(C.byref(p)) == 0
    n = C.c_uint64(0)
    assert lib.cf_kv_page_resident_bytes(C.byref(p), C.byref(n)) == 0
    assert n.value == (5 + 6) * 4 + (1 + 1 + 16 + 16) * 4 + (8 + 4) * 4       # kv_runtime_test.cpp:49-68
    assert lib.cf_kv_validate_page(None) == 1
    for field, value in [("struct_size", 4), ("abi_version", 9), ("flags", 0x2), ("token_count", 0), ("head_dim", 129),
                         ("block_size", 0), ("k_words", None), ("k_word_count", 0), ("k_scale_count", 7),
                         ("v_scale_count", 5), ("k_block_count", 0)]:
        bad = _page()
        setattr(bad, field, value)
        assert lib.cf_kv_validate_page(C.byref(bad)) == 1, field
    bad = _page(token_begin=0xFFFFFFFE, tokens=4)
    assert lib.cf_kv_validate_page(C.byref(bad)) == 1
    big = _page(tokens=4096, dim=128)
    big.block_size = 1
    big.k_block_count = big.v_block_count = 10          # fewer blocks than tokens*dim needs
    assert lib.cf_kv_validate_page(C.byref(big)) == 1
    assert lib.cf_kv_page_resident_bytes(C.byref(p), None) == 1
    over = _page()
    over.k_word_count = 0x7FFFFFFFFFFFFFFF                  # byte count overflows 64 bits: unsupported, not invalid
    assert lib.cf_kv_page_resident_bytes(C.byref(over), C.byref(n)) == 2


def test_layout_validation_and_memory_stats(native):
    lib = native.lib()
    pages = (PageView * 2)(_page(0, 4), _page(4, 4))
    lay = CacheLayout()
    lay.struct_size, lay.abi_version = C.sizeof(CacheLayout), 0
    lay.layer_count, lay.kv_head_count, lay.head_dim, lay.page_capacity_tokens = 1, 1, 8, 4
    lay.active_token_begin, lay.active_token_count, lay.active_element_bytes = 8, 2, 4
    lay.pages, lay.page_count = pages, 2
    lay.active_k_bytes = lay.active_v_bytes = 2 * 8 * 4
    assert lib.cf_kv_validate_layout(C.byref(lay)) == 0
    st = MemoryStats()
    assert lib.cf_kv_cache_memory_stats(C.byref(lay), C.byref(st)) == 0
    one = (5 + 6) * 4 + 34 * 4 + 12 * 4
    assert (st.page_count, st.sealed_tokens, st.active_tokens) == (2, 8, 2)
    assert st.sealed_payload_bytes == 2 * one and st.sealed_descriptor_bytes == 2 * 168
    assert st.active_payload_bytes == 128 and st.total_resident_bytes == 2 * one + 336 + 128
    pages[1].token_begin = 3                                  # overlap (kv_runtime_test.cpp:70-104)
    assert lib.cf_kv_validate_layout(C.byref(lay)) == 1
    pages[1].token_begin = 4
    lay.active_k_bytes = 1                                    # tail under-accounted
    assert lib.cf_kv_validate_layout(C.byref(lay)) == 1
    lay.active_k_bytes = 64
    lay.active_token_begin = 7                                # a sealed page reaches into the tail
    assert lib.cf_kv_validate_layout(C.byref(lay)) == 1
    lay.active_token_begin = 8
    lay.active_token_count = 5                                # tail longer than a page
    assert lib.cf_kv_validate_layout(C.byref(lay)) == 1
    assert lib.cf_kv_cache_memory_stats(C.byref(lay), None) == 1


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def test_online_softmax_matches_reference_golden(native):
    """Same inputs, same split into partial states, same merges as the golden file made with the reference's
    cf_online_softmax_* — every intermediate state must agree to the last bit of the double."""
    lib = native.lib()
    z = np.load(os.path.join(GOLD, "online_softmax.npz"))
    for name in sorted({k.split(".")[0] for k in z.files}):
        scores, values, cuts = z[f"{name}.scores"], z[f"{name}.values"], z[f"{name}.cuts"]
        dim = values.shape[1]
        merged, mbuf = SoftmaxState(), (C.c_double * dim)()
        assert lib.cf_online_softmax_init(C.byref(merged), mbuf, dim) == 0
        begin = 0
        for i, end in enumerate(cuts):
            st, buf = SoftmaxState(), (C.c_double * dim)()
            assert lib.cf_online_softmax_init(C.byref(st), buf, dim) == 0
            for j in range(begin, int(end)):
                assert lib.cf_online_softmax_accumulate(C.byref(st), C.c_double(scores[j]), _p(np.ascontiguousarray(values[j]))) == 0
            assert st.max_score == z[f"{name}.partial_max"][i] and st.exp_sum == z[f"{name}.partial_sum"][i]
            assert np.array_equal(np.array(buf[:]), z[f"{name}.partial_weighted"][i])
            assert lib.cf_online_softmax_merge(C.byref(merged), C.byref(st)) == 0
            begin = int(end)
        out = np.zeros(dim, np.float32)
        assert lib.cf_online_softmax_finalize(C.byref(merged), _p(out)) == 0
        assert merged.max_score == float(z[f"{name}.merged_max"]) and merged.exp_sum == float(z[f"{name}.merged_sum"])
        assert np.array_equal(out, z[f"{name}.output"])
    empty, ebuf = SoftmaxState(), (C.c_double * 4)()
    assert lib.cf_online_softmax_init(C.byref(empty), ebuf, 4) == 0
    assert lib.cf_online_softmax_finalize(C.byref(empty), _p(np.zeros(4, np.float32))) == 1     # kv_runtime_test.cpp:152-157
    assert lib.cf_online_softmax_init(C.byref(empty), ebuf, 129) == 1
    assert lib.cf_online_softmax_accumulate(C.byref(empty), C.c_double(float("nan")), _p(np.zeros(4, np.float32))) == 1


def test_adapter_options_and_null_handles(native):
    """integrations/llama.cpp/chromofold_kv_adapter.cpp:53-63 and tests/llama_kv_adapter_seam.cpp."""
    lib = native.lib()
    lib.cf_llama_kv_last_error.restype = C.c_char_p
    lib.cf_llama_kv_create.restype = C.c_void_p
    o = LlamaKvOptions()
    o.struct_size, o.backend = C.sizeof(LlamaKvOptions), 1
    o.layer_count, o.kv_head_count, o.query_head_count, o.head_dim, o.page_size, o.gqa_group_size = 2, 2, 8, 64, 32, 4
    assert lib.cf_llama_kv_options_validate(C.byref(o)) == 0
    assert lib.cf_llama_kv_options_validate(None) == -1
    o.query_head_count = 7
    assert lib.cf_llama_kv_options_validate(C.byref(o)) == -1      # Hq != Hkv * group
    assert lib.cf_llama_kv_create(C.byref(o)) is None
    o.backend = 0
    assert lib.cf_llama_kv_options_validate(C.byref(o)) == 0       # dense backend: nothing to check
    assert lib.cf_llama_kv_create(C.byref(o)) is None              # but no adapter is made for it
    o.struct_size = 8
    assert lib.cf_llama_kv_options_validate(C.byref(o)) == -1
    assert lib.cf_llama_kv_append(None, 0, 0, 0, None, None, 0, None) == -1
    assert lib.cf_llama_kv_flush(None, None) == -1 and lib.cf_llama_kv_get_stats(None, None) == -1
    assert lib.cf_llama_kv_last_error(None) == b"invalid ChromoFold KV adapter"


def test_device_engine_contracts_without_a_gpu(native):
    """The reference's no-GPU contracts: tests/m9_device_seal_contract.cpp and tests/device_kv_dataplane_contract.cpp.
    Handles are created, queried and destroyed without any CUDA call."""
    from compat_types import DeviceKvConfig, DeviceKvCounters, DeviceSealConfig, DeviceSealCounters, TensorView
    lib = native.lib()
    lib.cf_device_seal_create.restype = C.c_void_p
    lib.cf_device_kv_create.restype = C.c_void_p
    lib.cf_device_seal_last_error.restype = C.c_char_p
    cfg = DeviceSealConfig(2, 4, 8, 64, 64, 2, 32, 1)
    e = C.c_void_p(lib.cf_device_seal_create(C.byref(cfg)))
    assert e.value
    state = C.c_uint32(99)
    assert lib.cf_device_seal_get_state(e, 0, C.byref(state)) == 0 and state.value == 0      # CF_SEAL_ACTIVE_FILLING
    for fault in range(0, 11):
        assert lib.cf_device_seal_set_fault(e, fault) == 0
    assert lib.cf_device_seal_set_fault(e, 11) != 0
    n = DeviceSealCounters()
    assert lib.cf_device_seal_get_counters(e, C.byref(n)) == 0
    assert (n.seal_attempts, n.seal_successes, n.descriptor_publications, n.compressed_attention_launches) == (0, 0, 0, 0)
    assert lib.cf_device_seal_full_page_async(e, 0, None) == -1                                # nothing staged
    assert b"full active page" in lib.cf_device_seal_last_error(e)
    assert lib.cf_device_seal_get_state(e, 5, C.byref(state)) == -1
    lib.cf_device_seal_destroy(e, None)
    bad = DeviceSealConfig(2, 4, 7, 64, 64, 2, 32, 1)
    assert lib.cf_device_seal_create(C.byref(bad)) is None
    bad = DeviceSealConfig(2, 4, 8, 64, 64, 2, 0, 1)
    assert lib.cf_device_seal_create(C.byref(bad)) is None
    assert lib.cf_device_seal_last_error(None) == b"null seal engine"

    fake = (C.c_float * 1)()
    v = TensorView(C.addressof(fake), 3, 2, 4, 8, 4 * 8 * 4, 8 * 4, 4, 0)
    assert lib.cf_device_tensor_validate(C.byref(v)) == 0
    for field, value in [("scalar_type", 999), ("element_stride_bytes", 1), ("head_stride_bytes", 1),
                         ("token_stride_bytes", 1), ("data", None), ("token_count", 0)]:
        w = TensorView(C.addressof(fake), 3, 2, 4, 8, 4 * 8 * 4, 8 * 4, 4, 0)
        setattr(w, field, value)
        assert lib.cf_device_tensor_validate(C.byref(w)) != 0, field
    kc = DeviceKvConfig(2, 4, 8, 8, 64, 2, 1)
    d = C.c_void_p(lib.cf_device_kv_create(C.byref(kc)))
    assert d.value
    kn = DeviceKvCounters()
    assert lib.cf_device_kv_get_counters(d, C.byref(kn)) == 0
    assert kn.device_append_calls == 0 and kn.dense_fallback_launches == 0
    lib.cf_device_kv_destroy(d, None)
    kc.query_head_count = 7
    assert lib.cf_device_kv_create(C.byref(kc)) is None


def test_sequence_resolver_contract_without_a_gpu(native):
    """tests/m10_cuda_sequence_resolver_contract.cpp: create, duplicate rejection, a shift that moves nothing, cancel,
    audit, counters — no CUDA call is made."""
    from compat_types import MsConfig, MsCounters
    lib = native.lib()
    lib.cf_ms_cuda_create.restype = C.c_void_p
    lib.cf_ms_cuda_last_error.restype = C.c_char_p
    r = C.c_void_p(lib.cf_ms_cuda_create(C.byref(MsConfig(2, 2, 4, 64, 64, 2, 0))))
    assert r.value
    assert lib.cf_ms_cuda_sequence_create(r, C.c_int64(101)) == 0
    assert lib.cf_ms_cuda_sequence_create(r, C.c_int64(202)) == 0
    assert lib.cf_ms_cuda_sequence_create(r, C.c_int64(101)) != 0
    assert b"already exists" in lib.cf_ms_cuda_last_error(r)
    assert lib.cf_ms_cuda_shift_sequence(r, C.c_int64(101), 0, 0, 0) == 0
    assert lib.cf_ms_cuda_cancel_sequence_async(r, C.c_int64(202), None) == 0
    assert lib.cf_ms_cuda_cancel_sequence_async(r, C.c_int64(303), None) == -1
    assert lib.cf_ms_cuda_audit(r) == 0
    n = MsCounters()
    assert lib.cf_ms_cuda_get_counters(r, C.byref(n)) == 0
    assert n.cancellation_requests == 1 and n.dense_fallback_launches == 0 and n.cross_sequence_contamination == 0
    assert lib.cf_ms_cuda_sequence_remove_async(r, C.c_int64(101), None) == 0
    assert lib.cf_ms_cuda_sequence_remove_async(r, C.c_int64(101), None) == -1
    assert lib.cf_ms_cuda_copy_sequence_async(r, C.c_int64(5), C.c_int64(5), None) == -1
    lib.cf_ms_cuda_destroy(r, None)
    assert lib.cf_ms_cuda_create(C.byref(MsConfig(2, 2, 5, 64, 64, 2, 0))) is None
    assert lib.cf_ms_cuda_last_error(None) == b"null multi-sequence CUDA resolver"


def test_production_runtime_contract_without_a_gpu(native):
    """The cases of the reference's tests/m12_production_attention_contract.cpp: create / counters / invalidate /
    destroy, plus the argument checks that come before any CUDA call."""
    from compat_types import AttentionBatchItem, AttentionCounters, AttentionRuntimeConfig
    lib = native.lib()
    lib.cf_attention_runtime_create.restype = C.c_void_p
    lib.cf_attention_last_error.restype = C.c_char_p
    assert C.sizeof(AttentionBatchItem) == 168
    cfg = AttentionRuntimeConfig()
    cfg.layer_count, cfg.query_head_count, cfg.kv_head_count, cfg.head_dim = 2, 8, 2, 64
    cfg.page_size, cfg.block_size, cfg.gqa_group_size, cfg.mode = 16, 64, 4, 1
    assert lib.cf_attention_runtime_create(None) is None
    bad = AttentionRuntimeConfig.from_buffer_copy(cfg)
    bad.gqa_group_size = 3
    assert lib.cf_attention_runtime_create(C.byref(bad)) is None   # query heads != kv heads * group
    bad = AttentionRuntimeConfig.from_buffer_copy(cfg)
    bad.head_dim = 0
    assert lib.cf_attention_runtime_create(C.byref(bad)) is None
    rt = C.c_void_p(lib.cf_attention_runtime_create(C.byref(cfg)))
    assert rt.value
    counters = AttentionCounters()
    assert lib.cf_attention_get_counters(rt, C.byref(counters)) == 0
    assert all(getattr(counters, n) == 0 for n, _ in AttentionCounters._fields_)
    assert lib.cf_attention_invalidate_graphs(rt) == 0
    assert lib.cf_attention_get_counters(rt, C.byref(counters)) == 0
    assert counters.graph_invalidations == 1
    assert lib.cf_attention_get_counters(rt, None) == -1 and lib.cf_attention_get_counters(None, C.byref(counters)) == -1
    item = AttentionBatchItem()
    assert lib.cf_attention_execute_async(rt, None, 1, None) == -1
    assert lib.cf_attention_execute_async(rt, C.byref(item), 0, None) == -1
    assert lib.cf_attention_execute_async(None, C.byref(item), 1, None) == -1
    item.layer = 5
    assert lib.cf_attention_execute_async(rt, C.byref(item), 1, None) == -1
    assert b"layer" in lib.cf_attention_last_error(rt)
    assert lib.cf_attention_compare_async(rt, C.byref(item), 1, C.c_float(0.0), C.c_float(1.0), None) == -1
    assert lib.cf_attention_last_error(None) == b"runtime is null"
    lib.cf_attention_runtime_destroy(rt, None)
    lib.cf_attention_runtime_destroy(None, None)


def test_multisequence_cache_and_server_contracts_without_a_gpu(native):
    """The host-only cases of the reference's tests/m10_multisequence_host_contract.cpp and
    tests/m11_pinned_server_contract.cpp: create / duplicate-reject / copy / speculation / remove / reclaim / audit /
    counters, and the server runtime's config rules and shutdown audit. No row is appended, so no CUDA call is made."""
    from compat_types import (LlamaServerConfig, LlamaServerStats, MultisequenceConfig, MultisequenceCounters, TensorView)
    lib = native.lib()
    lib.cf_multisequence_create.restype = C.c_void_p
    lib.cf_multisequence_last_error.restype = C.c_char_p
    lib.cf_sequence_speculation_begin.restype = C.c_uint64
    lib.cf_llama_server_runtime_create.restype = C.c_void_p
    lib.cf_llama_server_last_error.restype = C.c_char_p
    assert lib.cf_multisequence_create(None) is None
    assert lib.cf_multisequence_create(C.byref(MultisequenceConfig(2, 2, 8, 64, 16, 3, 0, 1))) is None   # 8 != 2 * 3
    c = C.c_void_p(lib.cf_multisequence_create(C.byref(MultisequenceConfig(2, 2, 8, 64, 16, 4, 0, 1))))
    assert c.value
    i64 = C.c_int64
    assert lib.cf_sequence_create(c, i64(1)) == 0
    assert lib.cf_sequence_create(c, i64(1)) == -1 and b"already exists" in lib.cf_multisequence_last_error(c)
    assert lib.cf_sequence_copy_async(c, i64(1), i64(1), 0, 10, None) == -1          # onto itself
    assert lib.cf_sequence_copy_async(c, i64(1), i64(2), 5, 1, None) == -1           # end < begin
    assert lib.cf_sequence_copy_async(c, i64(9), i64(2), 0, 10, None) == -1          # unknown source
    assert lib.cf_sequence_copy_async(c, i64(1), i64(2), 0, 1 << 30, None) == 0
    assert lib.cf_sequence_copy_async(c, i64(1), i64(3), 4, 1 << 30, None) == 0      # any range (here of an empty sequence)
    assert lib.cf_sequence_copy_async(c, i64(1), i64(3), 0, 0, None) == 0            # tests/m10_multisequence_host_contract.cpp:28
    spec = lib.cf_sequence_speculation_begin(c, i64(2))
    assert spec != 0 and lib.cf_sequence_speculation_begin(c, i64(2)) == 0           # one at a time
    assert lib.cf_sequence_speculation_commit(c, i64(2), C.c_uint64(spec + 5), 0, None) == -1
    assert lib.cf_sequence_speculation_commit(c, i64(2), C.c_uint64(spec), 3, None) == -1    # nothing provisional
    assert lib.cf_sequence_speculation_rollback(c, i64(2), C.c_uint64(spec), None) == 0
    spec = lib.cf_sequence_speculation_begin(c, i64(2))
    assert lib.cf_sequence_speculation_commit(c, i64(2), C.c_uint64(spec), 0, None) == 0
    view = TensorView()
    assert lib.cf_sequence_append_async(c, i64(1), 0, 0, None, C.byref(view), None) == -1
    assert lib.cf_sequence_append_async(c, i64(1), 7, 0, C.byref(view), C.byref(view), None) == -1   # layer out of range
    assert lib.cf_multisequence_attention_async(c, None, 1, None) == -1
    assert lib.cf_sequence_shift_async(c, i64(1), 0, 0, 0, None) == 0                # a shift that moves nothing
    assert lib.cf_sequence_remove_async(c, i64(2), i64(5), i64(1), None) == -1
    assert lib.cf_sequence_remove_async(c, i64(2), i64(-1), i64(-1), None) == 0
    assert lib.cf_sequence_remove_async(c, i64(2), i64(-1), i64(-1), None) == -1
    assert lib.cf_multisequence_reclaim_async(c, None) == 0 and lib.cf_multisequence_audit(c) == 0
    k = MultisequenceCounters()
    assert lib.cf_multisequence_get_counters(c, C.byref(k)) == 0
    assert (k.sequences_created, k.sequences_copied, k.sequences_removed, k.active_sequences, k.active_sequences_peak) == (1, 3, 1, 2, 3)
    assert (k.speculative_transactions_started, k.speculative_transactions_committed, k.speculative_transactions_rolled_back) == (2, 1, 1)
    assert k.unsupported_operations == 0 and k.invariant_audits > 0 and k.invariant_failures == 0 and k.dense_fallback_launches == 0
    assert lib.cf_multisequence_last_error(None) == b"null multisequence cache"
    lib.cf_multisequence_destroy(c, None)

    cfg = LlamaServerConfig(2, 8, 2, 64, 16, 64, 4096, 4, 0, 1, None, b"76f46ad2", None)
    assert lib.cf_llama_server_runtime_create(C.byref(cfg)) is None                   # model_sha256 is required
    cfg.model_sha256 = b"0" * 64
    s = C.c_void_p(lib.cf_llama_server_runtime_create(C.byref(cfg)))
    assert s.value
    assert lib.cf_llama_server_slot_create(s, i64(11)) == 0 and lib.cf_llama_server_slot_create(s, i64(11)) == -1
    assert lib.cf_llama_server_slot_create(s, i64(12)) == 0
    assert lib.cf_llama_server_sequence_copy_async(s, i64(11), i64(13), 0, 1 << 30, None) == 0
    assert lib.cf_llama_server_cancel_async(s, i64(12), None) == 0
    assert lib.cf_llama_server_slot_reset_async(s, i64(12), None) == 0
    assert lib.cf_llama_server_slot_reset_async(s, i64(12), None) == -1
    assert lib.cf_llama_server_execute_batch_async(s, None, None) == -1
    assert lib.cf_llama_server_shutdown_async(s, None) == 0
    assert lib.cf_llama_server_slot_create(s, i64(14)) == -1 and b"shutting down" in lib.cf_llama_server_last_error(s)
    st = LlamaServerStats()
    assert lib.cf_llama_server_get_stats(s, C.byref(st)) == 0
    assert (st.http_requests, st.slot_reuses, st.cancelled_requests, st.shutdown_audits, st.shutdown_failures) == (2, 1, 1, 1, 0)
    lib.cf_llama_server_runtime_destroy(s, None)


def test_multigpu_runtime_contract_without_a_gpu(native):
    """The cases of the reference's tests/m15_multigpu_cuda_contract.cpp (two-device config, injected failure) plus
    the admission rules of src/cuda/multigpu_cuda_runtime.cu:34-55,103-134. Local pages only, so no CUDA call is made."""
    from compat_types import MultigpuCounters, MultigpuDeviceConfig, MultigpuPageView, MultigpuRuntimeConfig, MultigpuShard
    lib = native.lib()
    lib.cf_multigpu_cuda_create.restype = C.c_void_p
    lib.cf_multigpu_cuda_last_error.restype = C.c_char_p
    devs = (MultigpuDeviceConfig * 2)(MultigpuDeviceConfig(0, 1 << 30, 0), MultigpuDeviceConfig(1, 1 << 30, 0))
    mk = lambda **kw: MultigpuRuntimeConfig(**{**dict(devices=C.cast(devs, C.c_void_p), device_count=2, layer_count=4,
                                                      tensor_parallel_size=2, allow_host_staging=0, require_peer_access=1,
                                                      collective=0), **kw})
    assert lib.cf_multigpu_cuda_create(None) is None
    assert lib.cf_multigpu_cuda_create(C.byref(mk(device_count=1))) is None
    assert lib.cf_multigpu_cuda_create(C.byref(mk(tensor_parallel_size=3))) is None
    same = (MultigpuDeviceConfig * 2)(MultigpuDeviceConfig(0, 1 << 30, 0), MultigpuDeviceConfig(0, 1 << 30, 0))
    assert lib.cf_multigpu_cuda_create(C.byref(mk(devices=C.cast(same, C.c_void_p)))) is None   # ordinals must be unique
    r = C.c_void_p(lib.cf_multigpu_cuda_create(C.byref(mk(collective=1))))
    assert r.value
    page = MultigpuPageView(0x1000, 0x2000, 0x3000, 0x4000, 512, 512, 4, 4, 16, 2, 64, 32, 0, 1)
    shard = MultigpuShard(7, 0, 0, 4, 0, 0x5000, 0x6000, 1, 3, 64, 1, C.cast(C.pointer(page), C.c_void_p))
    assert lib.cf_multigpu_cuda_execute_async(r, C.byref(shard), 1, None) == 0
    bad = MultigpuShard.from_buffer_copy(shard)
    bad.layer = 9
    assert lib.cf_multigpu_cuda_execute_async(r, C.byref(bad), 1, None) == -1
    odd = MultigpuPageView.from_buffer_copy(page)
    odd.key_codec = 3
    bad = MultigpuShard.from_buffer_copy(shard)
    bad.pages = C.cast(C.pointer(odd), C.c_void_p)
    assert lib.cf_multigpu_cuda_execute_async(r, C.byref(bad), 1, None) == -1
    assert b"page descriptor" in lib.cf_multigpu_cuda_last_error(r)
    assert lib.cf_multigpu_cuda_migrate_sequence_async(r, C.c_uint64(7), 0, 1, C.byref(page), 1, None) == 0
    assert lib.cf_multigpu_cuda_migrate_sequence_async(r, C.c_uint64(7), 1, 0, C.byref(page), 1, None) == -1   # not the owner
    assert lib.cf_multigpu_cuda_inject_device_failure(r, 5) == -1 and lib.cf_multigpu_cuda_inject_device_failure(r, 0) == 0
    assert lib.cf_multigpu_cuda_execute_async(r, C.byref(shard), 1, None) == -1
    assert b"unknown or failed" in lib.cf_multigpu_cuda_last_error(r)
    assert lib.cf_multigpu_cuda_shutdown(r) == 0
    other = MultigpuShard.from_buffer_copy(shard)
    other.execution_device = 1
    assert lib.cf_multigpu_cuda_execute_async(r, C.byref(other), 1, None) == -1
    k = MultigpuCounters()
    assert lib.cf_multigpu_cuda_get_counters(r, C.byref(k)) == 0
    assert (k.batches_submitted, k.shards_dispatched, k.collective_calls, k.migrations_completed) == (1, 1, 1, 1)
    assert (k.device_failures_detected, k.fail_closed_rejections, k.remote_pages_loaded, k.dense_fallback_launches) == (1, 5, 0, 0)
    lib.cf_multigpu_cuda_destroy(r)
