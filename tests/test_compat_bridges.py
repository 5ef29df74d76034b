"""The llama.cpp-side bridges (include/chromofold_b200/compat_bridges.h, compat_llama_ms_bridge.h): the cases of the
reference's tests/llama_graph_contract_test.cpp and the contracts stated in integrations/llama.cpp/*_bridge.cpp,
graph/chromofold_graph_contract.cpp. The tests of this part touch no GPU; the GPU ones are marked."""
import ctypes as C
import json
import os

import numpy as np
import pytest

from compat_types import (DeviceKvCounters, DeviceSealCounters, LlamaDeviceGraphOptions, LlamaDeviceSealOptions,
                          LlamaGraphCounters, LlamaGraphOptions, LlamaKvOptions, LlamaModelTopology, LlamaRuntimeOptions,
                          LlamaRuntimeSnapshot, LlamaServerMultisequenceConfig, LlamaTensorView, MsConfig, TensorView)

DENSE, CHROMOFOLD = 0, 1


def _graph_options(backend=CHROMOFOLD, page=128, path=None):
    o = LlamaGraphOptions()
    o.struct_size, o.backend, o.page_size, o.evidence_path = C.sizeof(o), backend, page, path
    return o


def _topology(layers=32, hq=32, hkv=8, dim=128):
    t = LlamaModelTopology()
    t.struct_size, t.layer_count, t.query_head_count, t.kv_head_count, t.head_dim = C.sizeof(t), layers, hq, hkv, dim
    t.context_size, t.uniform_kv_geometry, t.causal = 8192, 1, 1
    return t


def _runtime_options(backend=CHROMOFOLD, layers=2, hq=8, hkv=2, dim=64, page=64):
    o = LlamaRuntimeOptions()
    o.struct_size = C.sizeof(o)
    o.kv.struct_size, o.kv.backend = C.sizeof(LlamaKvOptions), backend
    o.kv.layer_count, o.kv.kv_head_count, o.kv.query_head_count, o.kv.head_dim = layers, hkv, hq, dim
    o.kv.page_size, o.kv.gqa_group_size, o.kv.kv_bits = page, hq // hkv, 8
    o.require_cuda, o.allow_dense_fallback = 1, 0
    return o


def test_graph_contract_validation(native):
    """tests/llama_graph_contract_test.cpp, plus the other refusals of chromofold_graph_contract.cpp:34-50."""
    lib = native.lib()
    o = _graph_options()
    assert lib.cf_llama_graph_options_validate(C.byref(o)) == 0
    o.page_size = 96
    assert lib.cf_llama_graph_options_validate(C.byref(o)) != 0
    for page in (64, 256):
        o.page_size = page
        assert lib.cf_llama_graph_options_validate(C.byref(o)) == 0
    o.backend = 7
    assert lib.cf_llama_graph_options_validate(C.byref(o)) != 0
    o.backend, o.page_size = DENSE, 5                       # dense backend: the page size is not looked at
    assert lib.cf_llama_graph_options_validate(C.byref(o)) == 0
    o.struct_size = 4
    assert lib.cf_llama_graph_options_validate(C.byref(o)) != 0
    assert lib.cf_llama_graph_options_validate(None) != 0

    t = _topology()
    assert lib.cf_llama_model_topology_validate(C.byref(t)) == 0
    t.recurrent = 1
    assert lib.cf_llama_model_topology_validate(C.byref(t)) != 0
    t.recurrent, t.causal = 0, 0
    assert lib.cf_llama_model_topology_validate(C.byref(t)) != 0
    t.causal, t.uniform_kv_geometry = 1, 0
    assert lib.cf_llama_model_topology_validate(C.byref(t)) != 0
    t.uniform_kv_geometry, t.head_dim = 1, 256
    assert lib.cf_llama_model_topology_validate(C.byref(t)) != 0
    t.head_dim, t.query_head_count = 128, 30                # 30 query heads over 8 kv heads
    assert lib.cf_llama_model_topology_validate(C.byref(t)) != 0
    t.query_head_count, t.layer_count = 32, 0
    assert lib.cf_llama_model_topology_validate(C.byref(t)) != 0
    assert lib.cf_llama_model_topology_validate(None) != 0


def test_dense_graph_state_counts_and_never_owns_a_runtime(native):
    """A dense-backend graph state needs no GPU: dense dispatches are counted and allowed, everything that needs the
    ChromoFold runtime is refused and counted in unsupported_graphs (chromofold_graph_contract.cpp:86-118)."""
    lib = native.lib()
    lib.cf_llama_graph_create.restype = C.c_void_p
    lib.cf_llama_graph_last_error.restype = C.c_char_p
    o, t = _graph_options(backend=DENSE), _topology()
    g = lib.cf_llama_graph_create(C.byref(o), C.byref(t))
    assert g
    g = C.c_void_p(g)
    assert lib.cf_llama_graph_record_dense_dispatch(g) == 0
    assert lib.cf_llama_graph_record_dense_dispatch(g) == 0
    assert lib.cf_llama_graph_record_attention(g, C.c_uint64(10), C.c_uint64(2)) == -1
    assert lib.cf_llama_graph_last_error(g) == b"compressed attention recorded without runtime"
    assert lib.cf_llama_graph_append_device(g, 0, 0, None, None, None) == -1
    assert lib.cf_llama_graph_last_error(g) == b"ChromoFold graph backend is not active"
    assert lib.cf_llama_graph_write_evidence(g) == -1
    c = LlamaGraphCounters()
    assert lib.cf_llama_graph_get_counters(g, C.byref(c)) == 0
    assert (c.graph_dense_dispatches, c.unsupported_graphs, c.graph_attention_dispatches, c.graph_append_calls) == (2, 2, 0, 0)
    assert lib.cf_llama_graph_get_counters(g, None) == -1
    lib.cf_llama_graph_destroy(g)
    bad = _topology()
    bad.recurrent = 1
    assert lib.cf_llama_graph_create(C.byref(o), C.byref(bad)) is None
    assert lib.cf_llama_graph_create(None, C.byref(t)) is None
    assert lib.cf_llama_graph_last_error(None) == b"null graph state"
    assert lib.cf_llama_graph_record_dense_dispatch(None) == -1


def test_runtime_bridge_options_and_dense_runtime(native, tmp_path):
    """chromofold_runtime_bridge.cpp:43-50: a ChromoFold runtime needs CUDA and forbids the dense fallback. A dense
    runtime holds no adapter: appends and compressed launches are refused and counted, its evidence is never complete."""
    lib = native.lib()
    lib.cf_llama_runtime_create.restype = C.c_void_p
    lib.cf_llama_runtime_last_error.restype = C.c_char_p
    o = _runtime_options()
    assert lib.cf_llama_runtime_options_validate(C.byref(o)) == 0
    o.allow_dense_fallback = 1
    assert lib.cf_llama_runtime_options_validate(C.byref(o)) == -1
    assert lib.cf_llama_runtime_create(C.byref(o)) is None
    o.allow_dense_fallback, o.require_cuda = 0, 0
    assert lib.cf_llama_runtime_options_validate(C.byref(o)) == -1
    o.require_cuda, o.kv.query_head_count = 1, 7           # the adapter's own options are checked too
    assert lib.cf_llama_runtime_options_validate(C.byref(o)) == -1
    o = _runtime_options()
    o.struct_size -= 4
    assert lib.cf_llama_runtime_options_validate(C.byref(o)) == -1
    assert lib.cf_llama_runtime_options_validate(None) == -1

    d = _runtime_options(backend=DENSE)
    d.require_cuda, d.allow_dense_fallback = 0, 1          # fine for the dense backend
    assert lib.cf_llama_runtime_options_validate(C.byref(d)) == 0
    r = C.c_void_p(lib.cf_llama_runtime_create(C.byref(d)))
    assert r
    assert lib.cf_llama_runtime_record_dense_fallback(r) == 0
    assert lib.cf_llama_runtime_record_compressed_launch(r, C.c_uint64(1), C.c_uint64(1)) == -1
    assert lib.cf_llama_runtime_last_error(r) == b"compressed launch recorded for dense backend"
    k = np.zeros((1, 2, 64), np.float32)
    view = LlamaTensorView(k.ctypes.data, 2 * 64 * 4, 64 * 4, 4, 1, 2, 64, 0)
    assert lib.cf_llama_runtime_append(r, 0, 0, C.byref(view), C.byref(view), None) == -1
    assert lib.cf_llama_runtime_last_error(r) == b"ChromoFold backend is not selected"
    assert lib.cf_llama_runtime_record_cuda_error(r) == -1
    assert lib.cf_llama_runtime_last_error(r) == b"CUDA execution failed"
    s = LlamaRuntimeSnapshot()
    assert lib.cf_llama_runtime_snapshot_get(r, C.byref(s)) == 0
    assert (s.backend_selected, s.initialized, s.dense_fallback_allowed, s.evidence_complete) == (DENSE, 1, 1, 0)
    assert (s.counters.dense_fallback_launches, s.counters.rejected_operations, s.counters.cuda_errors) == (1, 3, 1)
    path = str(tmp_path / "evidence.json").encode()
    assert lib.cf_llama_runtime_write_json(r, path) == 0
    doc = json.load(open(path))
    assert doc["backend_selected"] == 0 and doc["evidence_complete"] == 0
    assert doc["counters"]["rejected_operations"] == 3 and doc["counters"]["cuda_errors"] == 1
    assert set(doc["kv"]) == {"appended_tokens", "sealed_tokens", "sealed_pages", "active_tokens", "dense_active_bytes",
                              "compressed_bytes", "descriptor_bytes"}
    assert lib.cf_llama_runtime_write_json(r, b"/nonexistent-directory/x.json") == -1
    assert lib.cf_llama_runtime_write_json(r, None) == -1
    assert lib.cf_llama_runtime_snapshot_get(r, None) == -1
    lib.cf_llama_runtime_destroy(r)
    lib.cf_llama_runtime_destroy(None)
    assert lib.cf_llama_runtime_last_error(None) == b"null runtime"
    assert lib.cf_llama_runtime_append(None, 0, 0, None, None, None) == -1


def test_forwarding_bridges_refuse_bad_options_without_a_gpu(native):
    """chromofold_device_seal_bridge.cpp:12-13, device_kv_graph_bridge.cpp:13-15, llama_server_multisequence_bridge.cpp:32."""
    lib = native.lib()
    for f in ("cf_llama_device_seal_bridge_create", "cf_llama_device_graph_create", "cf_llama_server_cuda_bridge_create"):
        getattr(lib, f).restype = C.c_void_p
    for f in ("cf_llama_device_seal_bridge_last_error", "cf_llama_device_graph_last_error", "cf_llama_server_cuda_last_error"):
        getattr(lib, f).restype = C.c_char_p
    so = LlamaDeviceSealOptions()
    so.struct_size, so.require_cuda, so.allow_dense_fallback = C.sizeof(so), 0, 0
    assert lib.cf_llama_device_seal_bridge_create(C.byref(so)) is None          # CUDA must be required
    so.require_cuda, so.allow_dense_fallback = 1, 1
    assert lib.cf_llama_device_seal_bridge_create(C.byref(so)) is None          # dense fallback must be off
    so.allow_dense_fallback, so.struct_size = 0, 12
    assert lib.cf_llama_device_seal_bridge_create(C.byref(so)) is None
    assert lib.cf_llama_device_seal_bridge_create(None) is None
    assert lib.cf_llama_device_seal_bridge_stage(None, 0, 0, None, None, 0, None) == -1
    assert lib.cf_llama_device_seal_bridge_seal(None, 0, None) == -1
    assert lib.cf_llama_device_seal_bridge_evidence(None, None, None) == -1
    assert lib.cf_llama_device_seal_bridge_last_error(None) == b"null llama device seal bridge"
    lib.cf_llama_device_seal_bridge_destroy(None, None)

    go = LlamaDeviceGraphOptions()
    go.struct_size = C.sizeof(go)
    for flags in ((0, 1, 1), (1, 0, 1), (1, 1, 0)):
        go.causal, go.linear_sequence_only, go.dense_fallback_forbidden = flags
        assert lib.cf_llama_device_graph_create(C.byref(go)) is None
    assert lib.cf_llama_device_graph_create(None) is None
    assert lib.cf_llama_device_graph_append_async(None, 0, 0, None, None, None) == -1
    assert lib.cf_llama_device_graph_get_counters(None, None) == -1
    assert lib.cf_llama_device_graph_last_error(None) == b"null llama device graph"

    assert lib.cf_llama_server_cuda_bridge_create(None) is None
    assert lib.cf_llama_server_cuda_slot_create(None, C.c_int64(1)) == -1
    assert lib.cf_llama_server_cuda_shutdown_audit(None) == -1
    assert lib.cf_llama_server_cuda_last_error(None) == b"null llama-server CUDA bridge"

    ms = native.ms_bridge_lib()
    ms.cf_llama_server_multisequence_create.restype = C.c_void_p
    ms.cf_llama_server_multisequence_last_error.restype = C.c_char_p
    cfg = LlamaServerMultisequenceConfig()
    cfg.cache.layer_count, cfg.cache.kv_head_count, cfg.cache.query_head_count = 1, 8, 32
    cfg.cache.head_dim, cfg.cache.page_size, cfg.cache.gqa_group_size = 128, 16, 4
    cfg.strict_no_fallback = 0
    assert ms.cf_llama_server_multisequence_create(C.byref(cfg)) is None        # the fallback ban must be stated
    assert ms.cf_llama_server_multisequence_create(None) is None
    assert ms.cf_llama_server_slot_create(None, C.c_int64(0), C.c_int64(0)) == -1
    assert ms.cf_llama_server_audit(None) == -1
    assert ms.cf_llama_server_multisequence_last_error(None) == b"null llama-server multisequence bridge"


# ---- on a GPU: each bridge must behave exactly like the ABI it forwards to ----------------------------------------
@pytest.mark.gpu
def test_runtime_bridge_and_graph_state_on_the_chromofold_backend(native, tmp_path):
    import torch  # noqa: F401  (makes sure a CUDA context can be had)
    lib = native.lib()
    lib.cf_llama_runtime_create.restype = C.c_void_p
    lib.cf_llama_runtime_last_error.restype = C.c_char_p
    lib.cf_llama_graph_create.restype = C.c_void_p
    lib.cf_llama_graph_last_error.restype = C.c_char_p
    layers, hq, hkv, dim, page, tokens = 2, 8, 2, 64, 64, 70
    o = _runtime_options(layers=layers, hq=hq, hkv=hkv, dim=dim, page=page)
    r = C.c_void_p(lib.cf_llama_runtime_create(C.byref(o)))
    assert r
    rng = np.random.default_rng(3)
    k = rng.standard_normal((tokens, hkv, dim)).astype(np.float32)
    v = rng.standard_normal((tokens, hkv, dim)).astype(np.float32)

    def view(a, begin, count, dtype_code=0):
        return LlamaTensorView(a[begin:].ctypes.data, hkv * dim * 4, dim * 4, 4, count, hkv, dim, dtype_code)

    for layer in range(layers):
        for begin, count in ((0, 50), (50, 20)):
            kv, vv = view(k, begin, count), view(v, begin, count)
            assert lib.cf_llama_runtime_append(r, layer, begin, C.byref(kv), C.byref(vv), None) == 0, lib.cf_llama_runtime_last_error(r)
    # refused and counted: a strided view, a half-precision view, a head count that is not the cache's, a gap in positions
    kv, vv = view(k, 0, 1), view(v, 0, 1)
    kv.head_stride_bytes = (dim + 8) * 4
    assert lib.cf_llama_runtime_append(r, 0, tokens, C.byref(kv), C.byref(vv), None) == -1
    assert b"contiguous fp32" in lib.cf_llama_runtime_last_error(r)
    kv = view(k, 0, 1, dtype_code=1)
    assert lib.cf_llama_runtime_append(r, 0, tokens, C.byref(kv), C.byref(vv), None) == -1
    one = LlamaTensorView(k.ctypes.data, dim * 4, dim * 4, 4, 1, 1, dim, 0)
    assert lib.cf_llama_runtime_append(r, 0, tokens, C.byref(one), C.byref(one), None) == -1
    assert b"topology" in lib.cf_llama_runtime_last_error(r)
    kv, vv = view(k, 0, 1), view(v, 0, 1)
    assert lib.cf_llama_runtime_append(r, 0, tokens + 5, C.byref(kv), C.byref(vv), None) == -1      # the adapter's refusal
    assert b"contiguous" in lib.cf_llama_runtime_last_error(r)
    assert lib.cf_llama_runtime_record_dense_fallback(r) == -1
    assert lib.cf_llama_runtime_last_error(r) == b"dense fallback is disabled"
    s = LlamaRuntimeSnapshot()
    assert lib.cf_llama_runtime_snapshot_get(r, C.byref(s)) == 0
    assert s.counters.append_calls == 2 * layers and s.counters.appended_values == layers * tokens * hkv * dim * 2
    assert s.counters.rejected_operations == 5 and s.counters.dense_fallback_launches == 1
    assert s.kv.appended_tokens == layers * hkv * tokens and s.kv.sealed_pages == layers * hkv and s.kv.active_tokens == layers * hkv * 6
    assert s.evidence_complete == 0                       # a dense fallback was recorded: the evidence stays incomplete
    lib.cf_llama_runtime_destroy(r)

    # the graph state owns such a runtime; its evidence file is the runtime's JSON
    path = str(tmp_path / "graph.json").encode()
    g = C.c_void_p(lib.cf_llama_graph_create(C.byref(_graph_options(page=page, path=path)), C.byref(_topology(layers, hq, hkv, dim))))
    assert g
    kv, vv = view(k, 0, 64), view(v, 0, 64)
    assert lib.cf_llama_graph_append_device(g, 0, 0, C.byref(kv), C.byref(vv), None) == 0, lib.cf_llama_graph_last_error(g)
    assert lib.cf_llama_graph_append_device(g, 0, 3, C.byref(kv), C.byref(vv), None) == -1
    assert lib.cf_llama_graph_record_attention(g, C.c_uint64(64 * hkv * dim * 2), C.c_uint64(0)) == 0
    assert lib.cf_llama_graph_write_evidence(g) == 0
    doc = json.load(open(path))
    assert doc["backend_selected"] == 1 and doc["evidence_complete"] == 1
    assert doc["kv"]["sealed_pages"] == hkv and doc["counters"]["compressed_attention_launches"] == 1
    assert lib.cf_llama_graph_record_dense_dispatch(g) == -1
    assert lib.cf_llama_graph_last_error(g) == b"dense graph dispatch is forbidden for ChromoFold"
    assert lib.cf_llama_graph_write_evidence(g) == 0
    assert json.load(open(path))["evidence_complete"] == 0          # the forbidden dispatch shows in the evidence
    c = LlamaGraphCounters()
    lib.cf_llama_graph_get_counters(g, C.byref(c))
    assert (c.graph_append_calls, c.graph_attention_dispatches, c.graph_dense_dispatches, c.unsupported_graphs) == (1, 1, 1, 2)
    lib.cf_llama_graph_destroy(g)


@pytest.mark.gpu
def test_device_seal_bridge_and_device_graph_bridge_equal_their_engines(native):
    import torch
    from compat_types import DeviceKvConfig, DeviceSealConfig
    lib = native.lib()
    for f in ("cf_llama_device_seal_bridge_create", "cf_llama_device_graph_create", "cf_device_seal_create", "cf_device_kv_create"):
        getattr(lib, f).restype = C.c_void_p
    lib.cf_llama_device_seal_bridge_last_error.restype = C.c_char_p
    lib.cf_llama_device_graph_last_error.restype = C.c_char_p
    layers, hkv, hq, d, page = 1, 2, 8, 128, 64
    rng = np.random.default_rng(12)
    tokens = page + 5
    dk = torch.from_numpy(rng.standard_normal((tokens, hkv, d)).astype(np.float32)).cuda()
    dv = torch.from_numpy(rng.standard_normal((tokens, hkv, d)).astype(np.float32)).cuda()
    q = torch.from_numpy(rng.standard_normal((2, hq, d)).astype(np.float32)).cuda()
    qv = TensorView(q.data_ptr(), 3, 2, hq, d, hq * d * 4, d * 4, 4, 0)
    scale = C.c_float(1.0 / np.sqrt(d))
    ptr = lambda t: C.c_void_p(t.data_ptr())

    so = LlamaDeviceSealOptions()
    so.struct_size, so.seal, so.require_cuda = C.sizeof(so), DeviceSealConfig(layers, hkv, hq, d, page, hq // hkv, 64, 0), 1
    b = C.c_void_p(lib.cf_llama_device_seal_bridge_create(C.byref(so)))
    e = C.c_void_p(lib.cf_device_seal_create(C.byref(so.seal)))
    assert b and e
    n, complete = DeviceSealCounters(), C.c_uint32(9)
    assert lib.cf_llama_device_seal_bridge_seal(b, 0, None) == -1                  # nothing staged: the engine's refusal and text
    assert lib.cf_llama_device_seal_bridge_last_error(b) != b""
    assert lib.cf_llama_device_seal_bridge_stage(b, 0, 0, ptr(dk), ptr(dv), page, None) == 0
    assert lib.cf_llama_device_seal_bridge_last_error(b) == b""
    assert lib.cf_llama_device_seal_bridge_evidence(b, C.byref(n), C.byref(complete)) == 0 and complete.value == 0
    assert lib.cf_llama_device_seal_bridge_seal(b, 0, None) == 0
    assert lib.cf_llama_device_seal_bridge_stage(b, 0, page, ptr(dk[page:]), ptr(dv[page:]), 5, None) == 0
    assert lib.cf_device_seal_stage_active_page(e, 0, 0, ptr(dk), ptr(dv), page, None) == 0
    assert lib.cf_device_seal_full_page_async(e, 0, None) == 0
    assert lib.cf_device_seal_stage_active_page(e, 0, page, ptr(dk[page:]), ptr(dv[page:]), 5, None) == 0
    out_b = torch.zeros((2, hq, d), dtype=torch.float32, device="cuda")
    out_e = torch.zeros_like(out_b)
    strides = (C.c_uint64(hq * d * 4), C.c_uint64(d * 4), C.c_uint64(4))
    assert lib.cf_llama_device_seal_bridge_attention(b, 0, C.byref(qv), ptr(out_b), 3, *strides, tokens - 2, scale, 0, None) == 0
    assert lib.cf_device_seal_attention_async(e, 0, C.byref(qv), ptr(out_e), 3, *strides, tokens - 2, scale, 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(out_b, out_e) and float(out_b.abs().max()) > 0
    assert lib.cf_llama_device_seal_bridge_evidence(b, C.byref(n), C.byref(complete)) == 0
    assert complete.value == 1 and n.seal_successes == 1 and n.descriptor_publications == 1 and n.compressed_attention_launches == 1
    lib.cf_llama_device_seal_bridge_destroy(b, None)
    lib.cf_device_seal_destroy(e, None)

    go = LlamaDeviceGraphOptions()
    go.struct_size, go.kv = C.sizeof(go), DeviceKvConfig(layers, hkv, hq, d, page, hq // hkv, 0)
    go.causal, go.linear_sequence_only, go.dense_fallback_forbidden = 1, 1, 1
    gb = C.c_void_p(lib.cf_llama_device_graph_create(C.byref(go)))
    p = C.c_void_p(lib.cf_device_kv_create(C.byref(go.kv)))
    assert gb and p
    kview = lambda t, begin, count: TensorView(t[begin:].data_ptr(), 3, count, hkv, d, hkv * d * 4, d * 4, 4, 0)
    for begin, count in ((0, 30), (30, 10)):
        kv, vv = kview(dk, begin, count), kview(dv, begin, count)
        assert lib.cf_llama_device_graph_append_async(gb, 0, begin, C.byref(kv), C.byref(vv), None) == 0
        assert lib.cf_device_kv_append_async(p, 0, begin, C.byref(kv), C.byref(vv), None) == 0
    kv, vv = kview(dk, 0, 1), kview(dv, 0, 1)
    assert lib.cf_llama_device_graph_append_async(gb, 0, 3, C.byref(kv), C.byref(vv), None) == -1
    assert b"non-contiguous" in lib.cf_llama_device_graph_last_error(gb)
    out_g, out_p = torch.zeros((2, hq, d), dtype=torch.float32, device="cuda"), torch.zeros((2, hq, d), dtype=torch.float32, device="cuda")
    assert lib.cf_llama_device_graph_attention_async(gb, 0, ptr(q), ptr(out_g), 2, 38, scale, 0, None) == 0
    assert lib.cf_llama_device_graph_last_error(gb) == b""
    assert lib.cf_device_kv_attention_async(p, 0, ptr(q), ptr(out_p), 2, 38, scale, 0, None) == 0
    torch.cuda.synchronize()
    assert torch.equal(out_g, out_p) and float(out_g.abs().max()) > 0
    # the bridge has no seal call (nor has the reference's): once the active page is full the next append is refused
    kv, vv = kview(dk, 40, page - 40), kview(dv, 40, page - 40)
    assert lib.cf_llama_device_graph_append_async(gb, 0, 40, C.byref(kv), C.byref(vv), None) == 0
    kv, vv = kview(dk, page, 1), kview(dv, page, 1)
    assert lib.cf_llama_device_graph_append_async(gb, 0, page, C.byref(kv), C.byref(vv), None) == -1
    assert b"seal before retry" in lib.cf_llama_device_graph_last_error(gb)
    c = DeviceKvCounters()
    assert lib.cf_llama_device_graph_get_counters(gb, C.byref(c)) == 0 and c.device_append_calls == 3 and c.dense_fallback_launches == 0
    lib.cf_llama_device_graph_destroy(gb, None)
    lib.cf_device_kv_destroy(p, None)


@pytest.mark.gpu
def test_llama_server_slot_bridges_over_the_resolver_and_the_cache(native):
    """Slots of llama-server over the CUDA sequence resolver (llama_server_cuda_resolver_bridge.cpp) and over the
    multi-sequence cache (llama_server_multisequence_bridge.cpp): create / duplicate / copy / cancel / reset / audit."""
    import torch  # noqa: F401
    lib, ms = native.lib(), native.ms_bridge_lib()
    lib.cf_llama_server_cuda_bridge_create.restype = C.c_void_p
    lib.cf_llama_server_cuda_last_error.restype = C.c_char_p
    i64 = C.c_int64
    b = C.c_void_p(lib.cf_llama_server_cuda_bridge_create(C.byref(MsConfig(1, 8, 32, 128, 64, 4, 0))))
    assert b
    assert lib.cf_llama_server_cuda_slot_create(b, i64(3)) == 0
    assert lib.cf_llama_server_cuda_slot_create(b, i64(3)) == -1              # the resolver refuses a duplicate id
    first_error = lib.cf_llama_server_cuda_last_error(b)
    assert first_error != b""
    assert lib.cf_llama_server_cuda_slot_copy_async(b, i64(3), i64(4), None) == 0
    assert lib.cf_llama_server_cuda_last_error(b) == first_error              # this bridge keeps the last failure's text
    assert lib.cf_llama_server_cuda_slot_copy_async(b, i64(99), i64(5), None) == -1
    assert lib.cf_llama_server_cuda_slot_cancel_async(b, i64(4), None) == 0
    assert lib.cf_llama_server_cuda_slot_reset_async(b, i64(3), None) == 0
    assert lib.cf_llama_server_cuda_slot_reset_async(b, i64(3), None) == -1   # gone
    assert lib.cf_llama_server_cuda_dispatch_batch_async(b, None, 0, None) == -1
    assert lib.cf_llama_server_cuda_shutdown_audit(b) == 0
    lib.cf_llama_server_cuda_bridge_destroy(b, None)

    ms.cf_llama_server_multisequence_create.restype = C.c_void_p
    ms.cf_llama_server_multisequence_last_error.restype = C.c_char_p
    cfg = LlamaServerMultisequenceConfig()
    cfg.cache.layer_count, cfg.cache.kv_head_count, cfg.cache.query_head_count = 1, 8, 32
    cfg.cache.head_dim, cfg.cache.page_size, cfg.cache.gqa_group_size = 128, 16, 4
    cfg.strict_no_fallback = 1
    m = C.c_void_p(ms.cf_llama_server_multisequence_create(C.byref(cfg)))
    assert m
    assert ms.cf_llama_server_slot_create(m, i64(0), i64(100)) == 0
    assert ms.cf_llama_server_slot_create(m, i64(0), i64(101)) == -1
    assert ms.cf_llama_server_multisequence_last_error(m) == b"slot already exists"
    assert ms.cf_llama_server_slot_create(m, i64(1), i64(100)) == -1          # the cache refuses a duplicate sequence id
    assert ms.cf_llama_server_multisequence_last_error(m) not in (b"", b"slot already exists")
    assert ms.cf_llama_server_sequence_copy_async(m, i64(100), i64(200), 0, 0, None) == 0
    assert ms.cf_llama_server_multisequence_last_error(m) == b""
    assert ms.cf_llama_server_context_shift_async(m, i64(100), 0, 0, 0, None) == 0
    assert ms.cf_llama_server_sequence_remove_async(m, i64(200), i64(-1), i64(-1), None) == 0
    assert ms.cf_llama_server_sequence_remove_async(m, i64(200), i64(-1), i64(-1), None) == -1
    assert ms.cf_llama_server_slot_reset_async(m, i64(7), None) == -1
    assert ms.cf_llama_server_multisequence_last_error(m) == b"slot does not exist"
    assert ms.cf_llama_server_slot_reset_async(m, i64(0), None) == 0          # removes sequence 100 and reclaims
    assert ms.cf_llama_server_slot_create(m, i64(0), i64(100)) == 0           # both ids are free again
    assert ms.cf_llama_server_cancel_sequence_async(m, i64(100), None) == 0
    assert ms.cf_llama_server_slot_create(m, i64(0), i64(102)) == 0           # the cancel forgot slot 0
    assert ms.cf_llama_server_batch_attention_async(m, None, 0, None) == -1
    assert ms.cf_llama_server_audit(m) == 0
    ms.cf_llama_server_multisequence_destroy(m, None)
