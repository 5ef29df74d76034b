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
