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
