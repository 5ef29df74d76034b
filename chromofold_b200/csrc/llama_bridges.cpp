// llama_bridges.cpp — the llama.cpp-side bridges of compat_bridges.h. Host code only: each bridge owns one handle of an
// ABI this library already serves (adapter, device seal engine, device KV dataplane, CUDA sequence resolver), forwards
// to it, keeps the last error text and the counters the reference's evidence files are made from
// (integrations/llama.cpp/chromofold_runtime_bridge.cpp, graph/chromofold_graph_contract.cpp,
// chromofold_device_seal_bridge.cpp, device_kv_graph_bridge.cpp, multisequence/llama_server_cuda_resolver_bridge.cpp).
#include <cstdio>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "chromofold_b200/compat_bridges.h"

namespace {

// Outcome of one bridge call: ok, or refused with a reason.
struct Outcome {
    bool ok;
    std::string why;
    static Outcome yes() { return {true, {}}; }
    static Outcome no(const char *reason) { return {false, reason ? reason : "unknown error"}; }
};

// A forwarded call: 0 clears the bridge's error text, anything else copies the owner's.
template <class ErrorText>
int forwarded(int rc, std::string &error, ErrorText &&text) {
    if (rc == 0) error.clear();
    else error = text();
    return rc;
}

bool is_chromofold(const cf_llama_kv_options &kv) { return kv.backend == CF_LLAMA_KV_BACKEND_CHROMOFOLD; }

// [token][head][dim] fp32 without gaps: what the runtime bridge accepts (chromofold_runtime_bridge.cpp:33-39).
bool packed_f32(const cf_llama_tensor_view *v) {
    if (!v || !v->data || v->scalar_type != CF_LLAMA_SCALAR_F32 || !v->token_count || !v->head_count || !v->head_dim) return false;
    const uint64_t row = static_cast<uint64_t>(v->head_dim) * sizeof(float);
    return v->element_stride_bytes == sizeof(float) && v->head_stride_bytes == row && v->token_stride_bytes == row * v->head_count;
}

}  // namespace

// ---- runtime bridge ---------------------------------------------------------------------------------------------
struct cf_llama_runtime {
    cf_llama_runtime_options options{};
    cf_llama_kv_adapter *adapter = nullptr;
    cf_llama_runtime_counters counters{};
    std::string error;
    std::vector<float> head_k, head_v;   // one head's rows, gathered for the adapter's per-head append

    // every refused operation is counted (chromofold_runtime_bridge.cpp:20-31)
    int settle(const Outcome &v) {
        if (v.ok) {
            error.clear();
            return 0;
        }
        error = v.why;
        ++counters.rejected_operations;
        return -1;
    }
};

extern "C" int cf_llama_runtime_options_validate(const cf_llama_runtime_options *options) {
    if (!options || options->struct_size != sizeof(cf_llama_runtime_options)) return -1;
    if (cf_llama_kv_options_validate(&options->kv) != 0) return -1;
    if (is_chromofold(options->kv) && (options->allow_dense_fallback != 0 || options->require_cuda == 0)) return -1;
    return 0;
}

extern "C" cf_llama_runtime *cf_llama_runtime_create(const cf_llama_runtime_options *options) {
    if (cf_llama_runtime_options_validate(options) != 0) return nullptr;
    cf_llama_runtime *runtime = new (std::nothrow) cf_llama_runtime();
    if (!runtime) return nullptr;
    runtime->options = *options;
    if (is_chromofold(options->kv)) {
        runtime->adapter = cf_llama_kv_create(&options->kv);
        if (!runtime->adapter) {
            delete runtime;
            return nullptr;
        }
    }
    return runtime;
}

extern "C" void cf_llama_runtime_destroy(cf_llama_runtime *runtime) {
    if (!runtime) return;
    if (runtime->adapter) cf_llama_kv_destroy(runtime->adapter);
    delete runtime;
}

extern "C" int cf_llama_runtime_append(cf_llama_runtime *runtime, uint32_t layer, uint32_t token_begin, const cf_llama_tensor_view *keys,
                                       const cf_llama_tensor_view *values, void *stream) {
    if (!runtime) return -1;
    auto run = [&]() -> Outcome {
        if (!is_chromofold(runtime->options.kv) || !runtime->adapter) return Outcome::no("ChromoFold backend is not selected");
        if (!packed_f32(keys) || !packed_f32(values)) return Outcome::no("initial runtime bridge requires contiguous fp32 K/V tensors");
        const cf_llama_kv_options &kv = runtime->options.kv;
        if (keys->token_count != values->token_count || keys->head_count != values->head_count || keys->head_dim != values->head_dim ||
            keys->head_count != kv.kv_head_count || keys->head_dim != kv.head_dim)
            return Outcome::no("K/V tensor topology does not match configured cache");
        const uint32_t tokens = keys->token_count, heads = keys->head_count, dim = keys->head_dim;
        const float *k = static_cast<const float *>(keys->data), *v = static_cast<const float *>(values->data);
        try {
            runtime->head_k.resize(static_cast<size_t>(tokens) * dim);
            runtime->head_v.resize(static_cast<size_t>(tokens) * dim);
        } catch (...) {
            return Outcome::no("out of host memory");
        }
        for (uint32_t h = 0; h < heads; ++h) {   // the adapter takes one head's rows at a time
            for (uint32_t t = 0; t < tokens; ++t) {
                const size_t src = (static_cast<size_t>(t) * heads + h) * dim, dst = static_cast<size_t>(t) * dim;
                std::memcpy(&runtime->head_k[dst], k + src, dim * sizeof(float));
                std::memcpy(&runtime->head_v[dst], v + src, dim * sizeof(float));
            }
            if (cf_llama_kv_append(runtime->adapter, layer, h, token_begin, runtime->head_k.data(), runtime->head_v.data(), tokens, stream) != 0)
                return Outcome::no(cf_llama_kv_last_error(runtime->adapter));
        }
        ++runtime->counters.append_calls;
        runtime->counters.appended_values += static_cast<uint64_t>(tokens) * heads * dim * 2u;
        return Outcome::yes();
    };
    return runtime->settle(run());
}

extern "C" int cf_llama_runtime_record_compressed_launch(cf_llama_runtime *runtime, uint64_t sealed_values, uint64_t active_values) {
    if (!runtime) return -1;
    if (!is_chromofold(runtime->options.kv)) return runtime->settle(Outcome::no("compressed launch recorded for dense backend"));
    ++runtime->counters.compressed_attention_launches;
    runtime->counters.sealed_values_consumed += sealed_values;
    runtime->counters.active_values_consumed += active_values;
    return runtime->settle(Outcome::yes());
}

extern "C" int cf_llama_runtime_record_dense_fallback(cf_llama_runtime *runtime) {
    if (!runtime) return -1;
    ++runtime->counters.dense_fallback_launches;   // counted even when it is refused
    return runtime->settle(runtime->options.allow_dense_fallback ? Outcome::yes() : Outcome::no("dense fallback is disabled"));
}

extern "C" int cf_llama_runtime_record_cuda_error(cf_llama_runtime *runtime) {
    if (!runtime) return -1;
    ++runtime->counters.cuda_errors;
    return runtime->settle(Outcome::no("CUDA execution failed"));   // recording an error is itself reported as one
}

extern "C" int cf_llama_runtime_snapshot_get(const cf_llama_runtime *runtime, cf_llama_runtime_snapshot *snapshot) {
    if (!runtime || !snapshot) return -1;
    *snapshot = cf_llama_runtime_snapshot{};
    snapshot->backend_selected = runtime->options.kv.backend;
    snapshot->initialized = 1;
    snapshot->dense_fallback_allowed = runtime->options.allow_dense_fallback;
    snapshot->counters = runtime->counters;
    if (runtime->adapter && cf_llama_kv_get_stats(runtime->adapter, &snapshot->kv) != 0) return -1;
    const cf_llama_runtime_counters &c = runtime->counters;
    snapshot->evidence_complete = is_chromofold(runtime->options.kv) && c.compressed_attention_launches > 0 &&
                                  c.sealed_values_consumed > 0 && c.dense_fallback_launches == 0 && c.cuda_errors == 0;
    return 0;
}

extern "C" int cf_llama_runtime_write_json(const cf_llama_runtime *runtime, const char *path) {
    cf_llama_runtime_snapshot s{};
    if (!runtime || !path || cf_llama_runtime_snapshot_get(runtime, &s) != 0) return -1;
    FILE *f = std::fopen(path, "wb");
    if (!f) return -1;
    struct Field { const char *name; uint64_t value; };
    const Field kv[] = {{"appended_tokens", s.kv.appended_tokens}, {"sealed_tokens", s.kv.sealed_tokens}, {"sealed_pages", s.kv.sealed_pages},
                        {"active_tokens", s.kv.active_tokens}, {"dense_active_bytes", s.kv.dense_active_bytes},
                        {"compressed_bytes", s.kv.compressed_bytes}, {"descriptor_bytes", s.kv.descriptor_bytes}};
    const Field counters[] = {{"append_calls", s.counters.append_calls}, {"appended_values", s.counters.appended_values},
                              {"compressed_attention_launches", s.counters.compressed_attention_launches},
                              {"sealed_values_consumed", s.counters.sealed_values_consumed},
                              {"active_values_consumed", s.counters.active_values_consumed},
                              {"dense_fallback_launches", s.counters.dense_fallback_launches},
                              {"rejected_operations", s.counters.rejected_operations}, {"cuda_errors", s.counters.cuda_errors}};
    bool good = std::fprintf(f, "{\n  \"backend_selected\":%u,\n  \"evidence_complete\":%u,\n  \"kv\":{", s.backend_selected, s.evidence_complete) >= 0;
    auto object = [&](const Field *fields, size_t n) {
        for (size_t i = 0; i < n; ++i)
            good = good && std::fprintf(f, "%s\"%s\":%llu", i ? "," : "", fields[i].name, static_cast<unsigned long long>(fields[i].value)) >= 0;
    };
    object(kv, sizeof kv / sizeof kv[0]);
    good = good && std::fprintf(f, "},\n  \"counters\":{") >= 0;
    object(counters, sizeof counters / sizeof counters[0]);
    good = good && std::fprintf(f, "}\n}\n") >= 0;
    return std::fclose(f) == 0 && good ? 0 : -1;
}

extern "C" const char *cf_llama_runtime_last_error(const cf_llama_runtime *runtime) {
    return runtime ? runtime->error.c_str() : "null runtime";
}

// ---- graph contract -----------------------------------------------------------------------------------------------
struct cf_llama_graph_state {
    cf_llama_graph_options options{};
    cf_llama_model_topology topology{};
    cf_llama_runtime *runtime = nullptr;   // only under the ChromoFold backend
    cf_llama_graph_counters counters{};
    std::string evidence_path, error;

    int settle(const Outcome &v) {   // every refused graph operation is counted (chromofold_graph_contract.cpp:18-31)
        if (v.ok) {
            error.clear();
            return 0;
        }
        error = v.why;
        ++counters.unsupported_graphs;
        return -1;
    }
};

extern "C" int cf_llama_graph_options_validate(const cf_llama_graph_options *options) {
    if (!options || options->struct_size != sizeof(cf_llama_graph_options)) return -1;
    if (options->backend == CF_LLAMA_KV_BACKEND_DENSE) return 0;
    if (options->backend != CF_LLAMA_KV_BACKEND_CHROMOFOLD) return -1;
    return options->page_size == 64 || options->page_size == 128 || options->page_size == 256 ? 0 : -1;
}

extern "C" int cf_llama_model_topology_validate(const cf_llama_model_topology *t) {
    if (!t || t->struct_size != sizeof(cf_llama_model_topology)) return -1;
    if (!t->uniform_kv_geometry || !t->causal || t->recurrent) return -1;
    if (!t->layer_count || !t->query_head_count || !t->kv_head_count || !t->head_dim) return -1;
    return t->head_dim <= 128 && t->query_head_count % t->kv_head_count == 0 ? 0 : -1;
}

extern "C" cf_llama_graph_state *cf_llama_graph_create(const cf_llama_graph_options *options, const cf_llama_model_topology *topology) {
    if (cf_llama_graph_options_validate(options) != 0 || cf_llama_model_topology_validate(topology) != 0) return nullptr;
    cf_llama_graph_state *state = new (std::nothrow) cf_llama_graph_state();
    if (!state) return nullptr;
    state->options = *options;
    state->topology = *topology;
    try {
        if (options->evidence_path) state->evidence_path = options->evidence_path;
    } catch (...) {
        delete state;
        return nullptr;
    }
    state->options.evidence_path = nullptr;   // the caller's string is not kept
    if (options->backend == CF_LLAMA_KV_BACKEND_CHROMOFOLD) {
        cf_llama_runtime_options r{};
        r.struct_size = sizeof r;
        r.kv.struct_size = sizeof r.kv;
        r.kv.backend = options->backend;
        r.kv.layer_count = topology->layer_count;
        r.kv.kv_head_count = topology->kv_head_count;
        r.kv.query_head_count = topology->query_head_count;
        r.kv.head_dim = topology->head_dim;
        r.kv.page_size = options->page_size;
        r.kv.gqa_group_size = topology->query_head_count / topology->kv_head_count;
        r.require_cuda = 1;
        r.allow_dense_fallback = 0;
        state->runtime = cf_llama_runtime_create(&r);
        if (!state->runtime) {
            delete state;
            return nullptr;
        }
    }
    return state;
}

extern "C" void cf_llama_graph_destroy(cf_llama_graph_state *state) {
    if (!state) return;
    cf_llama_runtime_destroy(state->runtime);
    delete state;
}

extern "C" int cf_llama_graph_append_device(cf_llama_graph_state *state, uint32_t layer, uint32_t token_begin,
                                            const cf_llama_tensor_view *keys, const cf_llama_tensor_view *values, void *stream) {
    if (!state) return -1;
    if (!state->runtime) return state->settle(Outcome::no("ChromoFold graph backend is not active"));
    if (cf_llama_runtime_append(state->runtime, layer, token_begin, keys, values, stream) != 0)
        return state->settle(Outcome::no(cf_llama_runtime_last_error(state->runtime)));
    ++state->counters.graph_append_calls;
    return state->settle(Outcome::yes());
}

extern "C" int cf_llama_graph_record_attention(cf_llama_graph_state *state, uint64_t sealed_values, uint64_t active_values) {
    if (!state) return -1;
    if (!state->runtime) return state->settle(Outcome::no("compressed attention recorded without runtime"));
    if (cf_llama_runtime_record_compressed_launch(state->runtime, sealed_values, active_values) != 0)
        return state->settle(Outcome::no(cf_llama_runtime_last_error(state->runtime)));
    ++state->counters.graph_attention_dispatches;
    return state->settle(Outcome::yes());
}

extern "C" int cf_llama_graph_record_dense_dispatch(cf_llama_graph_state *state) {
    if (!state) return -1;
    ++state->counters.graph_dense_dispatches;
    if (state->options.backend != CF_LLAMA_KV_BACKEND_CHROMOFOLD) return state->settle(Outcome::yes());
    if (state->runtime) cf_llama_runtime_record_dense_fallback(state->runtime);   // shows up in the runtime's evidence too
    return state->settle(Outcome::no("dense graph dispatch is forbidden for ChromoFold"));
}

extern "C" int cf_llama_graph_get_counters(const cf_llama_graph_state *state, cf_llama_graph_counters *counters) {
    if (!state || !counters) return -1;
    *counters = state->counters;
    return 0;
}

extern "C" int cf_llama_graph_write_evidence(const cf_llama_graph_state *state) {
    if (!state || !state->runtime || state->evidence_path.empty()) return -1;
    return cf_llama_runtime_write_json(state->runtime, state->evidence_path.c_str());
}

extern "C" const char *cf_llama_graph_last_error(const cf_llama_graph_state *state) {
    return state ? state->error.c_str() : "null graph state";
}

// ---- device seal bridge -------------------------------------------------------------------------------------------
struct cf_llama_device_seal_bridge {
    cf_llama_device_seal_options options{};
    cf_device_seal_engine *engine = nullptr;
    std::string error;
    int pass(int rc) { return forwarded(rc, error, [&] { return std::string(cf_device_seal_last_error(engine)); }); }
};

extern "C" cf_llama_device_seal_bridge *cf_llama_device_seal_bridge_create(const cf_llama_device_seal_options *options) {
    if (!options || options->struct_size != sizeof(cf_llama_device_seal_options) || !options->require_cuda || options->allow_dense_fallback)
        return nullptr;
    cf_llama_device_seal_bridge *bridge = new (std::nothrow) cf_llama_device_seal_bridge();
    if (!bridge) return nullptr;
    bridge->options = *options;
    bridge->engine = cf_device_seal_create(&options->seal);
    if (!bridge->engine) {
        delete bridge;
        return nullptr;
    }
    return bridge;
}

extern "C" void cf_llama_device_seal_bridge_destroy(cf_llama_device_seal_bridge *bridge, void *stream) {
    if (!bridge) return;
    cf_device_seal_destroy(bridge->engine, stream);
    delete bridge;
}

extern "C" int cf_llama_device_seal_bridge_stage(cf_llama_device_seal_bridge *bridge, uint32_t layer, uint32_t token_begin,
                                                 const float *active_k, const float *active_v, uint32_t token_count, void *stream) {
    return bridge ? bridge->pass(cf_device_seal_stage_active_page(bridge->engine, layer, token_begin, active_k, active_v, token_count, stream)) : -1;
}

extern "C" int cf_llama_device_seal_bridge_seal(cf_llama_device_seal_bridge *bridge, uint32_t layer, void *stream) {
    return bridge ? bridge->pass(cf_device_seal_full_page_async(bridge->engine, layer, stream)) : -1;
}

extern "C" int cf_llama_device_seal_bridge_attention(cf_llama_device_seal_bridge *bridge, uint32_t layer, const cf_device_tensor_view *query,
                                                     void *output, uint32_t output_scalar_type, uint64_t output_token_stride_bytes,
                                                     uint64_t output_head_stride_bytes, uint64_t output_element_stride_bytes,
                                                     uint32_t query_token_begin, float softmax_scale, uint32_t causal_window, void *stream) {
    if (!bridge) return -1;
    return bridge->pass(cf_device_seal_attention_async(bridge->engine, layer, query, output, output_scalar_type, output_token_stride_bytes,
                                                       output_head_stride_bytes, output_element_stride_bytes, query_token_begin,
                                                       softmax_scale, causal_window, stream));
}

extern "C" int cf_llama_device_seal_bridge_evidence(const cf_llama_device_seal_bridge *bridge, cf_device_seal_counters *counters,
                                                    uint32_t *complete) {
    if (!bridge || !counters || !complete || cf_device_seal_get_counters(bridge->engine, counters) != 0) return -1;
    // every seal published its descriptor, and compressed attention really consumed sealed values
    *complete = counters->seal_successes > 0 && counters->descriptor_publications == counters->seal_successes &&
                counters->compressed_attention_launches > 0 && counters->sealed_values_consumed > 0 && counters->cuda_errors == 0;
    return 0;
}

extern "C" const char *cf_llama_device_seal_bridge_last_error(const cf_llama_device_seal_bridge *bridge) {
    return bridge ? bridge->error.c_str() : "null llama device seal bridge";
}

// ---- device KV graph bridge ---------------------------------------------------------------------------------------
struct cf_llama_device_graph {
    cf_llama_device_graph_options options{};
    cf_device_kv_dataplane *dataplane = nullptr;
    std::string error;
    int pass(int rc) { return forwarded(rc, error, [&] { return std::string(cf_device_kv_last_error(dataplane)); }); }
};

extern "C" cf_llama_device_graph *cf_llama_device_graph_create(const cf_llama_device_graph_options *options) {
    if (!options || options->struct_size != sizeof(cf_llama_device_graph_options) || !options->causal || !options->linear_sequence_only ||
        !options->dense_fallback_forbidden)
        return nullptr;
    cf_llama_device_graph *graph = new (std::nothrow) cf_llama_device_graph();
    if (!graph) return nullptr;
    graph->options = *options;
    graph->dataplane = cf_device_kv_create(&options->kv);
    if (!graph->dataplane) {
        delete graph;
        return nullptr;
    }
    return graph;
}

extern "C" void cf_llama_device_graph_destroy(cf_llama_device_graph *graph, void *stream) {
    if (!graph) return;
    cf_device_kv_destroy(graph->dataplane, stream);
    delete graph;
}

extern "C" int cf_llama_device_graph_append_async(cf_llama_device_graph *graph, uint32_t layer, uint32_t token_begin,
                                                  const cf_device_tensor_view *keys, const cf_device_tensor_view *values, void *stream) {
    return graph ? graph->pass(cf_device_kv_append_async(graph->dataplane, layer, token_begin, keys, values, stream)) : -1;
}

extern "C" int cf_llama_device_graph_attention_async(cf_llama_device_graph *graph, uint32_t layer, const float *query, float *output,
                                                     uint32_t query_token_count, uint32_t query_token_begin, float softmax_scale,
                                                     uint32_t causal_window, void *stream) {
    if (!graph) return -1;
    return graph->pass(cf_device_kv_attention_async(graph->dataplane, layer, query, output, query_token_count, query_token_begin,
                                                    softmax_scale, causal_window, stream));
}

extern "C" int cf_llama_device_graph_get_counters(const cf_llama_device_graph *graph, cf_device_kv_counters *counters) {
    return graph ? cf_device_kv_get_counters(graph->dataplane, counters) : -1;
}

extern "C" const char *cf_llama_device_graph_last_error(const cf_llama_device_graph *graph) {
    return graph ? graph->error.c_str() : "null llama device graph";
}

// ---- llama-server CUDA resolver bridge: a server slot is a sequence of the resolver ------------------------------------
struct cf_llama_server_cuda_bridge {
    cf_ms_cuda_resolver *resolver = nullptr;
    std::string error;
    // unlike the other bridges this one keeps the last failure's text across later successes
    // (llama_server_cuda_resolver_bridge.cpp:25-58)
    int pass(int rc) {
        if (rc != 0) error = cf_ms_cuda_last_error(resolver);
        return rc;
    }
};

extern "C" cf_llama_server_cuda_bridge *cf_llama_server_cuda_bridge_create(const cf_ms_cuda_config *config) {
    cf_llama_server_cuda_bridge *bridge = new (std::nothrow) cf_llama_server_cuda_bridge();
    if (!bridge) return nullptr;
    bridge->resolver = cf_ms_cuda_create(config);
    if (!bridge->resolver) {
        delete bridge;
        return nullptr;
    }
    return bridge;
}

extern "C" void cf_llama_server_cuda_bridge_destroy(cf_llama_server_cuda_bridge *bridge, void *stream) {
    if (!bridge) return;
    cf_ms_cuda_destroy(bridge->resolver, stream);
    delete bridge;
}

extern "C" int cf_llama_server_cuda_slot_create(cf_llama_server_cuda_bridge *bridge, int64_t slot_id) {
    return bridge ? bridge->pass(cf_ms_cuda_sequence_create(bridge->resolver, slot_id)) : -1;
}

extern "C" int cf_llama_server_cuda_slot_copy_async(cf_llama_server_cuda_bridge *bridge, int64_t source_slot, int64_t destination_slot,
                                                    void *stream) {
    return bridge ? bridge->pass(cf_ms_cuda_copy_sequence_async(bridge->resolver, source_slot, destination_slot, stream)) : -1;
}

extern "C" int cf_llama_server_cuda_slot_cancel_async(cf_llama_server_cuda_bridge *bridge, int64_t slot_id, void *stream) {
    return bridge ? bridge->pass(cf_ms_cuda_cancel_sequence_async(bridge->resolver, slot_id, stream)) : -1;
}

extern "C" int cf_llama_server_cuda_slot_reset_async(cf_llama_server_cuda_bridge *bridge, int64_t slot_id, void *stream) {
    return bridge ? bridge->pass(cf_ms_cuda_sequence_remove_async(bridge->resolver, slot_id, stream)) : -1;
}

extern "C" int cf_llama_server_cuda_dispatch_batch_async(cf_llama_server_cuda_bridge *bridge, const cf_ms_batch_item *items,
                                                         uint32_t item_count, void *stream) {
    return bridge ? bridge->pass(cf_ms_cuda_execute_batch_async(bridge->resolver, items, item_count, stream)) : -1;
}

extern "C" int cf_llama_server_cuda_shutdown_audit(cf_llama_server_cuda_bridge *bridge) {
    if (!bridge) return -1;
    const int rc = cf_ms_cuda_audit(bridge->resolver);
    if (rc != 0) bridge->error = "CUDA multi-sequence shutdown audit failed";
    return rc;
}

extern "C" const char *cf_llama_server_cuda_last_error(const cf_llama_server_cuda_bridge *bridge) {
    return bridge ? bridge->error.c_str() : "null llama-server CUDA bridge";
}
