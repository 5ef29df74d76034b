/* compat_bridges.h — the reference's llama.cpp-side bridges over its runtime ABIs, same symbols and struct layouts.
 * None of them needs llama.cpp or ggml sources: they are what the patched llama.cpp links and calls.
 *   integrations/llama.cpp/chromofold_runtime_bridge.h:13-79        cf_llama_runtime_*        (over cf_llama_kv_*)
 *   integrations/llama.cpp/graph/chromofold_graph_contract.h:14-65  cf_llama_graph_*, cf_llama_model_topology_validate
 *   integrations/llama.cpp/chromofold_device_seal_bridge.h:11-46    cf_llama_device_seal_bridge_* (over cf_device_seal_*)
 *   integrations/llama.cpp/device_kv_graph_bridge.h:10-39           cf_llama_device_graph_*   (over cf_device_kv_*)
 *   integrations/llama.cpp/multisequence/llama_server_cuda_resolver_bridge.h:10-20  cf_llama_server_cuda_* (over cf_ms_cuda_*)
 * Kept from the reference: int 0 / -1 with a last_error string owned by the handle; NULL handle -> -1 (last_error of
 * a NULL handle is a fixed string); struct_size checked on every options struct; a ChromoFold backend must be created
 * with require_cuda = 1 and allow_dense_fallback = 0 (chromofold_runtime_bridge.cpp:44-50,
 * chromofold_device_seal_bridge.cpp:12-13); the device graph needs causal, linear_sequence_only and
 * dense_fallback_forbidden all set (device_kv_graph_bridge.cpp:13-15); the graph contract accepts page sizes 64, 128,
 * 256 and head_dim <= 128, uniform causal non-recurrent models only (chromofold_graph_contract.cpp:34-50); a dense
 * dispatch under the ChromoFold backend is counted and refused; every refused operation is counted
 * (rejected_operations / unsupported_graphs); "evidence complete" means compressed launches that consumed sealed
 * values with no dense fallback and no CUDA error (chromofold_runtime_bridge.cpp:139-144,
 * chromofold_device_seal_bridge.cpp:62-68). cf_llama_runtime_append takes contiguous fp32 [token][head][dim] views
 * in host memory, as the reference's does. The JSON written by cf_llama_runtime_write_json has the reference's keys.
 * The llama-server multi-sequence bridge (llama_server_multisequence_bridge.h) re-uses four symbol names of
 * llama_server_runtime.h with other signatures, so it lives in a library of its own: compat_llama_ms_bridge.h. */
#ifndef CHROMOFOLD_B200_COMPAT_BRIDGES_H
#define CHROMOFOLD_B200_COMPAT_BRIDGES_H

#include <stddef.h>
#include <stdint.h>

#include "chromofold_b200/compat_adapter.h"
#include "chromofold_b200/compat_device.h"
#include "chromofold_b200/compat_ms.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- runtime bridge (chromofold_runtime_bridge.h) ---- */
#ifndef CHROMOFOLD_LLAMA_RUNTIME_BRIDGE_H
typedef enum cf_llama_scalar_type { CF_LLAMA_SCALAR_F32 = 0, CF_LLAMA_SCALAR_F16 = 1 } cf_llama_scalar_type; /* :13-16 */

typedef struct cf_llama_tensor_view { /* :18-27 */
    const void *data;
    uint64_t token_stride_bytes, head_stride_bytes, element_stride_bytes;
    uint32_t token_count, head_count, head_dim;
    cf_llama_scalar_type scalar_type;
} cf_llama_tensor_view;

typedef struct cf_llama_runtime_options { /* :29-36 */
    uint32_t struct_size;
    cf_llama_kv_options kv;
    uint32_t causal_window, require_cuda, allow_dense_fallback, emit_stats;
} cf_llama_runtime_options;

typedef struct cf_llama_runtime_counters { /* :38-47 */
    uint64_t append_calls, appended_values, compressed_attention_launches, sealed_values_consumed;
    uint64_t active_values_consumed, dense_fallback_launches, rejected_operations, cuda_errors;
} cf_llama_runtime_counters;

typedef struct cf_llama_runtime_snapshot { /* :49-56 */
    cf_llama_kv_stats kv;
    cf_llama_runtime_counters counters;
    uint32_t backend_selected, initialized, dense_fallback_allowed, evidence_complete;
} cf_llama_runtime_snapshot;

typedef struct cf_llama_runtime cf_llama_runtime;
#endif

int cf_llama_runtime_options_validate(const cf_llama_runtime_options *options);                       /* :60 */
cf_llama_runtime *cf_llama_runtime_create(const cf_llama_runtime_options *options);                   /* :61 */
void cf_llama_runtime_destroy(cf_llama_runtime *runtime);                                             /* :62 */
int cf_llama_runtime_append(cf_llama_runtime *runtime, uint32_t layer, uint32_t token_begin, const cf_llama_tensor_view *keys,
                            const cf_llama_tensor_view *values, void *stream);                       /* :64-69 */
int cf_llama_runtime_record_compressed_launch(cf_llama_runtime *runtime, uint64_t sealed_values, uint64_t active_values); /* :71-73 */
int cf_llama_runtime_record_dense_fallback(cf_llama_runtime *runtime);                                /* :74 */
int cf_llama_runtime_record_cuda_error(cf_llama_runtime *runtime);                                    /* :75 */
int cf_llama_runtime_snapshot_get(const cf_llama_runtime *runtime, cf_llama_runtime_snapshot *snapshot); /* :76-77 */
int cf_llama_runtime_write_json(const cf_llama_runtime *runtime, const char *path);                   /* :78 */
const char *cf_llama_runtime_last_error(const cf_llama_runtime *runtime);                             /* :79 */

/* ---- graph contract (graph/chromofold_graph_contract.h) ---- */
#ifndef CHROMOFOLD_LLAMA_GRAPH_CONTRACT_H
typedef struct cf_llama_model_topology { /* :14-24 */
    uint32_t struct_size, layer_count, query_head_count, kv_head_count, head_dim, context_size;
    uint32_t uniform_kv_geometry, causal, recurrent;
} cf_llama_model_topology;

typedef struct cf_llama_graph_options { /* :26-33 */
    uint32_t struct_size;
    cf_llama_kv_backend backend;
    uint32_t page_size, window, emit_stats;
    const char *evidence_path;
} cf_llama_graph_options;

typedef struct cf_llama_graph_counters { /* :35-42 */
    uint64_t graph_append_calls, graph_attention_dispatches, graph_dense_dispatches;
    uint64_t query_layout_conversions, output_layout_conversions, unsupported_graphs;
} cf_llama_graph_counters;

typedef struct cf_llama_graph_state cf_llama_graph_state;
#endif

int cf_llama_graph_options_validate(const cf_llama_graph_options *options);                           /* :46 */
int cf_llama_model_topology_validate(const cf_llama_model_topology *topology);                        /* :47 */
cf_llama_graph_state *cf_llama_graph_create(const cf_llama_graph_options *options, const cf_llama_model_topology *topology); /* :48-49 */
void cf_llama_graph_destroy(cf_llama_graph_state *state);                                             /* :50 */
int cf_llama_graph_append_device(cf_llama_graph_state *state, uint32_t layer, uint32_t token_begin, const cf_llama_tensor_view *keys,
                                 const cf_llama_tensor_view *values, void *stream);                  /* :51-56 */
int cf_llama_graph_record_attention(cf_llama_graph_state *state, uint64_t sealed_values, uint64_t active_values); /* :57-59 */
int cf_llama_graph_record_dense_dispatch(cf_llama_graph_state *state);                                /* :60 */
int cf_llama_graph_get_counters(const cf_llama_graph_state *state, cf_llama_graph_counters *counters); /* :61-62 */
int cf_llama_graph_write_evidence(const cf_llama_graph_state *state);                                 /* :63 */
const char *cf_llama_graph_last_error(const cf_llama_graph_state *state);                             /* :64 */

/* ---- device seal bridge (chromofold_device_seal_bridge.h) ---- */
#ifndef CHROMOFOLD_LLAMA_DEVICE_SEAL_BRIDGE_H
typedef struct cf_llama_device_seal_bridge cf_llama_device_seal_bridge;

typedef struct cf_llama_device_seal_options { /* :13-18 */
    uint32_t struct_size;
    cf_device_seal_config seal;
    uint32_t require_cuda, allow_dense_fallback;
} cf_llama_device_seal_options;
#endif

cf_llama_device_seal_bridge *cf_llama_device_seal_bridge_create(const cf_llama_device_seal_options *options); /* :20 */
void cf_llama_device_seal_bridge_destroy(cf_llama_device_seal_bridge *bridge, void *stream);          /* :21 */
int cf_llama_device_seal_bridge_stage(cf_llama_device_seal_bridge *bridge, uint32_t layer, uint32_t token_begin,
                                      const float *active_k, const float *active_v, uint32_t token_count, void *stream); /* :22-28 */
int cf_llama_device_seal_bridge_seal(cf_llama_device_seal_bridge *bridge, uint32_t layer, void *stream); /* :29 */
int cf_llama_device_seal_bridge_attention(cf_llama_device_seal_bridge *bridge, uint32_t layer, const cf_device_tensor_view *query,
                                          void *output, uint32_t output_scalar_type, uint64_t output_token_stride_bytes,
                                          uint64_t output_head_stride_bytes, uint64_t output_element_stride_bytes,
                                          uint32_t query_token_begin, float softmax_scale, uint32_t causal_window,
                                          void *stream);                                             /* :30-41 */
int cf_llama_device_seal_bridge_evidence(const cf_llama_device_seal_bridge *bridge, cf_device_seal_counters *counters,
                                         uint32_t *complete);                                        /* :42-44 */
const char *cf_llama_device_seal_bridge_last_error(const cf_llama_device_seal_bridge *bridge);        /* :45 */

/* ---- device KV graph bridge (device_kv_graph_bridge.h) ---- */
#ifndef CHROMOFOLD_LLAMA_DEVICE_KV_GRAPH_BRIDGE_H
typedef struct cf_llama_device_graph cf_llama_device_graph;

typedef struct cf_llama_device_graph_options { /* :12-18 */
    uint32_t struct_size;
    cf_device_kv_config kv;
    uint32_t causal, linear_sequence_only, dense_fallback_forbidden;
} cf_llama_device_graph_options;
#endif

cf_llama_device_graph *cf_llama_device_graph_create(const cf_llama_device_graph_options *options);   /* :20 */
void cf_llama_device_graph_destroy(cf_llama_device_graph *graph, void *stream);                       /* :21 */
int cf_llama_device_graph_append_async(cf_llama_device_graph *graph, uint32_t layer, uint32_t token_begin,
                                       const cf_device_tensor_view *keys, const cf_device_tensor_view *values, void *stream); /* :22-27 */
int cf_llama_device_graph_attention_async(cf_llama_device_graph *graph, uint32_t layer, const float *query, float *output,
                                          uint32_t query_token_count, uint32_t query_token_begin, float softmax_scale,
                                          uint32_t causal_window, void *stream);                     /* :28-36 */
int cf_llama_device_graph_get_counters(const cf_llama_device_graph *graph, cf_device_kv_counters *counters); /* :37 */
const char *cf_llama_device_graph_last_error(const cf_llama_device_graph *graph);                     /* :38 */

/* ---- llama-server CUDA resolver bridge (multisequence/llama_server_cuda_resolver_bridge.h) ---- */
#ifndef CHROMOFOLD_LLAMA_SERVER_CUDA_RESOLVER_BRIDGE_H
typedef struct cf_llama_server_cuda_bridge cf_llama_server_cuda_bridge;
#endif

cf_llama_server_cuda_bridge *cf_llama_server_cuda_bridge_create(const cf_ms_cuda_config *config);    /* :12 */
void cf_llama_server_cuda_bridge_destroy(cf_llama_server_cuda_bridge *bridge, void *stream);          /* :13 */
int cf_llama_server_cuda_slot_create(cf_llama_server_cuda_bridge *bridge, int64_t slot_id);           /* :14 */
int cf_llama_server_cuda_slot_copy_async(cf_llama_server_cuda_bridge *bridge, int64_t source_slot, int64_t destination_slot,
                                         void *stream);                                              /* :15 */
int cf_llama_server_cuda_slot_cancel_async(cf_llama_server_cuda_bridge *bridge, int64_t slot_id, void *stream); /* :16 */
int cf_llama_server_cuda_slot_reset_async(cf_llama_server_cuda_bridge *bridge, int64_t slot_id, void *stream);  /* :17 */
int cf_llama_server_cuda_dispatch_batch_async(cf_llama_server_cuda_bridge *bridge, const cf_ms_batch_item *items,
                                              uint32_t item_count, void *stream);                    /* :18 */
int cf_llama_server_cuda_shutdown_audit(cf_llama_server_cuda_bridge *bridge);                         /* :19 */
const char *cf_llama_server_cuda_last_error(const cf_llama_server_cuda_bridge *bridge);               /* :20 */

#ifdef __cplusplus
}
#endif

#endif
