/* compat_production.h — the reference's batched decode runtime ABI, same symbols and struct layouts:
 *   include/chromofold/production_attention.h:11-104   cf_attention_runtime_*, cf_attention_execute_async, ...
 * A batch item names one (sequence, layer): a strided query view, a strided output, the layer's sealed pages as
 * cf_device_page_descriptor[] in device memory (int4 nibbles, one fp32 scale per block_size values, flat index
 * (token * kv_heads + head) * head_dim + d) and its unsealed fp32 tail [token][kv_head][head_dim].
 * Kept from the reference: opaque handle guarded by a mutex, int 0 / -1 returns with a last_error string owned by the
 * handle, create rejects query_heads != kv_heads * gqa_group_size, the counter set, one launch for the whole batch.
 * Different, on purpose:
 *   - nibbles are read as offset-binary (value = nibble - 8), which is what the reference's seal engine writes
 *     (src/cuda/device_kv_seal_attention.cu:102,118); the reference's own batch kernel reads them as two's
 *     complement (src/cuda/production_attention.cu:39-44) and so disagrees with the pages it is given (given the same
 *     values re-encoded as two's-complement nibbles, its kernel and this library agree to 2e-5:
 *     tests/test_gpu_random_cases.py runs the two side by side);
 *   - visibility is the rule of the rest of the path, first <= token <= query position with
 *     first = max(0, position + 1 - window) (src/runtime/kv_reference.cpp:205-207), not
 *     `token + window < query_token_begin` (production_attention.cu:84);
 *   - one block per (item, kv head, query token): a nibble is decoded once for the whole query group;
 *   - the item array goes through a pinned staging ring and a pooled device buffer (no allocation per call);
 *   - CF_ATTENTION_REFERENCE mode runs a plain one-thread-per-output kernel instead of failing, and
 *     cf_attention_compare_async runs both kernels and compares them (the reference ships it as a stub that fails,
 *     production_attention.cu:213-223). It waits for the stream: its result is the comparison. */
#ifndef CHROMOFOLD_B200_COMPAT_PRODUCTION_H
#define CHROMOFOLD_B200_COMPAT_PRODUCTION_H

#include <stdint.h>

#include "chromofold_b200/compat_device.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The reference's header uses `#pragma once`: a translation unit that has already included it defines
 * CHROMOFOLD_PRODUCTION_ATTENTION_TYPES before this header. */
#ifndef CHROMOFOLD_PRODUCTION_ATTENTION_TYPES
typedef enum cf_attention_kernel_mode { CF_ATTENTION_REFERENCE = 0, CF_ATTENTION_OPTIMIZED = 1 } cf_attention_kernel_mode;

typedef struct cf_attention_tuning { /* production_attention.h:16-24; accepted, not needed by this implementation */
    uint32_t threads_per_block, warps_per_block, heads_per_block, pages_per_work_unit, vector_width;
    uint32_t enable_cuda_graphs, enable_async_sealing;
} cf_attention_tuning;

typedef struct cf_attention_runtime_config { /* :26-38 */
    uint32_t layer_count, query_head_count, kv_head_count, head_dim, page_size, block_size, gqa_group_size;
    uint32_t cuda_device, use_async_allocator;
    cf_attention_kernel_mode mode;
    cf_attention_tuning tuning;
} cf_attention_runtime_config;

typedef struct cf_attention_batch_item { /* :40-58, 168 bytes */
    int64_t sequence_id;
    uint32_t layer;
    cf_device_tensor_view query;
    void *output;
    uint32_t output_type;
    uint64_t output_token_stride_bytes, output_head_stride_bytes, output_element_stride_bytes;
    uint32_t query_token_begin;
    float softmax_scale;
    uint32_t causal_window;
    const cf_device_page_descriptor *sealed_pages;
    uint32_t sealed_page_count;
    const float *active_keys;
    const float *active_values;
    uint32_t active_token_begin, active_token_count;
} cf_attention_batch_item;

typedef struct cf_attention_counters { /* :60-86 */
    uint64_t reference_launches, optimized_launches, decode_launches, prefill_launches, grouped_batches, grouped_items;
    uint64_t kernel_launches_avoided, graph_captures, graph_replays, graph_invalidations, graph_replay_failures;
    uint64_t async_seal_submissions, async_seal_overlaps, descriptor_bytes_read, compressed_payload_bytes_read;
    uint64_t scale_bytes_read, allocation_count, pool_hits, pool_misses, peak_reserved_bytes, peak_live_bytes;
    uint64_t numerical_failures, cross_sequence_contamination, dense_fallback_launches, cuda_errors;
} cf_attention_counters;
#endif

typedef struct cf_attention_runtime cf_attention_runtime;

cf_attention_runtime *cf_attention_runtime_create(const cf_attention_runtime_config *config);    /* :90 */
void cf_attention_runtime_destroy(cf_attention_runtime *runtime, void *stream);                   /* :91 */
int cf_attention_execute_async(cf_attention_runtime *runtime, const cf_attention_batch_item *items, uint32_t item_count,
                               void *stream);                                                     /* :92-95 */
int cf_attention_compare_async(cf_attention_runtime *runtime, const cf_attention_batch_item *items, uint32_t item_count,
                               float max_abs_error, float mean_abs_error, void *stream);          /* :96-101 */
int cf_attention_invalidate_graphs(cf_attention_runtime *runtime);                                /* :102 */
int cf_attention_get_counters(const cf_attention_runtime *runtime, cf_attention_counters *counters); /* :103 */
const char *cf_attention_last_error(const cf_attention_runtime *runtime);                         /* :104 */

#ifdef __cplusplus
}
#endif

#endif
