/* compat_mscache.h — the reference's multi-sequence cache ABI and its llama-server runtime ABI, same symbols and
 * struct layouts:
 *   include/chromofold/multisequence_cache.h:11-112     cf_multisequence_*, cf_sequence_*
 *   include/chromofold/llama_server_runtime.h:14-86      cf_llama_server_*
 * In the reference the cache is host bookkeeping only: cf_sequence_append_async counts tokens without storing a row
 * and cf_multisequence_attention_async always fails ("resolver is not connected yet; dense fallback is forbidden",
 * src/multisequence_cache.cpp:438-462). Here the same calls carry data: the cache owns a device sequence store
 * (compat_ms.h); an append writes the strided rows to the layer's active tail on the GPU and seals the tail into a
 * format-v1 page the moment it holds page_size tokens; attention runs the batched sealed-page kernels.
 * Kept from the reference: thread-safe handle, int 0 / -1 with last_error, ids may be any int64, duplicate ids are
 * refused, appends must be contiguous and never cross a page boundary, pages are immutable (a removal that cuts a
 * sealed page is refused and counted in unsupported_operations), speculation = begin / commit(accepted) / rollback over
 * the active tail (no page is sealed while a speculation is open), reclaim / audit / counters.
 * Copy (src/multisequence_cache.cpp:235-292): any range; the destination gets the sealed pages that lie wholly inside
 * it, shared by reference, and the active tail if it lies wholly inside; a range that starts after token 0 gives a
 * sequence whose first held token keeps its old position. Shift (:357-380): a range that cuts a sealed page is an
 * error; a range that covers the whole sequence moves it (positions are not stored in sealed pages, so only the
 * sequence's offset changes); a range that covers nothing, or a delta of 0, does nothing; an active tail that the
 * range cuts stays where it is without an error, as in the reference. A sequence that holds nothing takes the position
 * of the first rows appended to it (:423). A removal range that covers nothing cached succeeds, and every successful
 * range removal counts in sequences_removed (:345). A commit is refused when the tail has become shorter than it was
 * at speculation_begin (:497). The calls that can be compared with the reference's own cache (no sealed pages: its
 * cache never seals) return the same status for the same sequence of operations; tests/test_gpu_random_cases.py
 * runs both side by side.
 * Narrower than the reference: a non-zero shift of only part of a sequence (which would leave a gap inside it) and the
 * removal of a range that is not a suffix are refused and counted in unsupported_operations; the layers of one
 * sequence start at the same position; a rollback never lengthens a tail (the reference sets every layer to the
 * baseline count even when rows were removed in between). */
#ifndef CHROMOFOLD_B200_COMPAT_MSCACHE_H
#define CHROMOFOLD_B200_COMPAT_MSCACHE_H

#include <stdint.h>

#include "chromofold_b200/compat_ms.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CHROMOFOLD_MULTISEQUENCE_CACHE_H
typedef struct cf_multisequence_cache cf_multisequence_cache;
typedef uint64_t cf_speculation_id;

typedef struct cf_multisequence_config { /* multisequence_cache.h:14-23 */
    uint32_t layer_count, kv_head_count, query_head_count, head_dim, page_size, gqa_group_size;
    uint32_t use_async_allocator, enable_invariant_auditor;
} cf_multisequence_config;

typedef struct cf_multisequence_counters { /* :25-49 */
    uint64_t sequences_created, sequences_copied, sequences_removed, sequences_shifted, active_sequences;
    uint64_t active_sequences_peak, shared_pages, shared_page_references, page_ref_increments, page_ref_decrements;
    uint64_t pages_reclaimed, pages_pending_reclamation, pending_reclamation_bytes, pending_reclamation_bytes_peak;
    uint64_t speculative_transactions_started, speculative_transactions_committed, speculative_transactions_rolled_back;
    uint64_t batches_dispatched, sequences_per_batch_peak, invariant_audits, invariant_failures, unsupported_operations;
    uint64_t dense_fallback_launches;
} cf_multisequence_counters;

typedef struct cf_sequence_attention_item { /* :51-63; the layout of cf_ms_batch_item */
    int64_t sequence_id;
    uint32_t layer;
    cf_device_tensor_view query;
    void *output;
    uint32_t output_type;
    uint64_t output_token_stride_bytes, output_head_stride_bytes, output_element_stride_bytes;
    uint32_t query_token_begin;
    float softmax_scale;
    uint32_t causal_window;
} cf_sequence_attention_item;
#endif

cf_multisequence_cache *cf_multisequence_create(const cf_multisequence_config *config);                      /* :65 */
void cf_multisequence_destroy(cf_multisequence_cache *cache, void *stream);                                   /* :66 */
int cf_sequence_create(cf_multisequence_cache *cache, int64_t sequence_id);                                  /* :68 */
int cf_sequence_copy_async(cf_multisequence_cache *cache, int64_t source_sequence, int64_t destination_sequence,
                           uint32_t token_begin, uint32_t token_end, void *stream);                           /* :69-74 */
int cf_sequence_remove_async(cf_multisequence_cache *cache, int64_t sequence_id, int64_t position_begin,
                             int64_t position_end, void *stream);                                             /* :75-79 */
int cf_sequence_shift_async(cf_multisequence_cache *cache, int64_t sequence_id, uint32_t position_begin,
                            uint32_t position_end, int32_t delta, void *stream);                              /* :80-85 */
int cf_sequence_append_async(cf_multisequence_cache *cache, int64_t sequence_id, uint32_t layer, uint32_t token_begin,
                             const cf_device_tensor_view *keys, const cf_device_tensor_view *values, void *stream); /* :86-92 */
int cf_multisequence_attention_async(cf_multisequence_cache *cache, const cf_sequence_attention_item *items,
                                     uint32_t item_count, void *stream);                                      /* :93-96 */
cf_speculation_id cf_sequence_speculation_begin(cf_multisequence_cache *cache, int64_t sequence_id);        /* :98 */
int cf_sequence_speculation_commit(cf_multisequence_cache *cache, int64_t sequence_id, cf_speculation_id speculation_id,
                                   uint32_t accepted_tokens, void *stream);                                   /* :99-103 */
int cf_sequence_speculation_rollback(cf_multisequence_cache *cache, int64_t sequence_id, cf_speculation_id speculation_id,
                                     void *stream);                                                           /* :104-107 */
int cf_multisequence_reclaim_async(cf_multisequence_cache *cache, void *stream);                             /* :109 */
int cf_multisequence_audit(const cf_multisequence_cache *cache);                                             /* :110 */
int cf_multisequence_get_counters(const cf_multisequence_cache *cache, cf_multisequence_counters *counters); /* :111 */
const char *cf_multisequence_last_error(const cf_multisequence_cache *cache);                                /* :112 */

/* ---- include/chromofold/llama_server_runtime.h ---------------------------------------------------------- */
typedef struct cf_llama_server_runtime cf_llama_server_runtime;

/* The reference's header uses `#pragma once`, so there is no guard macro to test for it: a translation unit that has
 * already included it defines CHROMOFOLD_LLAMA_SERVER_RUNTIME_TYPES before this header. */
#ifndef CHROMOFOLD_LLAMA_SERVER_RUNTIME_TYPES
typedef struct cf_llama_server_config { /* :16-30 */
    uint32_t layer_count, query_head_count, kv_head_count, head_dim, page_size, block_size, context_window;
    uint32_t gqa_group_size, cuda_device, strict_mode;
    const char *evidence_path;
    const char *llama_commit;   /* required */
    const char *model_sha256;   /* required */
} cf_llama_server_config;

typedef struct cf_llama_server_batch_token { /* :32-37 */
    int64_t sequence_id;
    uint32_t batch_index, absolute_position, token_count;
} cf_llama_server_batch_token;

typedef struct cf_llama_server_batch { /* :39-44 */
    const cf_llama_server_batch_token *tokens;
    uint32_t token_item_count;
    const cf_sequence_attention_item *attention_items;
    uint32_t attention_item_count;
} cf_llama_server_batch;

typedef struct cf_llama_server_stats { /* :46-56 */
    uint64_t http_requests, interleaved_batches, slot_reuses, cancelled_requests, context_shifts, speculative_rollbacks;
    uint64_t dense_nodes_scheduled, shutdown_audits, shutdown_failures;
} cf_llama_server_stats;
#endif

cf_llama_server_runtime *cf_llama_server_runtime_create(const cf_llama_server_config *config);              /* :58 */
void cf_llama_server_runtime_destroy(cf_llama_server_runtime *runtime, void *stream);                        /* :59 */
int cf_llama_server_slot_create(cf_llama_server_runtime *runtime, int64_t sequence_id);                      /* :61 */
int cf_llama_server_slot_reset_async(cf_llama_server_runtime *runtime, int64_t sequence_id, void *stream);   /* :62 */
int cf_llama_server_cancel_async(cf_llama_server_runtime *runtime, int64_t sequence_id, void *stream);       /* :63 */
int cf_llama_server_sequence_copy_async(cf_llama_server_runtime *runtime, int64_t source, int64_t destination,
                                        uint32_t token_begin, uint32_t token_end, void *stream);              /* :64-65 */
int cf_llama_server_sequence_remove_async(cf_llama_server_runtime *runtime, int64_t sequence_id, int64_t position_begin,
                                          int64_t position_end, void *stream);                                /* :66-67 */
int cf_llama_server_sequence_shift_async(cf_llama_server_runtime *runtime, int64_t sequence_id, uint32_t position_begin,
                                         uint32_t position_end, int32_t delta, void *stream);                 /* :68-69 */
/* key / value: DEVICE fp32 rows [token_count][kv_head_count][head_dim] (:71-78). Rows are appended to the layer's
 * history; a full page is sealed on the GPU at once. */
int cf_llama_server_append_layer_async(cf_llama_server_runtime *runtime, int64_t sequence_id, uint32_t layer_index,
                                       uint32_t token_begin, const float *key, const float *value, uint32_t token_count,
                                       void *stream);
int cf_llama_server_execute_batch_async(cf_llama_server_runtime *runtime, const cf_llama_server_batch *batch, void *stream); /* :80-82 */
int cf_llama_server_shutdown_async(cf_llama_server_runtime *runtime, void *stream);                          /* :84 */
int cf_llama_server_get_stats(const cf_llama_server_runtime *runtime, cf_llama_server_stats *out);           /* :85 */
const char *cf_llama_server_last_error(const cf_llama_server_runtime *runtime);                              /* :86 */

#ifdef __cplusplus
}
#endif

#endif
