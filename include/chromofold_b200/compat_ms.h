/* compat_ms.h — the reference's device sequence resolver ABI (include/chromofold/multisequence_cuda_resolver.h:11-93),
 * same symbols and struct layouts, served by this library's multi-sequence page store.
 *
 * Kept: thread-safe handle (one mutex), sequences by id, shared pages with logical and in-flight reference counts,
 * whole-batch validation and snapshotting before the first launch, snapshot release on a CUDA event, deferred
 * reclamation, copy-on-write tails, cancel / remove / audit, the counter block, int 0 / -1 + last_error.
 * Different:
 *   - a batch is served by ONE attention launch per layer present in the batch (the reference launches one
 *     single-thread-per-head kernel per item, src/cuda/multisequence_cuda_resolver.cu:391-402);
 *   - cf_ms_cuda_publish_page_async takes the reference's int4 page descriptor (offset-binary nibbles, one fp32 scale
 *     per flat block, src/cuda/device_kv_seal_attention.cu:80-134) and TRANSCODES it on the GPU into format-v1
 *     records (int8 + entropy coded, one fp16 scale per stream); the int8 step is 1/16 of the int4 step or finer, so
 *     values move by at most 3.2 % of an int4 step;
 *   - a page must continue its sequence's sealed history (token_begin == tokens already published for that layer) and
 *     only the last published page of a layer may be shorter than page_size; cf_ms_cuda_shift_sequence accepts only
 *     shifts that move nothing (the reference itself refuses shifts that cut a page, :431-443). */
#ifndef CHROMOFOLD_B200_COMPAT_MS_H
#define CHROMOFOLD_B200_COMPAT_MS_H

#include <stdint.h>

#include "chromofold_b200/compat_device.h"

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CHROMOFOLD_MULTISEQUENCE_CUDA_RESOLVER_H
typedef struct cf_ms_cuda_config { /* :11-19 */
    uint32_t layer_count, kv_head_count, query_head_count, head_dim, page_size, gqa_group_size, use_async_allocator;
} cf_ms_cuda_config;

typedef struct cf_ms_page_publication { /* :21-27 */
    int64_t sequence_id;
    uint32_t layer;
    cf_device_page_descriptor descriptor;
    uint64_t resident_bytes;
    uint64_t seal_generation;
} cf_ms_page_publication;

typedef struct cf_ms_batch_item { /* :29-41 */
    int64_t sequence_id;
    uint32_t layer;
    cf_device_tensor_view query;
    void *output;
    uint32_t output_type;
    uint64_t output_token_stride_bytes, output_head_stride_bytes, output_element_stride_bytes;
    uint32_t query_token_begin;
    float softmax_scale;
    uint32_t causal_window;
} cf_ms_batch_item;

typedef struct cf_ms_cuda_counters { /* :43-68 */
    uint64_t pages_registered, page_registration_failures, descriptor_tables_built, descriptor_table_rebuilds;
    uint64_t snapshots_acquired, snapshots_released, in_flight_page_references, snapshot_release_events;
    uint64_t stale_snapshot_rejections, server_batches_received, compressed_batches_executed, sequence_attention_launches;
    uint64_t prefill_items, decode_items, tokens_per_batch_peak, copy_on_write_tail_copies, cancellation_requests;
    uint64_t pages_retired, pages_reclaimed, pending_reclamation_bytes, pending_reclamation_bytes_peak;
    uint64_t cross_sequence_contamination, dense_fallback_launches, cuda_errors;
} cf_ms_cuda_counters;

typedef struct cf_ms_cuda_resolver cf_ms_cuda_resolver;
#endif

cf_ms_cuda_resolver *cf_ms_cuda_create(const cf_ms_cuda_config *config);                                   /* :73 */
void cf_ms_cuda_destroy(cf_ms_cuda_resolver *resolver, void *stream);                                       /* :74 */
int cf_ms_cuda_sequence_create(cf_ms_cuda_resolver *resolver, int64_t sequence_id);                         /* :75 */
int cf_ms_cuda_sequence_remove_async(cf_ms_cuda_resolver *resolver, int64_t sequence_id, void *stream);     /* :76 */
int cf_ms_cuda_publish_page_async(cf_ms_cuda_resolver *resolver, const cf_ms_page_publication *publication, void *stream); /* :77 */
int cf_ms_cuda_stage_active_async(cf_ms_cuda_resolver *resolver, int64_t sequence_id, uint32_t layer, uint32_t token_begin,
                                  const float *keys, const float *values, uint32_t token_count, void *stream); /* :78-80 */
int cf_ms_cuda_copy_sequence_async(cf_ms_cuda_resolver *resolver, int64_t source_sequence, int64_t destination_sequence,
                                   void *stream);                                                           /* :81-82 */
int cf_ms_cuda_shift_sequence(cf_ms_cuda_resolver *resolver, int64_t sequence_id, uint32_t position_begin,
                              uint32_t position_end, int32_t delta);                                        /* :83-84 */
int cf_ms_cuda_execute_batch_async(cf_ms_cuda_resolver *resolver, const cf_ms_batch_item *items, uint32_t item_count,
                                   void *stream);                                                           /* :85-88 */
int cf_ms_cuda_cancel_sequence_async(cf_ms_cuda_resolver *resolver, int64_t sequence_id, void *stream);     /* :89 */
int cf_ms_cuda_reclaim_async(cf_ms_cuda_resolver *resolver, void *stream);                                  /* :90 */
int cf_ms_cuda_audit(const cf_ms_cuda_resolver *resolver);                                                  /* :91 */
int cf_ms_cuda_get_counters(const cf_ms_cuda_resolver *resolver, cf_ms_cuda_counters *counters);            /* :92 */
const char *cf_ms_cuda_last_error(const cf_ms_cuda_resolver *resolver);                                     /* :93 */

/* ---- additive, beside the reference's symbols: the append / seal / truncate seam of a data-bearing sequence cache.
 * In the reference a page reaches the resolver as an int4 descriptor made elsewhere (the seal engine) and rows reach
 * it only as a whole staged tail; here rows are appended to the active tail as strided typed views (the rules of
 * cf_device_kv_append_async: contiguous, never across a page boundary) and the tail is sealed in one launch into
 * format-v1 records and published in the same call. */
int cf_b200_ms_append_active_async(cf_ms_cuda_resolver *resolver, int64_t sequence_id, uint32_t layer, uint32_t token_begin,
                                   const cf_device_tensor_view *keys, const cf_device_tensor_view *values, void *stream);
int cf_b200_ms_seal_active_async(cf_ms_cuda_resolver *resolver, int64_t sequence_id, uint32_t layer, void *stream);
/* Keep the first token_count tokens of every layer: drops later whole pages (this sequence's reference to them) and
 * shortens the active tail; a cut inside a sealed page is refused. */
int cf_b200_ms_truncate_async(cf_ms_cuda_resolver *resolver, int64_t sequence_id, uint32_t token_count, void *stream);
/* Forget the first token_count tokens of every layer (whole sealed pages only): later pages move to the front of the
 * sequence's page-table row and its token 0 becomes what was token token_count. */
int cf_b200_ms_drop_prefix_async(cf_ms_cuda_resolver *resolver, int64_t sequence_id, uint32_t token_count, void *stream);
int cf_b200_ms_sequence_tokens(const cf_ms_cuda_resolver *resolver, int64_t sequence_id, uint32_t layer,
                               uint32_t *sealed_tokens, uint32_t *active_tokens);
/* Pages referenced by two or more sequences, the references they hold, and the references taken / dropped so far. */
int cf_b200_ms_page_sharing(const cf_ms_cuda_resolver *resolver, uint64_t *shared_pages, uint64_t *shared_references,
                            uint64_t *reference_increments, uint64_t *reference_decrements);

/* Arena bookkeeping: room is handed out in page slots (one page's records at their largest size), a reclaimed page's
 * slot is reused by the next page sealed, so the arena stops growing once the number of live pages does.
 * device_status_seen: CF_B200_DEVSTAT_* bits the resolver has read back at its synchronisation points (every seal). */
int cf_b200_ms_arena_stats(const cf_ms_cuda_resolver *resolver, uint64_t *slots_in_use, uint64_t *slots_free,
                           uint64_t *live_record_bytes, uint64_t *arena_bytes, uint32_t *device_status_seen);

#ifdef __cplusplus
}
#endif

#endif
