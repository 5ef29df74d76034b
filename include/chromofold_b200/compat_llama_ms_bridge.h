/* compat_llama_ms_bridge.h — the reference's llama-server multi-sequence bridge, same symbols and struct layouts:
 *   integrations/llama.cpp/multisequence/llama_server_multisequence_bridge.h:11-62   cf_llama_server_multisequence_*,
 *   cf_llama_server_slot_*, cf_llama_server_sequence_*, cf_llama_server_context_shift_async,
 *   cf_llama_server_cancel_sequence_async, cf_llama_server_batch_attention_async, cf_llama_server_audit
 * Four of its names (cf_llama_server_slot_create, _slot_reset_async, _sequence_copy_async, _sequence_remove_async) are
 * also names of include/chromofold/llama_server_runtime.h with other signatures; the reference never links the two
 * together. So this bridge is a shared library of its own, libchromofold_b200_llama_ms.so, built beside
 * libchromofold_b200.so and linked against it (it calls cf_multisequence_* / cf_sequence_* of compat_mscache.h).
 * Kept from the reference: thread-safe handle (one mutex); creation needs strict_no_fallback != 0; a slot id maps to
 * one sequence id, a second create of a live slot is refused; resetting a slot removes its sequence and reclaims
 * pages; cancelling a sequence forgets every slot that names it; copy / remove / shift / batch attention forward to
 * the cache and report its error text; int 0 / -1. */
#ifndef CHROMOFOLD_B200_COMPAT_LLAMA_MS_BRIDGE_H
#define CHROMOFOLD_B200_COMPAT_LLAMA_MS_BRIDGE_H

#include <stdint.h>

#include "chromofold_b200/compat_ms.h"

#ifdef __cplusplus
extern "C" {
#endif

/* the cache's types, as in compat_mscache.h (that header cannot be included here: it declares the clashing names) */
#if !defined(CHROMOFOLD_B200_COMPAT_MSCACHE_H) && !defined(CHROMOFOLD_MULTISEQUENCE_CACHE_H)
typedef struct cf_multisequence_cache cf_multisequence_cache;
typedef struct cf_multisequence_config { /* multisequence_cache.h:14-23 */
    uint32_t layer_count, kv_head_count, query_head_count, head_dim, page_size, gqa_group_size;
    uint32_t use_async_allocator, enable_invariant_auditor;
} cf_multisequence_config;
typedef struct cf_sequence_attention_item { /* multisequence_cache.h:51-63; the layout of cf_ms_batch_item */
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

#ifndef CHROMOFOLD_LLAMA_SERVER_MULTISEQUENCE_BRIDGE_H
typedef struct cf_llama_server_multisequence cf_llama_server_multisequence;

typedef struct cf_llama_server_multisequence_config { /* :13-18 */
    cf_multisequence_config cache;
    uint32_t strict_no_fallback, enable_prefix_sharing, enable_speculative_transactions;
} cf_llama_server_multisequence_config;

typedef struct cf_llama_server_slot_event { /* :20-25 */
    int64_t slot_id, sequence_id;
    uint32_t token_begin, token_end;
} cf_llama_server_slot_event;
#endif

cf_llama_server_multisequence *cf_llama_server_multisequence_create(const cf_llama_server_multisequence_config *config); /* :27-28 */
void cf_llama_server_multisequence_destroy(cf_llama_server_multisequence *bridge, void *stream);      /* :29 */
int cf_llama_server_slot_create(cf_llama_server_multisequence *bridge, int64_t slot_id, int64_t sequence_id); /* :31-33 */
int cf_llama_server_slot_reset_async(cf_llama_server_multisequence *bridge, int64_t slot_id, void *stream);   /* :34-36 */
int cf_llama_server_sequence_copy_async(cf_llama_server_multisequence *bridge, int64_t source_sequence, int64_t destination_sequence,
                                        uint32_t token_begin, uint32_t token_end, void *stream);     /* :37-42 */
int cf_llama_server_sequence_remove_async(cf_llama_server_multisequence *bridge, int64_t sequence_id, int64_t position_begin,
                                          int64_t position_end, void *stream);                       /* :43-47 */
int cf_llama_server_context_shift_async(cf_llama_server_multisequence *bridge, int64_t sequence_id, uint32_t position_begin,
                                        uint32_t position_end, int32_t delta, void *stream);         /* :48-53 */
int cf_llama_server_cancel_sequence_async(cf_llama_server_multisequence *bridge, int64_t sequence_id, void *stream); /* :54-56 */
int cf_llama_server_batch_attention_async(cf_llama_server_multisequence *bridge, const cf_sequence_attention_item *items,
                                          uint32_t item_count, void *stream);                        /* :57-60 */
int cf_llama_server_audit(const cf_llama_server_multisequence *bridge);                               /* :61 */
const char *cf_llama_server_multisequence_last_error(const cf_llama_server_multisequence *bridge);    /* :62 */

#ifdef __cplusplus
}
#endif

#endif
