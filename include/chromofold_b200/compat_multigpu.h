/* compat_multigpu.h — the reference's multi-GPU runtime ABI (include/chromofold/multigpu_cuda_runtime.h:9-111), same
 * symbols and struct layouts. In the reference these calls admit or refuse a batch of shards and account for the
 * pages that would cross GPUs; they launch nothing (src/cuda/multigpu_cuda_runtime.cu:92-193). The same holds here:
 * the rules (at least two devices with unique ordinals and a memory budget, 2 <= tensor_parallel_size <= devices,
 * a failed or unknown execution device refuses the batch, pages need a codec of 2 / 4 / 8 / 16 bits and the shard's
 * head_dim, remote pages need a peer path or permitted host staging) and the counters are kept so that a scheduler
 * written against them keeps working. The data path of this library on several GPUs is one process per GPU with
 * sequences or kv heads sharded by chromofold_b200/scheduler.py and no exchange but an output gather. */
#ifndef CHROMOFOLD_B200_COMPAT_MULTIGPU_H
#define CHROMOFOLD_B200_COMPAT_MULTIGPU_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* The reference's header uses `#pragma once`: a translation unit that has already included it defines
 * CHROMOFOLD_MULTIGPU_CUDA_RUNTIME_TYPES before this header. */
#ifndef CHROMOFOLD_MULTIGPU_CUDA_RUNTIME_TYPES
typedef enum cf_multigpu_transport { CF_MULTIGPU_TRANSPORT_P2P = 1, CF_MULTIGPU_TRANSPORT_HOST_STAGED = 2 } cf_multigpu_transport;
typedef enum cf_multigpu_collective {
    CF_MULTIGPU_COLLECTIVE_NONE = 0, CF_MULTIGPU_COLLECTIVE_NCCL_ALL_REDUCE = 1, CF_MULTIGPU_COLLECTIVE_HOST_REDUCE = 2,
} cf_multigpu_collective;

typedef struct cf_multigpu_device_config { /* :20-24 */
    int32_t device_ordinal;
    uint64_t memory_budget_bytes;
    uint32_t peer_group;
} cf_multigpu_device_config;

typedef struct cf_multigpu_runtime_config { /* :26-34 */
    const cf_multigpu_device_config *devices;
    uint32_t device_count, layer_count, tensor_parallel_size, allow_host_staging, require_peer_access, collective;
} cf_multigpu_runtime_config;

typedef struct cf_multigpu_page_view { /* :36-51 */
    const void *key_payload, *value_payload, *key_scales, *value_scales;
    uint64_t key_payload_bytes, value_payload_bytes;
    uint32_t key_codec, value_codec, token_count, kv_head_count, head_dim, block_size;
    int32_t source_device;
    uint64_t generation;
} cf_multigpu_page_view;

typedef struct cf_multigpu_attention_shard { /* :53-66 */
    uint64_t sequence_id;
    uint32_t layer, query_head_begin, query_head_count;
    int32_t execution_device;
    const void *query;
    void *output;
    uint32_t query_type, output_type, head_dim, page_count;
    const cf_multigpu_page_view *pages;
} cf_multigpu_attention_shard;

typedef struct cf_multigpu_counters { /* :68-88 */
    uint64_t batches_submitted, shards_dispatched, p2p_copy_calls, p2p_bytes, host_staged_copy_calls, host_staged_bytes;
    uint64_t collective_calls, collective_bytes, mixed_codec_pages_consumed, remote_pages_loaded, migrations_completed;
    uint64_t device_failures_detected, fail_closed_rejections, cross_device_contamination, dense_fallback_launches;
    uint64_t cuda_errors, transfer_errors, page_refs_at_shutdown, snapshot_refs_at_shutdown;
} cf_multigpu_counters;
#endif

typedef struct cf_multigpu_cuda_runtime cf_multigpu_cuda_runtime;

cf_multigpu_cuda_runtime *cf_multigpu_cuda_create(const cf_multigpu_runtime_config *config);                  /* :92 */
void cf_multigpu_cuda_destroy(cf_multigpu_cuda_runtime *runtime);                                             /* :93 */
int cf_multigpu_cuda_validate_topology(cf_multigpu_cuda_runtime *runtime);                                    /* :94 */
int cf_multigpu_cuda_execute_async(cf_multigpu_cuda_runtime *runtime, const cf_multigpu_attention_shard *shards,
                                   uint32_t shard_count, void *stream);                                       /* :95-98 */
int cf_multigpu_cuda_migrate_sequence_async(cf_multigpu_cuda_runtime *runtime, uint64_t sequence_id, int32_t source_device,
                                            int32_t destination_device, const cf_multigpu_page_view *pages,
                                            uint32_t page_count, void *stream);                               /* :99-105 */
int cf_multigpu_cuda_inject_device_failure(cf_multigpu_cuda_runtime *runtime, int32_t device_ordinal);        /* :106-107 */
int cf_multigpu_cuda_shutdown(cf_multigpu_cuda_runtime *runtime);                                             /* :108 */
int cf_multigpu_cuda_get_counters(const cf_multigpu_cuda_runtime *runtime, cf_multigpu_counters *counters);  /* :109-110 */
const char *cf_multigpu_cuda_last_error(const cf_multigpu_cuda_runtime *runtime);                             /* :111 */

#ifdef __cplusplus
}
#endif

#endif
