/* sealed_kv_multigpu.h — batch scheduler for the GPUs of one box: ONE host process drives every GPU, one stream per
 * GPU, and a decode step is split either by sequence or by kv head. Attention of one (sequence, kv head) depends on
 * nothing else, so no collective is needed; the only exchange is moving the query rows out to the GPUs and the
 * output rows back to the root GPU, as ordinary peer copies (no multicast, and no kernel is ever given another
 * GPU's memory as an operand).
 *
 * What it stands in for: the reference's shard descriptor names an execution device and a block of query heads
 * (cf_multigpu_attention_shard, include/chromofold/multigpu_cuda_runtime.h:53-66) and its executor checks the shards
 * and counts what would move, but launches nothing (src/cuda/multigpu_cuda_runtime.cu:92-193); its only placement
 * rule is a seeded hash that ignores load (src/distributed_runtime.cpp:37-43,73-74). The reference's symbols with
 * those semantics are kept in compat_multigpu.h; the entry points here are the ones that run.
 *
 *   sequences over GPUs — longest-processing-time bin packing on context length (ties: lower sequence index, then
 *                         lower device index), every GPU holds the pages of its own sequences;
 *   kv heads over GPUs  — contiguous blocks of kv heads, query heads follow their kv head, so the per-GPU outputs are
 *                         disjoint column blocks of the output: a gather, not a reduction.
 *
 * A GPU marked failed (host-side flag, as src/cuda/multigpu_cuda_runtime.cu:119-123,219-232) gets no work from the
 * planners and makes cf_b200_mg_execute_async refuse a batch that still names it.
 */
#ifndef CHROMOFOLD_B200_SEALED_KV_MULTIGPU_H
#define CHROMOFOLD_B200_SEALED_KV_MULTIGPU_H

#include "chromofold_b200/sealed_kv.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CF_B200_MG_MAX_DEVICES 16u

typedef struct cf_b200_mg_config {
    uint32_t struct_size;
    uint32_t abi_version;            /* CF_B200_ABI_VERSION */
    uint32_t device_count;           /* 1..CF_B200_MG_MAX_DEVICES */
    const int32_t *device_ordinals;  /* [device_count] CUDA ordinals, unique; [0] is the root: queries arrive there and
                                        outputs are gathered there */
    uint32_t max_rows;               /* largest batch (query rows) of a step */
    uint32_t query_head_count;
    uint32_t head_dim;
    uint32_t query_type;             /* CF_B200_F16 or CF_B200_F32; outputs are float */
} cf_b200_mg_config;

typedef struct cf_b200_mg_scheduler cf_b200_mg_scheduler;

/* Creates the per-device streams and events and the root's staging buffers (2 x max_rows rows); nothing is allocated
 * after this call. Returns NULL on a bad config or a CUDA error. */
cf_b200_mg_scheduler *cf_b200_mg_create(const cf_b200_mg_config *config);
void cf_b200_mg_destroy(cf_b200_mg_scheduler *scheduler);
const char *cf_b200_mg_last_error(const cf_b200_mg_scheduler *scheduler);

/* Host-side failure flag of one device (by ordinal); `failed` != 0 marks, 0 clears. Nothing is done to the GPU. */
cf_status cf_b200_mg_set_device_failed(cf_b200_mg_scheduler *scheduler, int32_t device_ordinal, uint32_t failed);

/* Planners (host arithmetic only; scheduler may be NULL = no device is failed).
 * Sequences: out_device[i] = index (into device_ordinals) of the device that serves sequence i.
 * KV heads: out_begin[d], out_span[d] = block of kv heads of device index d (span 0 = idle). */
cf_status cf_b200_mg_plan_sequences(const cf_b200_mg_scheduler *scheduler, const uint64_t *context_lengths,
                                    uint32_t sequence_count, uint32_t device_count, uint32_t *out_device);
cf_status cf_b200_mg_plan_kv_heads(const cf_b200_mg_scheduler *scheduler, uint32_t kv_head_count, uint32_t device_count,
                                   uint32_t *out_begin, uint32_t *out_span);

/* One device's share of a step. `desc` is a complete descriptor over that device's own store (arena, directory,
 * page table, tables, tails, workspace, status: all in that device's memory), with
 *   desc.seq_count / desc.seq_slots = the batch entries this device serves (0 = the device sits the step out),
 *   desc.queries / desc.output      = device-local buffers of seq_count rows [query_head_count][head_dim]
 *                                     (the scheduler fills queries and reads output),
 *   desc.kv_head_begin / _span      = the device's kv heads (kv-head sharding).
 * rows (HOST array, [desc.seq_count]) = for each batch entry the row of the root's query / output tensors it stands
 * for; NULL = entry i is row i. */
typedef struct cf_b200_mg_shard {
    cf_b200_sealed_attention_desc desc;
    const uint32_t *rows;
} cf_b200_mg_shard;

#define CF_B200_MG_BY_SEQUENCE 1u   /* every device writes whole output rows (its own sequences) */
#define CF_B200_MG_BY_KV_HEAD 2u    /* every device writes its query-head columns of every row it lists */

/* One decode step over all devices. root_queries / root_output: [row_count][query_head_count][head_dim] in the root
 * device's memory (query_type / float). On root_stream (a stream of the root device) the call is ordered like a
 * kernel launch: it starts after the work queued there before, and work queued there afterwards sees the gathered
 * output. Per device: query rows are copied over, cf_b200_sealed_attention_async runs on the device's own stream,
 * the output rows (or columns) are copied back. Returns CF_ERR_UNSUPPORTED when a listed device is marked failed.
 *
 * Direct output: where every GPU has the root's memory mapped (peer access, enabled at creation) and the driver
 * confirms, per root_output, that every GPU may store to it, a GPU keeps a copy of the batch's query rows (one peer
 * copy per step), gets the rows of its entries as a row map (cf_b200_sealed_attention_desc.row_map) and its combine
 * kernel stores the output rows straight into root_output: no staging, no row permutation, no copies back. All loads
 * stay local to the GPU that issues them. CHROMOFOLD_B200_MG_COPIES=1 in the environment keeps the copy path. */
cf_status cf_b200_mg_execute_async(cf_b200_mg_scheduler *scheduler, const cf_b200_mg_shard *shards, uint32_t shard_count,
                                   const void *root_queries, void *root_output, uint32_t row_count, uint32_t mode,
                                   void *root_stream);

/* Launch counters since creation: steps, per-device attention launches, peer copies issued, bytes that crossed between
 * GPUs, refused batches, and the steps whose outputs were stored directly into the root's tensor (below). */
typedef struct cf_b200_mg_counters {
    uint64_t steps, attention_launches, peer_copies, peer_bytes, refused_batches, direct_steps;
} cf_b200_mg_counters;
cf_status cf_b200_mg_get_counters(const cf_b200_mg_scheduler *scheduler, cf_b200_mg_counters *out);

#ifdef __cplusplus
}
#endif

#endif
