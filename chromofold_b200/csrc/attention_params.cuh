// attention_params.cuh — launch parameters shared by the plan, attention and combine kernels.
#ifndef CHROMOFOLD_B200_ATTENTION_PARAMS_CUH
#define CHROMOFOLD_B200_ATTENTION_PARAMS_CUH

#include "cf_device_common.cuh"

namespace cfb {

constexpr uint32_t kDefaultWaitPolls = 1u << 22;   // about a microsecond each at most: seconds before a wait gives up

struct AttentionParams {
    // geometry
    uint32_t kv_head_count, query_head_count, head_dim, page_tokens, block_size;
    uint32_t kv_head_begin, kv_head_span, group;  // group = query heads per kv head
    uint32_t symbols, nblocks, codebook_id;
    // sealed pages
    const uint8_t *arena;
    const uint64_t *page_dir;
    const uint32_t *page_table;
    const uint32_t *seq_sealed_tokens;
    const uint32_t *seq_slots;
    uint32_t page_table_stride, seq_count;
    const cf_b200_codebook_tables *k_tables, *v_tables;
    // tails
    const void *tail_k, *tail_v;
    const uint32_t *tail_tokens;
    uint32_t tail_type, tail_capacity;
    const uint32_t *query_positions;
    const uint32_t *row_map;        // optional: batch entry -> row of queries / output
    // io
    const void *queries;
    void *output;
    uint32_t query_type, output_type;
    float softmax_scale;
    uint32_t causal_window;
    // split-KV
    uint8_t *workspace;
    WorkspaceLayout layout;
    uint32_t min_pages_per_unit;    // 0 = the plan kernel chooses (default_pages_per_unit)
    uint32_t shared_prefix_pages;   // the caller's hint, already zeroed when the launch cannot use it
    uint32_t sm_count;
    uint32_t decode_probe;          // 1 = measurement: decode every page, fold the symbols into a checksum, no attention;
                                    // 2 = test: store every decoded symbol to `output` ([page id][kv head][K | V stream])
    uint32_t dump_pages;            // page ids the dump buffer covers (1 when decode_probe != 2)
    uint32_t wait_polls;            // bound of every wait on a copy or a barrier, in polls
    uint32_t skip_copy_page;        // test hook: the record of this page id is never fetched (its wait must run out); 0 = off
    uint32_t *status;
    // uncompressed comparison pools (dense kernel only)
    const __half *pool_k, *pool_v;
};

#ifdef __CUDACC__
__device__ __forceinline__ PlanHeader *plan_header(const AttentionParams &p) {
    return reinterpret_cast<PlanHeader *>(p.workspace);
}
__device__ __forceinline__ uint32_t *chunk_prefix(const AttentionParams &p) {
    return reinterpret_cast<uint32_t *>(p.workspace + p.layout.prefix_offset);
}
__device__ __forceinline__ ChunkInfo *chunk_info(const AttentionParams &p) {
    return reinterpret_cast<ChunkInfo *>(p.workspace + p.layout.info_offset);
}
__device__ __forceinline__ float *partial_ptr(const AttentionParams &p, uint32_t chunk, uint32_t local_q_head) {
    return reinterpret_cast<float *>(p.workspace + p.layout.partials_offset) +
           (static_cast<uint64_t>(chunk) * (p.kv_head_span * p.group) + local_q_head) * p.layout.partial_stride_floats;
}
// Shared-prefix partial of (cell, batch entry, local query head); cells as SharedSplit numbers them.
__device__ __forceinline__ float *shared_partial_ptr(const AttentionParams &p, uint32_t chunk, uint32_t seq, uint32_t local_q_head) {
    return reinterpret_cast<float *>(p.workspace + p.layout.shared_offset) +
           ((static_cast<uint64_t>(chunk) * p.seq_count + seq) * (p.kv_head_span * p.group) + local_q_head) *
               p.layout.partial_stride_floats;
}
// Row of the query and output tensors that batch entry `seq` stands for.
__device__ __forceinline__ uint32_t row_of(const AttentionParams &p, uint32_t seq) {
    return p.row_map ? p.row_map[seq] : seq;
}
__device__ __forceinline__ uint32_t slot_of(const AttentionParams &p, uint32_t seq) {
    return p.seq_slots ? p.seq_slots[seq] : seq;
}
// Position of the query token of batch entry `seq`: given, or right after everything cached (a decode step).
__device__ __forceinline__ uint32_t query_position(const AttentionParams &p, uint32_t seq, uint32_t sealed, uint32_t tail) {
    return p.query_positions ? p.query_positions[seq] : sealed + tail;
}
__device__ __forceinline__ float load_tail(const void *base, uint32_t type, uint64_t i) {
    return type == CF_B200_F32 ? static_cast<const float *>(base)[i] : __half2float(static_cast<const __half *>(base)[i]);
}
__device__ __forceinline__ void raise_status(const AttentionParams &p, uint32_t bits) {
    if (p.status) atomicOr(p.status, bits);
}
// Sequence that owns chunk `c`: the last s with chunk_prefix[s] <= c.
__device__ __forceinline__ uint32_t sequence_of_chunk(const uint32_t *prefix, uint32_t seq_count, uint32_t c) {
    uint32_t lo = 0, hi = seq_count;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (prefix[mid] <= c) lo = mid; else hi = mid;
    }
    return lo;
}
#endif

// Implemented in sealed_attention.cu
cf_status sealed_attention_stages(const cf_b200_sealed_attention_desc *d, uint32_t stages, void *stream, bool output_on_peer);
cudaError_t launch_plan(const AttentionParams &p, cudaStream_t stream);
cudaError_t launch_combine(const AttentionParams &p, cudaStream_t stream);
cudaError_t launch_generic_attention(const AttentionParams &p, cudaStream_t stream);
// Implemented in sealed_attention_lanes.cu
bool lanes_kernel_supports(const AttentionParams &p);
cudaError_t launch_lanes_attention(const AttentionParams &p, cudaStream_t stream);
// Implemented in sealed_attention_prefix.cu
cudaError_t launch_prefix_attention(const AttentionParams &p, cudaStream_t stream);
// Implemented in dense_attention.cu
cudaError_t launch_dense_attention(const AttentionParams &p, cudaStream_t stream);

}  // namespace cfb

#endif
