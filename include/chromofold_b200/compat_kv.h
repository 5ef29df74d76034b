/* compat_kv.h — the reference's own C symbols for this path, re-implemented: a program compiled against the
 * reference headers (include/chromofold/{chromofold,kv_runtime,kv_cuda}.h) links against this library unchanged.
 * Struct layouts are byte-identical to the reference's (sizes: cf_kv_page_view 168, cf_kv_cache_layout 72,
 * cf_kv_device_page 104, cf_kv_paged_attention_desc 96, cf_online_softmax_state 32 bytes on x86-64). */
#ifndef CHROMOFOLD_B200_COMPAT_KV_H
#define CHROMOFOLD_B200_COMPAT_KV_H

#include <stddef.h>
#include <stdint.h>

#include "chromofold_b200/cf_status.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- include/chromofold/kv_runtime.h ------------------------------------------------------------------ */
#ifndef CHROMOFOLD_KV_RUNTIME_H
#define CF_KV_RUNTIME_ABI_VERSION 0u
#define CF_KV_PAGE_FLAG_SEALED 0x1u
#define CF_KV_PAGE_FLAG_DEVICE_RESIDENT 0x2u

typedef struct cf_kv_page_view { /* kv_runtime.h:23-53 */
    uint32_t struct_size, abi_version, flags, layer, kv_head, token_begin, token_count, head_dim, block_size, zero_point;
    const uint32_t *k_words;       uint64_t k_word_count;
    const int32_t *k_block_offsets; uint64_t k_block_count;
    const int32_t *k_lut;          uint64_t k_lut_count;
    const float *k_scales;         uint64_t k_scale_count;
    const uint32_t *v_words;       uint64_t v_word_count;
    const int32_t *v_block_offsets; uint64_t v_block_count;
    const int32_t *v_lut;          uint64_t v_lut_count;
    const float *v_scales;         uint64_t v_scale_count;
} cf_kv_page_view;

typedef struct cf_kv_cache_layout { /* kv_runtime.h:59-75 */
    uint32_t struct_size, abi_version, layer_count, kv_head_count, head_dim, page_capacity_tokens;
    uint32_t active_token_begin, active_token_count, active_element_bytes, reserved;
    const cf_kv_page_view *pages;
    uint64_t page_count, active_k_bytes, active_v_bytes;
} cf_kv_cache_layout;

typedef struct cf_kv_memory_stats { /* kv_runtime.h:77-85 */
    uint64_t sealed_payload_bytes, sealed_descriptor_bytes, active_payload_bytes, total_resident_bytes;
    uint64_t sealed_tokens, active_tokens, page_count;
} cf_kv_memory_stats;

typedef struct cf_online_softmax_state { /* kv_runtime.h:90-96 */
    double max_score, exp_sum;
    double *weighted_values;
    uint32_t dim, initialized;
} cf_online_softmax_state;
#endif

cf_status cf_kv_validate_page(const cf_kv_page_view *page);                                   /* kv_runtime.h:98 */
cf_status cf_kv_validate_layout(const cf_kv_cache_layout *layout);                            /* :99 */
cf_status cf_kv_page_resident_bytes(const cf_kv_page_view *page, uint64_t *out_bytes);        /* :100 */
cf_status cf_kv_cache_memory_stats(const cf_kv_cache_layout *layout, cf_kv_memory_stats *out_stats); /* :101 */
cf_status cf_online_softmax_init(cf_online_softmax_state *state, double *weighted_values, uint32_t dim); /* :103 */
cf_status cf_online_softmax_accumulate(cf_online_softmax_state *state, double score, const float *value); /* :104 */
cf_status cf_online_softmax_merge(cf_online_softmax_state *dst, const cf_online_softmax_state *src);      /* :105 */
cf_status cf_online_softmax_finalize(const cf_online_softmax_state *state, float *out);                   /* :106 */

/* ---- include/chromofold/kv_cuda.h ------------------------------------------------------------------- */
#ifndef CHROMOFOLD_KV_CUDA_H
#define CF_KV_CUDA_ABI_VERSION 0u
#define CF_KV_CUDA_MAX_PAGES_PER_LAUNCH 4096u

typedef struct cf_kv_device_page { /* kv_cuda.h:21-41 */
    const uint32_t *k_words; const int32_t *k_block_offsets; const int32_t *k_lut; const float *k_scales;
    const uint32_t *v_words; const int32_t *v_block_offsets; const int32_t *v_lut; const float *v_scales;
    uint32_t token_begin, token_count, head_dim, block_size, k_max_code_length, v_max_code_length, zero_point, kv_head;
    uint32_t fixed_code_length;
} cf_kv_device_page;

typedef struct cf_kv_paged_attention_desc { /* kv_cuda.h:53-75 */
    uint32_t struct_size, abi_version;
    const cf_kv_device_page *pages;
    uint32_t page_count, kv_head_count, query_head_count, gqa_group_size;
    const float *active_k; const float *active_v;
    uint32_t active_token_begin, active_token_count;
    const float *queries; float *output;
    uint32_t query_token_begin, query_count, head_dim, causal_window;
    float softmax_scale;
} cf_kv_paged_attention_desc;
#endif

/* Host-side structural validation (src/cuda/paged_kv_attention.cu:280-299). */
cf_status cf_kv_validate_paged_attention_desc(const cf_kv_paged_attention_desc *desc);        /* kv_cuda.h:78 */
/* Paged attention over the reference's own page descriptors: fixed-width 4/8-bit and variable-length Huffman
 * pages (per-page LUT, K per-channel and V per-token fp32 scales), fp32 active tail, fp32 queries, several query
 * rows with the causal rule. No allocation, synchronisation or host transfer (kv_cuda.h:80-86). Here one thread
 * block serves (query row, kv head) for the whole query group, decodes each page once into shared memory with one
 * thread per coded block, and variable-length pages take the same parallel path (the reference walks them one
 * bit per global load in a single thread, src/cuda/paged_kv_attention.cu:41-176). */
cf_status cf_kv_paged_attention_async(const cf_kv_paged_attention_desc *desc, void *stream);  /* kv_cuda.h:86 */

/* ---- src/cuda/rans.cu:38-50 ------------------------------------------------------------------------- */
/* Whole-tensor block-rANS decode of the flat stream layout of tools/export_rans.py:13-17. */
cf_status cf_rans_decode_async(const uint8_t *data, const int32_t *byte_off, const uint32_t *state0,
                               const int32_t *slot2sym, const int32_t *freq, const int32_t *cum, int block, int n,
                               int32_t *out, void *stream);

/* ---- include/chromofold/chromofold.h:81-98 ------------------------------------------------------------ */
/* Flat (non-paged) causal windowed attention over block-Huffman coded K / V (K per-channel, V per-token scales):
 * query row i attends rows max(0, i-window+1) .. i. The fused call decodes inside the consumer; the dense call first
 * writes fp32 K / V to the caller's scratch and runs the same arithmetic — both give bit-identical outputs
 * (src/cuda/fused_kv_attention.cu:1-8). Bounds as in the reference: dim <= 128, window <= 512, nq <= seq. */
cf_status cf_kv_attn_fused_async(const uint32_t *kw, const int32_t *kb, const int32_t *kl, int kmax, const uint32_t *vw,
                                 const int32_t *vb, const int32_t *vl, int vmax, const float *kscale, const float *vscale,
                                 const float *Q, float *out, int seq, int dim, int nq, int window, int block, int zero,
                                 float sscale, void *stream);
cf_status cf_kv_attn_dense_async(const uint32_t *kw, const int32_t *kb, const int32_t *kl, int kmax, const uint32_t *vw,
                                 const int32_t *vb, const int32_t *vl, int vmax, const float *kscale, const float *vscale,
                                 const float *Q, float *Kd, float *Vd, float *out, int seq, int dim, int nq, int window,
                                 int block, int zero, float sscale, void *stream);

/* Token-id fetch from a reference/delta cluster (src/cuda/delta_apply.cu:30-44; cluster layout of
 * tools/export_delta.py:13-17): out[i] = the override of leaf device_leaf[i] at position device_pos[i] if it has one
 * (its dpos[dstart[leaf] .. +dlen[leaf]) is sorted ascending), else base[pos], else -1 when pos is past the base.
 * All pointers are device pointers; dpos / dval may be NULL when every dlen is 0. */
cf_status cf_delta_fetch_async(const int32_t *base, int nbase, const int32_t *dpos, const int32_t *dval,
                               const int32_t *dstart, const int32_t *dlen, const int32_t *device_leaf,
                               const int32_t *device_pos, int32_t *out, size_t count, void *stream);

#ifdef __cplusplus
}
#endif

#endif
