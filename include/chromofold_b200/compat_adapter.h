/* compat_adapter.h — the llama.cpp-facing KV adapter, same symbols and struct layouts as the reference's
 * integrations/llama.cpp/chromofold_kv_adapter.h:13-89, served by the sealed-KV path of this library.
 *
 * A caller compiled against the reference header links against this library unchanged: every function below has
 * the reference's name, argument list and return convention (0 / -1 and a last_error string owned by the handle,
 * exceptions never cross the boundary — chromofold_kv_adapter.cpp:35-49).
 *
 * What is kept: one sequence (id 0) per adapter (src/runtime/compressed_kv_cache.cu:180-193); append takes HOST fp32
 * rows per (layer, kv head) and must be logically contiguous (:78-80); full pages seal on append (:87), flush seals
 * the partial tail (:111-125); attention takes DEVICE fp32 queries [query_count][Hq][head_dim], query row i sits at
 * token query_token_begin + i and sees tokens <= its position inside the causal window
 * (src/cuda/paged_kv_attention.cu:48-52,67-69); all kv heads must hold the same tokens when attention runs
 * (compressed_kv_cache.cu:152-154).
 * Pages. By default they are the reference's own: kv_bits 8 gives int8, anything else int4 (chromofold_kv_adapter.cpp:30-31),
 * K with one fp32 scale per channel and V with one per token (src/runtime/kv_gpu_fixture.cpp:46-95), made on the GPU bit
 * for bit as gpu_fixture::encode_int{4,8}_page makes them on the host, one page per page_size tokens, and attended through
 * cf_kv_paged_attention_async as the reference's adapter does — so a caller that swaps this library in gets the
 * reference's numbers. With CHROMOFOLD_B200_CODER = rans | huffman | fixed8 | rans4 | huffman4 in the environment the pages
 * are instead quantised to int8 with one fp16 scale per stream and entropy coded (format v1, sealed_page_format.h):
 * physically a page of page_size tokens is then page_size / T records of T tokens with T * head_dim <= 4096 (T = 16 at
 * head_dim 128, 96, 64 and 32 with pages of a multiple of 16 tokens: the record geometry of the lane-per-block
 * attention kernels, which take the fp32 queries of this ABI as binary16 + residue rows). Statistics are reported in the
 * reference's units in both modes.
 * tests/test_gpu_random_cases.py runs this adapter beside the reference's own, end to end (compiled from its sources):
 * same status for every call, equal statistics, attention equal to 2e-4. Narrower in one point: rows appended right
 * after a page was sealed must start at the next position (the reference takes any position there). */
#ifndef CHROMOFOLD_B200_COMPAT_ADAPTER_H
#define CHROMOFOLD_B200_COMPAT_ADAPTER_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CHROMOFOLD_LLAMA_KV_ADAPTER_H /* the reference header declares the same types */
typedef enum cf_llama_kv_backend {
    CF_LLAMA_KV_BACKEND_DENSE = 0,
    CF_LLAMA_KV_BACKEND_CHROMOFOLD = 1,
} cf_llama_kv_backend;

typedef struct cf_llama_kv_options { /* chromofold_kv_adapter.h:18-28 */
    uint32_t struct_size;
    cf_llama_kv_backend backend;
    uint32_t layer_count;
    uint32_t kv_head_count;
    uint32_t query_head_count;
    uint32_t head_dim;
    uint32_t page_size;
    uint32_t gqa_group_size;
    uint32_t kv_bits;
} cf_llama_kv_options;

typedef struct cf_llama_kv_stats { /* chromofold_kv_adapter.h:30-38 */
    uint64_t appended_tokens;
    uint64_t sealed_tokens;
    uint64_t sealed_pages;
    uint64_t active_tokens;
    uint64_t dense_active_bytes;
    uint64_t compressed_bytes;
    uint64_t descriptor_bytes;
} cf_llama_kv_stats;

typedef struct cf_llama_kv_adapter cf_llama_kv_adapter;
#endif

int cf_llama_kv_options_validate(const cf_llama_kv_options *options);                 /* :42 */
cf_llama_kv_adapter *cf_llama_kv_create(const cf_llama_kv_options *options);          /* :43 */
void cf_llama_kv_destroy(cf_llama_kv_adapter *adapter);                               /* :44 */
int cf_llama_kv_append(cf_llama_kv_adapter *adapter, uint32_t layer, uint32_t kv_head, uint32_t token_begin,
                       const float *keys, const float *values, uint32_t token_count, void *stream); /* :46-53 */
int cf_llama_kv_attention(cf_llama_kv_adapter *adapter, uint32_t layer, const float *queries_device,
                          float *output_device, uint32_t query_count, uint32_t query_head_count,
                          uint32_t gqa_group_size, uint32_t query_token_begin, float softmax_scale,
                          uint32_t causal_window, void *stream);                       /* :58-68 */
int cf_llama_kv_attention_host(cf_llama_kv_adapter *adapter, uint32_t layer, const float *queries_host,
                               float *output_host, uint32_t query_count, uint32_t query_head_count,
                               uint32_t gqa_group_size, uint32_t query_token_begin, float softmax_scale,
                               uint32_t causal_window, void *stream);                  /* :72-82 */
int cf_llama_kv_flush(cf_llama_kv_adapter *adapter, void *stream);                    /* :84 */
int cf_llama_kv_seq_rm(cf_llama_kv_adapter *adapter, uint64_t sequence_id);           /* :85 */
int cf_llama_kv_seq_cp(cf_llama_kv_adapter *adapter, uint64_t source_id, uint64_t destination_id); /* :86 */
int cf_llama_kv_seq_shift(cf_llama_kv_adapter *adapter, uint64_t sequence_id, int32_t delta);      /* :87 */
int cf_llama_kv_clear(cf_llama_kv_adapter *adapter);                                  /* :88 */
int cf_llama_kv_get_stats(const cf_llama_kv_adapter *adapter, cf_llama_kv_stats *stats); /* :89 */
const char *cf_llama_kv_last_error(const cf_llama_kv_adapter *adapter);               /* :91 */

#include "chromofold_b200/compat_kv.h"
/* Additive: the descriptor (device pointers) of page `page_index` of `layer` in reference-exact mode, pages counted in
 * the order they were sealed over all kv heads; -1 in format-v1 mode or out of range. */
int cf_b200_llama_kv_reference_page(const cf_llama_kv_adapter *adapter, uint32_t layer, uint32_t page_index,
                                    cf_kv_device_page *out_page);
/* Additive: bytes of page memory the adapter holds on the device (reference-exact mode). The reference's options have no
 * context limit, so page memory grows in 32 MB chunks as tokens arrive; CHROMOFOLD_B200_RESERVE_TOKENS=<tokens per
 * sequence position, i.e. context length> in the environment makes cf_llama_kv_create take the chunks and the
 * descriptor arrays for that many tokens of every layer and kv head up front, so that no append allocates. */
uint64_t cf_b200_llama_kv_reserved_bytes(const cf_llama_kv_adapter *adapter);

#ifdef __cplusplus
}
#endif

#endif
