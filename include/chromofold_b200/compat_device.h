/* compat_device.h — the reference's device-resident KV ABIs, same symbols and struct layouts, served by the sealed-KV
 * path of this library:
 *   include/chromofold/device_kv_dataplane.h:11-89      cf_device_tensor_view, cf_device_kv_*   (append seam)
 *   include/chromofold/device_kv_seal_attention.h:11-123 cf_device_seal_*                        (GPU seal engine)
 * Kept from the reference: opaque handles, int 0 / -1 returns with a last_error string owned by the handle, exceptions
 * never cross the boundary, handles are created without touching CUDA (device memory is taken on first use), the ten
 * host-side fault points and the seal state machine: a failed seal leaves the active page intact, the page table
 * generation unchanged and the layer in CF_SEAL_ACTIVE_FULL (src/cuda/device_kv_seal_attention.cu:328-333). The fault
 * points fire in the reference's order: a page with NaN / Inf is refused ahead of every point after FINITE_VALIDATION,
 * PAGE_TABLE_GROW fires at a layer's 1st, 5th, 9th, 17th ... page (where the reference's descriptor table grows), an
 * armed fault stays armed, and an aborted attempt books the scan / quantise / pack work it got past, as the reference
 * does. tests/test_gpu_random_cases.py runs this engine beside the reference's own (compiled from its source): same
 * status for every call, same state after it, equal counters. A layer without sealed pages is staged at any
 * position; with sealed pages only at the next one (the reference takes any, and would publish pages with gaps).
 * Different: pages are int8 + entropy-coded format-v1 records sealed in ONE launch (the reference: int4 nibbles,
 * six launches); a page of page_size tokens is stored as page_size / T records of T tokens (T * head_dim <= 4096;
 * T = 16 at head_dim 128, 96, 64 and 32 with pages of a multiple of 16 tokens, where the lane-per-block attention
 * kernels serve these calls, fp32 queries included);
 * cf_device_kv_seal_full_pages_async and cf_device_kv_attention_async work (the reference ships them as fail-closed
 * stubs, src/cuda/device_kv_dataplane.cu:208-224). cf_device_page_descriptor is declared for layout compatibility;
 * this engine keeps its pages in its own arena and hands out no descriptors. */
#ifndef CHROMOFOLD_B200_COMPAT_DEVICE_H
#define CHROMOFOLD_B200_COMPAT_DEVICE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#ifndef CHROMOFOLD_DEVICE_KV_DATAPLANE_H
typedef enum cf_device_scalar_type { CF_DEVICE_F16 = 1, CF_DEVICE_BF16 = 2, CF_DEVICE_F32 = 3 } cf_device_scalar_type;

typedef struct cf_device_tensor_view { /* device_kv_dataplane.h:17-27 */
    const void *data;
    uint32_t scalar_type, token_count, head_count, head_dim;
    uint64_t token_stride_bytes, head_stride_bytes, element_stride_bytes;
    int32_t device_ordinal;
} cf_device_tensor_view;

typedef struct cf_device_kv_config { /* :29-37 */
    uint32_t layer_count, kv_head_count, query_head_count, head_dim, page_size, gqa_group_size, use_async_allocator;
} cf_device_kv_config;

typedef struct cf_device_kv_counters { /* :39-64 */
    uint64_t device_append_calls, device_values_appended, fp16_values_converted, bf16_values_converted, fp32_values_copied;
    uint64_t quantization_launches, huffman_pack_launches, seal_attempts, seal_successes, seal_failures;
    uint64_t descriptor_publications, compressed_attention_launches, sealed_values_consumed, active_values_consumed;
    uint64_t query_conversion_launches, output_conversion_launches, dense_fallback_launches, cuda_errors;
    uint64_t active_bytes, compressed_bytes, descriptor_bytes, workspace_bytes, retired_pending_bytes, peak_owned_bytes;
} cf_device_kv_counters;

typedef struct cf_device_kv_dataplane cf_device_kv_dataplane;
#endif

int cf_device_tensor_validate(const cf_device_tensor_view *view);                               /* :68 */
cf_device_kv_dataplane *cf_device_kv_create(const cf_device_kv_config *config);                 /* :69 */
void cf_device_kv_destroy(cf_device_kv_dataplane *dataplane, void *stream);                      /* :70 */
int cf_device_kv_append_async(cf_device_kv_dataplane *dataplane, uint32_t layer, uint32_t token_begin,
                              const cf_device_tensor_view *keys, const cf_device_tensor_view *values, void *stream); /* :71-76 */
int cf_device_kv_seal_full_pages_async(cf_device_kv_dataplane *dataplane, void *stream);         /* :77 */
int cf_device_kv_attention_async(cf_device_kv_dataplane *dataplane, uint32_t layer, const float *query, float *output,
                                 uint32_t query_token_count, uint32_t query_token_begin, float softmax_scale,
                                 uint32_t causal_window, void *stream);                           /* :78-86 */
int cf_device_kv_clear_async(cf_device_kv_dataplane *dataplane, void *stream);                   /* :87 */
int cf_device_kv_get_counters(const cf_device_kv_dataplane *dataplane, cf_device_kv_counters *counters); /* :88 */
const char *cf_device_kv_last_error(const cf_device_kv_dataplane *dataplane);                    /* :89 */

#ifndef CHROMOFOLD_DEVICE_KV_SEAL_ATTENTION_H
typedef enum cf_device_seal_state { /* device_kv_seal_attention.h:11-19 */
    CF_SEAL_ACTIVE_FILLING = 0, CF_SEAL_ACTIVE_FULL = 1, CF_SEAL_VALIDATING = 2, CF_SEAL_QUANTIZING = 3,
    CF_SEAL_PACKING = 4, CF_SEAL_PUBLISHING = 5, CF_SEAL_FAILED = 6,
} cf_device_seal_state;

typedef enum cf_device_seal_fault { /* :21-33 */
    CF_SEAL_FAULT_NONE = 0, CF_SEAL_FAULT_CANDIDATE_ALLOC = 1, CF_SEAL_FAULT_FINITE_VALIDATION = 2,
    CF_SEAL_FAULT_SCALE_ALLOC = 3, CF_SEAL_FAULT_QUANTIZE_LAUNCH = 4, CF_SEAL_FAULT_PAYLOAD_ALLOC = 5,
    CF_SEAL_FAULT_PACK_LAUNCH = 6, CF_SEAL_FAULT_DESCRIPTOR_VALIDATE = 7, CF_SEAL_FAULT_PAGE_TABLE_GROW = 8,
    CF_SEAL_FAULT_DESCRIPTOR_PUBLISH = 9, CF_SEAL_FAULT_ACTIVE_REPLACEMENT = 10,
} cf_device_seal_fault;

typedef struct cf_device_page_descriptor { /* :35-50 */
    const uint8_t *key_payload; const uint8_t *value_payload; const float *key_scales; const float *value_scales;
    uint32_t token_begin, token_count, kv_head_count, head_dim, block_size, blocks_per_page;
    uint64_t key_payload_bytes, value_payload_bytes, resident_bytes, generation;
} cf_device_page_descriptor;

typedef struct cf_device_seal_counters { /* :52-82 */
    uint64_t seal_attempts, seal_successes, seal_failures, finite_validation_launches, values_scanned, nan_values;
    uint64_t inf_values, invalid_pages_rejected, quantization_launches, values_quantized, saturation_count;
    uint64_t packing_launches, symbols_packed, payload_bytes_written, descriptor_validations, descriptor_publications;
    uint64_t page_table_reallocations, page_table_generation, compressed_attention_launches, sealed_pages_consumed;
    uint64_t sealed_values_consumed, active_values_consumed, query_conversion_launches, output_conversion_launches;
    uint64_t cuda_errors, compressed_bytes, descriptor_bytes, workspace_bytes, peak_owned_bytes;
} cf_device_seal_counters;

typedef struct cf_device_seal_config { /* :84-93 */
    uint32_t layer_count, kv_head_count, query_head_count, head_dim, page_size, gqa_group_size, block_size, use_async_allocator;
} cf_device_seal_config;

typedef struct cf_device_seal_engine cf_device_seal_engine;
#endif

cf_device_seal_engine *cf_device_seal_create(const cf_device_seal_config *config);               /* :97 */
void cf_device_seal_destroy(cf_device_seal_engine *engine, void *stream);                         /* :98 */
int cf_device_seal_stage_active_page(cf_device_seal_engine *engine, uint32_t layer, uint32_t token_begin,
                                     const float *active_k, const float *active_v, uint32_t token_count, void *stream); /* :99-105 */
int cf_device_seal_full_page_async(cf_device_seal_engine *engine, uint32_t layer, void *stream); /* :106 */
int cf_device_seal_attention_async(cf_device_seal_engine *engine, uint32_t layer, const cf_device_tensor_view *query,
                                   void *output, uint32_t output_scalar_type, uint64_t output_token_stride_bytes,
                                   uint64_t output_head_stride_bytes, uint64_t output_element_stride_bytes,
                                   uint32_t query_token_begin, float softmax_scale, uint32_t causal_window, void *stream); /* :107-118 */
int cf_device_seal_clear_async(cf_device_seal_engine *engine, void *stream);                     /* :119 */
int cf_device_seal_set_fault(cf_device_seal_engine *engine, uint32_t fault);                     /* :120 */
int cf_device_seal_get_state(const cf_device_seal_engine *engine, uint32_t layer, uint32_t *state); /* :121 */
int cf_device_seal_get_counters(const cf_device_seal_engine *engine, cf_device_seal_counters *counters); /* :122 */
const char *cf_device_seal_last_error(const cf_device_seal_engine *engine);                       /* :123 */

#ifdef __cplusplus
}
#endif

#endif
