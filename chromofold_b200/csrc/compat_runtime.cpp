// compat_runtime.cpp — host-side functions of the reference's kv_runtime.h, re-implemented (declared in
// include/chromofold_b200/compat_kv.h). Behaviour follows src/runtime/kv_runtime.cpp: which inputs are rejected with
// which status, exact byte accounting with overflow reported as CF_ERR_UNSUPPORTED, and the double-precision online
// softmax with its merge rule. Nothing here touches CUDA.

#include <cmath>
#include <initializer_list>
#include <cstring>
#include <limits>

#include "chromofold_b200/compat_kv.h"

namespace {

constexpr uint64_t kU64Max = std::numeric_limits<uint64_t>::max();

// Checked arithmetic: false on overflow.
bool checked_add(uint64_t a, uint64_t b, uint64_t &out) {
    if (a > kU64Max - b) return false;
    out = a + b;
    return true;
}
bool checked_mul(uint64_t a, uint64_t b, uint64_t &out) {
    if (a != 0 && b > kU64Max / a) return false;
    out = a * b;
    return true;
}

struct CountedArray { const void *data; uint64_t count; uint64_t element; bool must_exist; };

// The eight arrays of a page view in one table so that validation and accounting walk the same list.
void arrays_of(const cf_kv_page_view &p, CountedArray (&out)[8]) {
    out[0] = {p.k_words, p.k_word_count, sizeof(uint32_t), true};
    out[1] = {p.v_words, p.v_word_count, sizeof(uint32_t), true};
    out[2] = {p.k_block_offsets, p.k_block_count, sizeof(int32_t), true};
    out[3] = {p.v_block_offsets, p.v_block_count, sizeof(int32_t), true};
    out[4] = {p.k_lut, p.k_lut_count, sizeof(int32_t), true};
    out[5] = {p.v_lut, p.v_lut_count, sizeof(int32_t), true};
    out[6] = {p.k_scales, p.k_scale_count, sizeof(float), false};
    out[7] = {p.v_scales, p.v_scale_count, sizeof(float), false};
}

bool intervals_overlap(uint32_t a_begin, uint32_t a_count, uint32_t b_begin, uint32_t b_count) {
    return a_begin < static_cast<uint64_t>(b_begin) + b_count && b_begin < static_cast<uint64_t>(a_begin) + a_count;
}

}  // namespace

extern "C" cf_status cf_kv_validate_page(const cf_kv_page_view *page) {  // kv_runtime.cpp:41-74
    if (!page || page->struct_size != sizeof(cf_kv_page_view) || page->abi_version != CF_KV_RUNTIME_ABI_VERSION)
        return CF_ERR_INVALID_ARGUMENT;
    const bool sealed = (page->flags & CF_KV_PAGE_FLAG_SEALED) != 0;
    if (!sealed || page->token_count == 0 || page->head_dim == 0 || page->head_dim > CF_KV_MAX_HEAD_DIM ||
        page->block_size == 0)
        return CF_ERR_INVALID_ARGUMENT;
    CountedArray arrays[8];
    arrays_of(*page, arrays);
    for (const CountedArray &a : arrays) {
        if (a.count != 0 && a.data == nullptr) return CF_ERR_INVALID_ARGUMENT;
        if (a.must_exist && a.count == 0) return CF_ERR_INVALID_ARGUMENT;
    }
    if (page->k_scale_count != page->head_dim || page->v_scale_count != page->token_count) return CF_ERR_INVALID_ARGUMENT;
    uint64_t values;
    if (!checked_mul(page->token_count, page->head_dim, values)) return CF_ERR_UNSUPPORTED;
    const uint64_t blocks_needed = (values + page->block_size - 1) / page->block_size;
    if (page->k_block_count < blocks_needed || page->v_block_count < blocks_needed) return CF_ERR_INVALID_ARGUMENT;
    if (page->token_begin > std::numeric_limits<uint32_t>::max() - page->token_count) return CF_ERR_INVALID_ARGUMENT;
    return CF_OK;
}

extern "C" cf_status cf_kv_validate_layout(const cf_kv_cache_layout *layout) {  // kv_runtime.cpp:76-120
    if (!layout || layout->struct_size != sizeof(cf_kv_cache_layout) || layout->abi_version != CF_KV_RUNTIME_ABI_VERSION)
        return CF_ERR_INVALID_ARGUMENT;
    if (layout->layer_count == 0 || layout->kv_head_count == 0 || layout->head_dim == 0 ||
        layout->head_dim > CF_KV_MAX_HEAD_DIM || layout->page_capacity_tokens == 0 || layout->active_element_bytes == 0 ||
        layout->active_element_bytes > 8 || layout->active_token_count > layout->page_capacity_tokens ||
        (layout->page_count != 0 && layout->pages == nullptr))
        return CF_ERR_INVALID_ARGUMENT;
    uint64_t tail_bytes = layout->active_token_count;
    for (uint64_t factor : {static_cast<uint64_t>(layout->layer_count), static_cast<uint64_t>(layout->kv_head_count),
                            static_cast<uint64_t>(layout->head_dim), static_cast<uint64_t>(layout->active_element_bytes)})
        if (!checked_mul(tail_bytes, factor, tail_bytes)) return CF_ERR_UNSUPPORTED;
    if (layout->active_k_bytes < tail_bytes || layout->active_v_bytes < tail_bytes) return CF_ERR_INVALID_ARGUMENT;

    for (uint64_t i = 0; i < layout->page_count; ++i) {
        const cf_kv_page_view &page = layout->pages[i];
        const cf_status status = cf_kv_validate_page(&page);
        if (status != CF_OK) return status;
        if (page.layer >= layout->layer_count || page.kv_head >= layout->kv_head_count || page.head_dim != layout->head_dim ||
            page.token_count > layout->page_capacity_tokens ||
            page.token_begin + page.token_count > layout->active_token_begin)
            return CF_ERR_INVALID_ARGUMENT;
        for (uint64_t j = i + 1; j < layout->page_count; ++j) {
            const cf_kv_page_view &other = layout->pages[j];
            if (other.layer == page.layer && other.kv_head == page.kv_head &&
                intervals_overlap(page.token_begin, page.token_count, other.token_begin, other.token_count))
                return CF_ERR_INVALID_ARGUMENT;
        }
    }
    return CF_OK;
}

extern "C" cf_status cf_kv_page_resident_bytes(const cf_kv_page_view *page, uint64_t *out_bytes) {  // :122-140
    if (!out_bytes) return CF_ERR_INVALID_ARGUMENT;
    const cf_status status = cf_kv_validate_page(page);
    if (status != CF_OK) return status;
    CountedArray arrays[8];
    arrays_of(*page, arrays);
    uint64_t total = 0;
    for (const CountedArray &a : arrays) {
        uint64_t bytes;
        if (!checked_mul(a.count, a.element, bytes) || !checked_add(total, bytes, total)) return CF_ERR_UNSUPPORTED;
    }
    *out_bytes = total;
    return CF_OK;
}

extern "C" cf_status cf_kv_cache_memory_stats(const cf_kv_cache_layout *layout, cf_kv_memory_stats *out_stats) {  // :142-177
    if (!out_stats) return CF_ERR_INVALID_ARGUMENT;
    const cf_status status = cf_kv_validate_layout(layout);
    if (status != CF_OK) return status;
    cf_kv_memory_stats s{};
    s.page_count = layout->page_count;
    s.active_tokens = layout->active_token_count;
    if (!checked_add(layout->active_k_bytes, layout->active_v_bytes, s.active_payload_bytes) ||
        !checked_mul(layout->page_count, sizeof(cf_kv_page_view), s.sealed_descriptor_bytes))
        return CF_ERR_UNSUPPORTED;
    for (uint64_t i = 0; i < layout->page_count; ++i) {
        uint64_t bytes = 0;
        if (cf_kv_page_resident_bytes(&layout->pages[i], &bytes) != CF_OK ||
            !checked_add(s.sealed_payload_bytes, bytes, s.sealed_payload_bytes) ||
            !checked_add(s.sealed_tokens, layout->pages[i].token_count, s.sealed_tokens))
            return CF_ERR_UNSUPPORTED;
    }
    if (!checked_add(s.sealed_payload_bytes, s.sealed_descriptor_bytes, s.total_resident_bytes) ||
        !checked_add(s.total_resident_bytes, s.active_payload_bytes, s.total_resident_bytes))
        return CF_ERR_UNSUPPORTED;
    *out_stats = s;
    return CF_OK;
}

// ---- double-precision online softmax (kv_runtime.cpp:179-253) -------------------------------------------------

extern "C" cf_status cf_online_softmax_init(cf_online_softmax_state *state, double *weighted_values, uint32_t dim) {
    if (!state || !weighted_values || dim == 0 || dim > CF_KV_MAX_HEAD_DIM) return CF_ERR_INVALID_ARGUMENT;
    *state = cf_online_softmax_state{-std::numeric_limits<double>::infinity(), 0.0, weighted_values, dim, 0u};
    std::memset(weighted_values, 0, sizeof(double) * dim);
    return CF_OK;
}

extern "C" cf_status cf_online_softmax_accumulate(cf_online_softmax_state *state, double score, const float *value) {
    if (!state || !state->weighted_values || !value || state->dim == 0 || !std::isfinite(score)) return CF_ERR_INVALID_ARGUMENT;
    double *w = state->weighted_values;
    if (!state->initialized) {
        for (uint32_t d = 0; d < state->dim; ++d) w[d] = value[d];
        state->max_score = score;
        state->exp_sum = 1.0;
        state->initialized = 1;
        return CF_OK;
    }
    const double top = std::fmax(state->max_score, score);
    const double keep = std::exp(state->max_score - top), add = std::exp(score - top);
    for (uint32_t d = 0; d < state->dim; ++d) w[d] = w[d] * keep + static_cast<double>(value[d]) * add;
    state->exp_sum = state->exp_sum * keep + add;
    state->max_score = top;
    return CF_OK;
}

extern "C" cf_status cf_online_softmax_merge(cf_online_softmax_state *dst, const cf_online_softmax_state *src) {
    if (!dst || !src || !dst->weighted_values || !src->weighted_values || dst->dim == 0 || dst->dim != src->dim)
        return CF_ERR_INVALID_ARGUMENT;
    if (!src->initialized) return CF_OK;
    if (!dst->initialized) {
        std::memcpy(dst->weighted_values, src->weighted_values, sizeof(double) * dst->dim);
        dst->max_score = src->max_score;
        dst->exp_sum = src->exp_sum;
        dst->initialized = 1;
        return CF_OK;
    }
    const double top = std::fmax(dst->max_score, src->max_score);
    const double keep = std::exp(dst->max_score - top), add = std::exp(src->max_score - top);
    for (uint32_t d = 0; d < dst->dim; ++d)
        dst->weighted_values[d] = dst->weighted_values[d] * keep + src->weighted_values[d] * add;
    dst->exp_sum = dst->exp_sum * keep + src->exp_sum * add;
    dst->max_score = top;
    return CF_OK;
}

extern "C" cf_status cf_online_softmax_finalize(const cf_online_softmax_state *state, float *out) {
    if (!state || !out || !state->weighted_values || !state->initialized || state->dim == 0 ||
        !std::isfinite(state->exp_sum) || state->exp_sum <= 0.0)
        return CF_ERR_INVALID_ARGUMENT;
    for (uint32_t d = 0; d < state->dim; ++d) out[d] = static_cast<float>(state->weighted_values[d] / state->exp_sum);
    return CF_OK;
}
