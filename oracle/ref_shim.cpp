// ref_shim.cpp — flat C entry points over the reference's own C++ CPU sources, so that Python tests and the
// golden-vector generator can call them. TEST INFRASTRUCTURE ONLY. This file contains no reference code; it is
// compiled together with the reference's src/runtime/{kv_reference,kv_gpu_fixture,kv_runtime}.cpp, taken from
// where they lie, into oracle/_ref/libcfref_cpu.so (see oracle/Makefile).

#include <algorithm>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "chromofold/kv_gpu_fixture.hpp"
#include "chromofold/kv_reference.hpp"

// The decoder header is device code; on the host the two CUDA qualifiers are defined away.
#define __device__
#define __forceinline__ inline
#include "chromofold/detail/block_huffman_device.cuh"

namespace ref = chromofold::reference;
namespace fix = chromofold::gpu_fixture;

extern "C" {

int ref_bh_decode_at(const uint32_t *words, const int *lut, int maxlen, int pos) {
    return cf_bh_decode_at(words, lut, maxlen, pos);
}

// gpu_fixture::encode_int{4,8}_page. Output arrays are sized by the caller:
//   words: ceil(tokens*dim*bits/32), offsets: ceil(tokens*dim/block), lut: 2^bits, k_scales: dim, v_scales: tokens,
//   dequantized_*: tokens*dim. Returns 0, or 1 if the reference threw.
int ref_fixture_encode(const float *keys, const float *values, uint32_t token_begin, uint32_t token_count,
                       uint32_t head_dim, uint32_t kv_head, uint32_t block_size, uint32_t bits, uint32_t *k_words,
                       int32_t *k_offsets, uint32_t *v_words, int32_t *v_offsets, int32_t *lut, float *k_scales,
                       float *v_scales, float *dequantized_k, float *dequantized_v, uint64_t *resident_bytes) {
    try {
        const size_t count = static_cast<size_t>(token_count) * head_dim;
        const std::vector<float> k(keys, keys + count), v(values, values + count);
        const fix::EncodedKvPage page = bits == 8
            ? fix::encode_int8_page(k, v, token_begin, token_count, head_dim, kv_head, block_size)
            : fix::encode_int4_page(k, v, token_begin, token_count, head_dim, kv_head, block_size);
        std::memcpy(k_words, page.k.words.data(), page.k.words.size() * 4);
        std::memcpy(v_words, page.v.words.data(), page.v.words.size() * 4);
        std::memcpy(k_offsets, page.k.block_offsets.data(), page.k.block_offsets.size() * 4);
        std::memcpy(v_offsets, page.v.block_offsets.data(), page.v.block_offsets.size() * 4);
        std::memcpy(lut, page.k.lut.data(), page.k.lut.size() * 4);
        std::memcpy(k_scales, page.k_scales.data(), page.k_scales.size() * 4);
        std::memcpy(v_scales, page.v_scales.data(), page.v_scales.size() * 4);
        std::memcpy(dequantized_k, page.dequantized_k.data(), count * 4);
        std::memcpy(dequantized_v, page.dequantized_v.data(), count * 4);
        if (resident_bytes) *resident_bytes = page.resident_bytes();
        return 0;
    } catch (const std::exception &) {
        return 1;
    }
}

// gpu_fixture::decode_symbols on a fixed-width stream.
int ref_fixture_decode(const uint32_t *words, uint64_t word_count, uint32_t bits, uint64_t symbol_count, uint8_t *out) {
    try {
        fix::EncodedStream s;
        s.words.assign(words, words + word_count);
        s.max_code_length = bits;
        s.lut.resize(1u << bits);
        const auto r = fix::decode_symbols(s, symbol_count);
        std::memcpy(out, r.data(), r.size());
        return 0;
    } catch (const std::exception &) {
        return 1;
    }
}

// reference::paged_attention fed with dense rows as active tails (quantiser-agnostic route).
//   keys/values: [kv_head_count][token_count][head_dim], one tail per kv head covering tokens token_begin...
// Returns 0, 1 for std::invalid_argument, 2 for anything else.
int ref_paged_attention_dense(const float *keys, const float *values, uint32_t token_begin, uint32_t token_count,
                              const float *queries, uint32_t query_count, uint32_t query_head_count,
                              uint32_t kv_head_count, uint32_t head_dim, uint32_t query_token_begin,
                              uint32_t causal_window, float score_scale, float *output) {
    try {
        std::vector<ref::ActiveKvTail> tails;
        for (uint32_t h = 0; h < kv_head_count; ++h) {
            tails.push_back(ref::ActiveKvTail{token_begin, token_count, 0, h, head_dim,
                                              keys + static_cast<size_t>(h) * token_count * head_dim,
                                              values + static_cast<size_t>(h) * token_count * head_dim});
        }
        ref::AttentionShape shape{query_count, query_head_count, kv_head_count, head_dim, query_token_begin,
                                  causal_window, score_scale};
        std::vector<float> out;
        ref::paged_attention({}, tails, queries, shape, &out);
        std::memcpy(output, out.data(), out.size() * 4);
        return 0;
    } catch (const std::invalid_argument &) {
        return 1;
    } catch (const std::exception &) {
        return 2;
    }
}

// reference::seal_int4_page + paged_attention over sealed int4 pages plus one fp32 tail per kv head.
//   sealed rows: [kv_head_count][sealed_tokens][head_dim], cut into pages of page_sizes[i] tokens;
//   tail rows  : [kv_head_count][tail_tokens][head_dim] starting at token sealed_tokens.
// Also returns the dequantised sealed rows so that a caller can replay the same numbers elsewhere.
int ref_paged_attention_int4(const float *keys, const float *values, uint32_t sealed_tokens,
                             const uint32_t *page_sizes, uint32_t page_count, const float *tail_keys,
                             const float *tail_values, uint32_t tail_tokens, const float *queries,
                             uint32_t query_count, uint32_t query_head_count, uint32_t kv_head_count,
                             uint32_t head_dim, uint32_t query_token_begin, uint32_t causal_window,
                             float score_scale, int reverse_pages, float *output, float *dequantized_k,
                             float *dequantized_v) {
    try {
        std::vector<ref::SealedKvPage> pages;
        std::vector<ref::ActiveKvTail> tails;
        for (uint32_t h = 0; h < kv_head_count; ++h) {
            uint32_t begin = 0;
            for (uint32_t p = 0; p < page_count; ++p) {
                const size_t off = (static_cast<size_t>(h) * sealed_tokens + begin) * head_dim;
                pages.push_back(ref::seal_int4_page(keys + off, values + off, begin, page_sizes[p], 0, h, head_dim));
                std::vector<float> dk, dv;
                ref::dequantize_page(pages.back(), &dk, &dv);
                if (dequantized_k) std::memcpy(dequantized_k + off, dk.data(), dk.size() * 4);
                if (dequantized_v) std::memcpy(dequantized_v + off, dv.data(), dv.size() * 4);
                begin += page_sizes[p];
            }
            if (tail_tokens) {
                tails.push_back(ref::ActiveKvTail{sealed_tokens, tail_tokens, 0, h, head_dim,
                                                  tail_keys + static_cast<size_t>(h) * tail_tokens * head_dim,
                                                  tail_values + static_cast<size_t>(h) * tail_tokens * head_dim});
            }
        }
        if (reverse_pages) std::vector<ref::SealedKvPage>(pages.rbegin(), pages.rend()).swap(pages);
        ref::AttentionShape shape{query_count, query_head_count, kv_head_count, head_dim, query_token_begin,
                                  causal_window, score_scale};
        std::vector<float> out;
        ref::paged_attention(pages, tails, queries, shape, &out);
        std::memcpy(output, out.data(), out.size() * 4);
        return 0;
    } catch (const std::invalid_argument &) {
        return 1;
    } catch (const std::exception &) {
        return 2;
    }
}

// A sequence sealed once with reference::seal_int4_page, attended many times with reference::paged_attention
// (the timed part of the CPU baseline). keys/values: [kv_head_count][tokens][head_dim], cut into page_tokens pages.
struct RefCache {
    std::vector<ref::SealedKvPage> pages;
    uint32_t kv_head_count, head_dim, tokens;
};

void *ref_cache_create(const float *keys, const float *values, uint32_t tokens, uint32_t page_tokens,
                       uint32_t kv_head_count, uint32_t head_dim) {
    try {
        auto *c = new RefCache{{}, kv_head_count, head_dim, tokens};
        for (uint32_t h = 0; h < kv_head_count; ++h) {
            for (uint32_t begin = 0; begin < tokens; begin += page_tokens) {
                const uint32_t count = std::min(page_tokens, tokens - begin);
                const size_t off = (static_cast<size_t>(h) * tokens + begin) * head_dim;
                c->pages.push_back(ref::seal_int4_page(keys + off, values + off, begin, count, 0, h, head_dim));
            }
        }
        return c;
    } catch (const std::exception &) {
        return nullptr;
    }
}

int ref_cache_attention(const void *cache, const float *queries, uint32_t query_head_count, uint32_t causal_window,
                        float score_scale, float *output) {
    try {
        const auto *c = static_cast<const RefCache *>(cache);
        ref::AttentionShape shape{1, query_head_count, c->kv_head_count, c->head_dim, c->tokens, causal_window, score_scale};
        std::vector<float> out;
        ref::paged_attention(c->pages, {}, queries, shape, &out);
        std::memcpy(output, out.data(), out.size() * 4);
        return 0;
    } catch (const std::invalid_argument &) {
        return 1;
    } catch (const std::exception &) {
        return 2;
    }
}

uint64_t ref_cache_bytes(const void *cache) {
    uint64_t total = 0;
    for (const auto &p : static_cast<const RefCache *>(cache)->pages) total += p.resident_bytes();
    return total;
}

void ref_cache_destroy(void *cache) { delete static_cast<RefCache *>(cache); }

}  // extern "C"
