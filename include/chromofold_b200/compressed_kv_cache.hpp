// compressed_kv_cache.hpp — the reference's C++ cache class (include/chromofold/compressed_kv_cache.hpp:13-84) as a
// header-only front of this library's adapter ABI (compat_adapter.h): same namespace, class name, configuration and
// statistics structs, method names, argument meaning and exception types, so that code written against the
// reference's class compiles against this header and links libchromofold_b200.so.
//   chromofold::CompressedKvCache cache({layers, kv_heads, query_heads, head_dim, page_size, group});
//   cache.append(layer, kv_head, token_begin, host_keys, host_values, token_count);   // fp32 [token][dim], host memory
//   cache.attention(layer, q_device, out_device, query_count, query_token_begin, softmax_scale, causal_window);
// Kept: append is per (layer, kv head), contiguous in token positions (std::invalid_argument otherwise); a layer / head
// out of range is std::out_of_range; a bad configuration is std::invalid_argument; only sequence 0 exists
// (remove_sequence of another id, a copy to another id and a non-zero shift throw, compressed_kv_cache.cu:180-192);
// move-only; nothing is thrown from the destructor.
// Different: pages are sealed on the GPU the moment a page of every kv head of a layer is full, so seal_full_pages()
// has nothing left to do and returns; the codec is int8 symbols under the store's entropy coder (KvCodecMode is
// accepted and ignored, as the adapter ignores it for kv_bits 8); and there is no attention_view(): that call hands out
// the reference's own page descriptors (cf_kv_device_page), which sealed format-v1 pages do not have. attention() and
// attention_host() take its place: they run what the reference's callers do with the view
// (integrations/llama.cpp/chromofold_kv_adapter.cpp:96-130).
#ifndef CHROMOFOLD_COMPRESSED_KV_CACHE_HPP   /* the reference header's guard: whichever comes first wins */
#define CHROMOFOLD_COMPRESSED_KV_CACHE_HPP
#define CHROMOFOLD_B200_COMPRESSED_KV_CACHE_HPP

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>

#include "chromofold_b200/compat_adapter.h"

namespace chromofold {

enum class KvCodecMode : std::uint32_t { fixed_int4_huffman = 0, adaptive_huffman = 1, fixed_int8_huffman = 2 };

struct KvCacheConfig {
    std::uint32_t layer_count = 0;
    std::uint32_t kv_head_count = 0;
    std::uint32_t query_head_count = 0;
    std::uint32_t head_dim = 0;
    std::uint32_t page_size = 128;
    std::uint32_t gqa_group_size = 1;
    KvCodecMode codec = KvCodecMode::fixed_int8_huffman;
};

struct KvCacheStats {
    std::uint64_t appended_tokens = 0;
    std::uint64_t sealed_tokens = 0;
    std::uint64_t sealed_pages = 0;
    std::uint64_t active_tokens = 0;
    std::uint64_t dense_active_bytes = 0;
    std::uint64_t compressed_bytes = 0;
    std::uint64_t descriptor_bytes = 0;
};

class CompressedKvCache {
public:
    explicit CompressedKvCache(KvCacheConfig config) : config_(config) {
        cf_llama_kv_options o{};
        o.struct_size = sizeof o;
        o.backend = CF_LLAMA_KV_BACKEND_CHROMOFOLD;
        o.layer_count = config.layer_count;
        o.kv_head_count = config.kv_head_count;
        o.query_head_count = config.query_head_count;
        o.head_dim = config.head_dim;
        o.page_size = config.page_size;
        o.gqa_group_size = config.gqa_group_size;
        o.kv_bits = 8;
        if (cf_llama_kv_options_validate(&o) != 0 || config.head_dim > 128)   // 128 = CF_KV_MAX_HEAD_DIM (compressed_kv_cache.cu:29-36)
            throw std::invalid_argument("invalid compressed KV cache configuration");
        adapter_ = cf_llama_kv_create(&o);
        if (!adapter_) throw std::runtime_error("the compressed KV cache could not be created on this device");
    }
    CompressedKvCache(const CompressedKvCache &) = delete;
    CompressedKvCache &operator=(const CompressedKvCache &) = delete;
    CompressedKvCache(CompressedKvCache &&other) noexcept : adapter_(other.adapter_), config_(other.config_) { other.adapter_ = nullptr; }
    CompressedKvCache &operator=(CompressedKvCache &&other) noexcept {
        if (this != &other) {
            release();
            adapter_ = other.adapter_;
            config_ = other.config_;
            other.adapter_ = nullptr;
        }
        return *this;
    }
    ~CompressedKvCache() { release(); }

    void append(std::uint32_t layer, std::uint32_t kv_head, std::uint32_t token_begin, const float *keys, const float *values,
                std::uint32_t token_count, void *stream = nullptr) {
        if (!keys || !values || token_count == 0) throw std::invalid_argument("invalid KV append");
        if (layer >= config_.layer_count || kv_head >= config_.kv_head_count) throw std::out_of_range("KV layer/head out of range");
        if (cf_llama_kv_append(live(), layer, kv_head, token_begin, keys, values, token_count, stream) != 0)
            throw std::invalid_argument(error_text());
    }
    void seal_full_pages(void * /*stream*/ = nullptr) { live(); }   // full pages were sealed when they filled up
    void flush(void *stream = nullptr) {
        if (cf_llama_kv_flush(live(), stream) != 0) throw std::runtime_error(error_text());
    }
    // Decode attention of `query_count` query tokens at positions query_token_begin.. over the layer's sealed pages and
    // its active tail; queries [query][query head][dim] and output are fp32 in device memory.
    void attention(std::uint32_t layer, const float *queries_device, float *output_device, std::uint32_t query_count,
                   std::uint32_t query_token_begin, float softmax_scale, std::uint32_t causal_window = 0, void *stream = nullptr) {
        if (layer >= config_.layer_count) throw std::out_of_range("KV layer out of range");
        if (cf_llama_kv_attention(live(), layer, queries_device, output_device, query_count, config_.query_head_count,
                                  config_.gqa_group_size, query_token_begin, softmax_scale, causal_window, stream) != 0)
            throw std::runtime_error(error_text());
    }
    // The same with queries and output in host memory; returns when the output is there.
    void attention_host(std::uint32_t layer, const float *queries, float *output, std::uint32_t query_count,
                        std::uint32_t query_token_begin, float softmax_scale, std::uint32_t causal_window = 0, void *stream = nullptr) {
        if (layer >= config_.layer_count) throw std::out_of_range("KV layer out of range");
        if (cf_llama_kv_attention_host(live(), layer, queries, output, query_count, config_.query_head_count, config_.gqa_group_size,
                                       query_token_begin, softmax_scale, causal_window, stream) != 0)
            throw std::runtime_error(error_text());
    }

    void remove_sequence(std::uint64_t sequence_id) {
        if (cf_llama_kv_seq_rm(live(), sequence_id) != 0) throw std::invalid_argument(error_text());
    }
    void copy_sequence(std::uint64_t source_sequence_id, std::uint64_t destination_sequence_id) {
        if (cf_llama_kv_seq_cp(live(), source_sequence_id, destination_sequence_id) != 0) throw std::runtime_error(error_text());
    }
    void shift_sequence(std::uint64_t sequence_id, std::int32_t delta) {
        if (cf_llama_kv_seq_shift(live(), sequence_id, delta) != 0) throw std::runtime_error(error_text());
    }
    void clear() {
        if (cf_llama_kv_clear(live()) != 0) throw std::runtime_error(error_text());
    }

    const KvCacheConfig &config() const noexcept { return config_; }
    KvCacheStats stats() const noexcept {
        KvCacheStats out;
        cf_llama_kv_stats s{};
        if (adapter_ && cf_llama_kv_get_stats(adapter_, &s) == 0) {
            out.appended_tokens = s.appended_tokens;
            out.sealed_tokens = s.sealed_tokens;
            out.sealed_pages = s.sealed_pages;
            out.active_tokens = s.active_tokens;
            out.dense_active_bytes = s.dense_active_bytes;
            out.compressed_bytes = s.compressed_bytes;
            out.descriptor_bytes = s.descriptor_bytes;
        }
        return out;
    }

private:
    cf_llama_kv_adapter *live() const {
        if (!adapter_) throw std::runtime_error("the compressed KV cache was moved from");
        return adapter_;
    }
    std::string error_text() const { return cf_llama_kv_last_error(adapter_); }
    void release() noexcept {
        if (adapter_) cf_llama_kv_destroy(adapter_);
        adapter_ = nullptr;
    }
    cf_llama_kv_adapter *adapter_ = nullptr;
    KvCacheConfig config_;
};

}  // namespace chromofold

#endif
