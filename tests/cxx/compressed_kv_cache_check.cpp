// Exercises chromofold::CompressedKvCache (include/chromofold_b200/compressed_kv_cache.hpp) the way the reference's
// tests/adapter_attention_test.cu drives its class. Built and run by tests/test_cxx_cache.py.
//   contract : configuration checks and exception types; needs no GPU
//   gpu      : append / stats / attention through the class equal the same calls on the adapter ABI, bit for bit
#include <cmath>
#include <cstdio>
#include <cstring>
#include <random>
#include <vector>

#include "chromofold_b200/compressed_kv_cache.hpp"

#define CHECK(cond)                                                   \
    do {                                                              \
        if (!(cond)) {                                                \
            std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, #cond); \
            return 1;                                                 \
        }                                                             \
    } while (0)

template <class Exception, class F>
static bool throws(F &&f) {
    try {
        f();
    } catch (const Exception &) {
        return true;
    } catch (...) {
        return false;
    }
    return false;
}

static int contract() {
    using namespace chromofold;
    KvCacheConfig bad;                       // all zero
    CHECK(throws<std::invalid_argument>([&] { CompressedKvCache c(bad); }));
    KvCacheConfig gqa{2, 2, 7, 64, 32, 4};   // 7 query heads over 2 kv heads x 4
    CHECK(throws<std::invalid_argument>([&] { CompressedKvCache c(gqa); }));
    KvCacheConfig wide{1, 1, 1, 256, 32, 1}; // beyond CF_KV_MAX_HEAD_DIM
    CHECK(throws<std::invalid_argument>([&] { CompressedKvCache c(wide); }));
    static_assert(!std::is_copy_constructible<CompressedKvCache>::value && std::is_move_constructible<CompressedKvCache>::value, "move-only");
    std::puts("contract ok");
    return 0;
}

static int gpu() {
    using namespace chromofold;
    const uint32_t layers = 2, hkv = 2, hq = 8, dim = 64, page = 32, tokens = 70, nq = 3;
    KvCacheConfig cfg{layers, hkv, hq, dim, page, hq / hkv};
    CompressedKvCache cache(cfg);
    cf_llama_kv_options o{};
    o.struct_size = sizeof o;
    o.backend = CF_LLAMA_KV_BACKEND_CHROMOFOLD;
    o.layer_count = layers; o.kv_head_count = hkv; o.query_head_count = hq; o.head_dim = dim; o.page_size = page;
    o.gqa_group_size = hq / hkv; o.kv_bits = 8;
    cf_llama_kv_adapter *direct = cf_llama_kv_create(&o);
    CHECK(direct != nullptr);
    std::mt19937 rng(7);
    std::normal_distribution<float> normal;
    std::vector<float> k(static_cast<size_t>(tokens) * dim), v(k.size());
    for (uint32_t layer = 0; layer < layers; ++layer)
        for (uint32_t h = 0; h < hkv; ++h) {
            for (auto &x : k) x = normal(rng);
            for (auto &x : v) x = normal(rng);
            cache.append(layer, h, 0, k.data(), v.data(), 50);
            cache.append(layer, h, 50, k.data() + 50 * dim, v.data() + 50 * dim, 20);
            CHECK(cf_llama_kv_append(direct, layer, h, 0, k.data(), v.data(), tokens, nullptr) == 0);
        }
    CHECK(throws<std::invalid_argument>([&] { cache.append(0, 0, 99, k.data(), v.data(), 1); }));   // not contiguous
    CHECK(throws<std::invalid_argument>([&] { cache.append(0, 0, tokens, nullptr, v.data(), 1); }));
    CHECK(throws<std::out_of_range>([&] { cache.append(layers, 0, tokens, k.data(), v.data(), 1); }));
    CHECK(throws<std::out_of_range>([&] { cache.append(0, hkv, tokens, k.data(), v.data(), 1); }));
    cache.seal_full_pages();
    const KvCacheStats s = cache.stats();
    CHECK(s.appended_tokens == uint64_t(layers) * hkv * tokens && s.sealed_pages == uint64_t(layers) * hkv * 2);
    CHECK(s.sealed_tokens == uint64_t(layers) * hkv * 64 && s.active_tokens == uint64_t(layers) * hkv * 6);
    CHECK(s.compressed_bytes > 0 && s.compressed_bytes < uint64_t(layers) * hkv * 64 * dim * 2 * 2);

    std::vector<float> q(static_cast<size_t>(nq) * hq * dim), a(q.size()), b(q.size());
    for (auto &x : q) x = normal(rng);
    const float scale = 1.0f / std::sqrt(static_cast<float>(dim));
    for (uint32_t layer = 0; layer < layers; ++layer) {
        cache.attention_host(layer, q.data(), a.data(), nq, tokens - nq, scale, 40);
        CHECK(cf_llama_kv_attention_host(direct, layer, q.data(), b.data(), nq, hq, hq / hkv, tokens - nq, scale, 40, nullptr) == 0);
        CHECK(std::memcmp(a.data(), b.data(), a.size() * sizeof(float)) == 0);
        double norm = 0;
        for (float x : a) norm += double(x) * x;
        CHECK(norm > 0 && std::isfinite(norm));
    }
    CHECK(throws<std::out_of_range>([&] { cache.attention_host(layers, q.data(), a.data(), nq, tokens - nq, scale); }));
    CompressedKvCache moved(std::move(cache));
    CHECK(throws<std::runtime_error>([&] { cache.flush(); }));                     // moved from
    moved.flush();
    CHECK(moved.stats().active_tokens == 0 && moved.stats().sealed_pages == uint64_t(layers) * hkv * 3);
    CHECK(throws<std::runtime_error>([&] { moved.copy_sequence(0, 1); }));
    CHECK(throws<std::runtime_error>([&] { moved.shift_sequence(0, 1); }));
    CHECK(throws<std::invalid_argument>([&] { moved.remove_sequence(1); }));
    moved.shift_sequence(0, 0);
    moved.remove_sequence(0);
    CHECK(moved.stats().appended_tokens == 0);
    moved.append(0, 0, 0, k.data(), v.data(), 4);                                  // usable after the removal
    moved.clear();
    cf_llama_kv_destroy(direct);
    std::puts("gpu ok");
    return 0;
}

int main(int argc, char **argv) {
    if (argc == 2 && !std::strcmp(argv[1], "contract")) return contract();
    if (argc == 2 && !std::strcmp(argv[1], "gpu")) return gpu();
    std::fprintf(stderr, "usage: %s contract|gpu\n", argv[0]);
    return 2;
}
