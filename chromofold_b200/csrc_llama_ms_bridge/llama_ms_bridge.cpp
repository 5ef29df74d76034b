// llama_ms_bridge.cpp — libchromofold_b200_llama_ms.so: llama-server's slot <-> sequence bridge over the multi-sequence
// cache of libchromofold_b200.so (integrations/llama.cpp/multisequence/llama_server_multisequence_bridge.cpp).
// A library of its own because four of its symbol names are also names of the llama-server runtime ABI.
#include <map>
#include <mutex>
#include <new>
#include <string>

#include "chromofold_b200/compat_llama_ms_bridge.h"

// the cache calls this bridge forwards to (declared in compat_mscache.h, which cannot be included here)
extern "C" {
cf_multisequence_cache *cf_multisequence_create(const cf_multisequence_config *config);
void cf_multisequence_destroy(cf_multisequence_cache *cache, void *stream);
int cf_sequence_create(cf_multisequence_cache *cache, int64_t sequence_id);
int cf_sequence_copy_async(cf_multisequence_cache *cache, int64_t source_sequence, int64_t destination_sequence, uint32_t token_begin,
                           uint32_t token_end, void *stream);
int cf_sequence_remove_async(cf_multisequence_cache *cache, int64_t sequence_id, int64_t position_begin, int64_t position_end, void *stream);
int cf_sequence_shift_async(cf_multisequence_cache *cache, int64_t sequence_id, uint32_t position_begin, uint32_t position_end,
                            int32_t delta, void *stream);
int cf_multisequence_attention_async(cf_multisequence_cache *cache, const cf_sequence_attention_item *items, uint32_t item_count, void *stream);
int cf_multisequence_reclaim_async(cf_multisequence_cache *cache, void *stream);
int cf_multisequence_audit(const cf_multisequence_cache *cache);
const char *cf_multisequence_last_error(const cf_multisequence_cache *cache);
}

struct cf_llama_server_multisequence {
    cf_llama_server_multisequence_config config{};
    cf_multisequence_cache *cache = nullptr;
    std::map<int64_t, int64_t> sequence_of_slot;
    mutable std::mutex lock;
    std::string error;

    // result of a cache call: 0 clears the error text, anything else copies the cache's
    int pass(int rc) {
        if (rc == 0) error.clear();
        else error = cf_multisequence_last_error(cache);
        return rc;
    }
    int refuse(const char *why) {
        error = why;
        return -1;
    }
};

using Guard = std::lock_guard<std::mutex>;

extern "C" cf_llama_server_multisequence *cf_llama_server_multisequence_create(const cf_llama_server_multisequence_config *config) {
    if (!config || config->strict_no_fallback == 0) return nullptr;
    cf_llama_server_multisequence *bridge = new (std::nothrow) cf_llama_server_multisequence();
    if (!bridge) return nullptr;
    bridge->config = *config;
    bridge->cache = cf_multisequence_create(&config->cache);
    if (!bridge->cache) {
        delete bridge;
        return nullptr;
    }
    return bridge;
}

extern "C" void cf_llama_server_multisequence_destroy(cf_llama_server_multisequence *bridge, void *stream) {
    if (!bridge) return;
    {
        Guard g(bridge->lock);
        cf_multisequence_destroy(bridge->cache, stream);
        bridge->cache = nullptr;
        bridge->sequence_of_slot.clear();
    }
    delete bridge;
}

extern "C" int cf_llama_server_slot_create(cf_llama_server_multisequence *bridge, int64_t slot_id, int64_t sequence_id) {
    if (!bridge) return -1;
    Guard g(bridge->lock);
    if (bridge->sequence_of_slot.count(slot_id)) return bridge->refuse("slot already exists");
    if (bridge->pass(cf_sequence_create(bridge->cache, sequence_id)) != 0) return -1;
    try {
        bridge->sequence_of_slot.emplace(slot_id, sequence_id);
    } catch (...) {
        return bridge->refuse("out of host memory");
    }
    return 0;
}

extern "C" int cf_llama_server_slot_reset_async(cf_llama_server_multisequence *bridge, int64_t slot_id, void *stream) {
    if (!bridge) return -1;
    Guard g(bridge->lock);
    auto slot = bridge->sequence_of_slot.find(slot_id);
    if (slot == bridge->sequence_of_slot.end()) return bridge->refuse("slot does not exist");
    if (bridge->pass(cf_sequence_remove_async(bridge->cache, slot->second, -1, -1, stream)) != 0) return -1;   // the whole sequence
    bridge->sequence_of_slot.erase(slot);
    return bridge->pass(cf_multisequence_reclaim_async(bridge->cache, stream));
}

extern "C" int cf_llama_server_sequence_copy_async(cf_llama_server_multisequence *bridge, int64_t source_sequence, int64_t destination_sequence,
                                                   uint32_t token_begin, uint32_t token_end, void *stream) {
    if (!bridge) return -1;
    Guard g(bridge->lock);
    return bridge->pass(cf_sequence_copy_async(bridge->cache, source_sequence, destination_sequence, token_begin, token_end, stream));
}

extern "C" int cf_llama_server_sequence_remove_async(cf_llama_server_multisequence *bridge, int64_t sequence_id, int64_t position_begin,
                                                     int64_t position_end, void *stream) {
    if (!bridge) return -1;
    Guard g(bridge->lock);
    return bridge->pass(cf_sequence_remove_async(bridge->cache, sequence_id, position_begin, position_end, stream));
}

extern "C" int cf_llama_server_context_shift_async(cf_llama_server_multisequence *bridge, int64_t sequence_id, uint32_t position_begin,
                                                   uint32_t position_end, int32_t delta, void *stream) {
    if (!bridge) return -1;
    Guard g(bridge->lock);
    return bridge->pass(cf_sequence_shift_async(bridge->cache, sequence_id, position_begin, position_end, delta, stream));
}

extern "C" int cf_llama_server_cancel_sequence_async(cf_llama_server_multisequence *bridge, int64_t sequence_id, void *stream) {
    if (!bridge) return -1;
    Guard g(bridge->lock);
    for (auto it = bridge->sequence_of_slot.begin(); it != bridge->sequence_of_slot.end();)   // every slot that names it is forgotten
        it = it->second == sequence_id ? bridge->sequence_of_slot.erase(it) : std::next(it);
    return bridge->pass(cf_sequence_remove_async(bridge->cache, sequence_id, -1, -1, stream));
}

extern "C" int cf_llama_server_batch_attention_async(cf_llama_server_multisequence *bridge, const cf_sequence_attention_item *items,
                                                     uint32_t item_count, void *stream) {
    if (!bridge) return -1;
    Guard g(bridge->lock);
    return bridge->pass(cf_multisequence_attention_async(bridge->cache, items, item_count, stream));
}

extern "C" int cf_llama_server_audit(const cf_llama_server_multisequence *bridge) {
    if (!bridge) return -1;
    Guard g(bridge->lock);
    return cf_multisequence_audit(bridge->cache);
}

extern "C" const char *cf_llama_server_multisequence_last_error(const cf_llama_server_multisequence *bridge) {
    return bridge ? bridge->error.c_str() : "null llama-server multisequence bridge";
}
