// llama_ms_bridge.cpp — libchromofold_b200_llama_ms.so: llama-server's slot <-> sequence bridge over the multi-sequence
// cache of libchromofold_b200.so (integrations/llama.cpp/multisequence/llama_server_multisequence_bridge.cpp).
// A library of its own because four of its symbol names are also names of the llama-server runtime ABI.
//
// Shape of this file: one handle type that owns the cache, the slot table and the last error; one helper, `relay`,
// that takes the lock, runs a call on the cache and records its outcome. Every entry point below is that helper plus,
// for the three slot functions, the bookkeeping of the slot table.
#include <map>
#include <mutex>
#include <new>
#include <string>

#include "chromofold_b200/compat_llama_ms_bridge.h"

extern "C" {   // the cache ABI of the main library (compat_mscache.h cannot be included here: it declares the clashing names)
cf_multisequence_cache *cf_multisequence_create(const cf_multisequence_config *);
void cf_multisequence_destroy(cf_multisequence_cache *, void *);
int cf_sequence_create(cf_multisequence_cache *, int64_t);
int cf_sequence_copy_async(cf_multisequence_cache *, int64_t, int64_t, uint32_t, uint32_t, void *);
int cf_sequence_remove_async(cf_multisequence_cache *, int64_t, int64_t, int64_t, void *);
int cf_sequence_shift_async(cf_multisequence_cache *, int64_t, uint32_t, uint32_t, int32_t, void *);
int cf_multisequence_attention_async(cf_multisequence_cache *, const cf_sequence_attention_item *, uint32_t, void *);
int cf_multisequence_reclaim_async(cf_multisequence_cache *, void *);
int cf_multisequence_audit(const cf_multisequence_cache *);
const char *cf_multisequence_last_error(const cf_multisequence_cache *);
}

struct cf_llama_server_multisequence {
    cf_llama_server_multisequence_config settings{};
    cf_multisequence_cache *cache = nullptr;
    std::map<int64_t, int64_t> slot_table;   // slot id -> sequence id
    mutable std::mutex lock;
    std::string error;

    int outcome(int rc) {   // 0 clears the error text, anything else takes the cache's
        error = rc == 0 ? std::string() : std::string(cf_multisequence_last_error(cache));
        return rc;
    }
    int refuse(const char *why) {
        error = why;
        return -1;
    }
};

namespace {

using Bridge = cf_llama_server_multisequence;

// Lock, call the cache, record the outcome. `call` gets the bridge so that slot functions can touch the slot table.
template <class Call>
int relay(Bridge *bridge, Call &&call) {
    if (bridge == nullptr) return -1;
    std::lock_guard<std::mutex> hold(bridge->lock);
    return call(*bridge);
}

constexpr int64_t kWholeSequence = -1;   // position_begin = position_end = -1 removes everything

}  // namespace

extern "C" Bridge *cf_llama_server_multisequence_create(const cf_llama_server_multisequence_config *config) {
    if (config == nullptr || !config->strict_no_fallback) return nullptr;   // the dense fallback ban must be stated
    Bridge *bridge = new (std::nothrow) Bridge();
    if (bridge == nullptr) return nullptr;
    bridge->settings = *config;
    bridge->cache = cf_multisequence_create(&config->cache);
    if (bridge->cache != nullptr) return bridge;
    delete bridge;
    return nullptr;
}

extern "C" void cf_llama_server_multisequence_destroy(Bridge *bridge, void *stream) {
    if (bridge == nullptr) return;
    relay(bridge, [&](Bridge &b) {
        cf_multisequence_destroy(b.cache, stream);
        b.cache = nullptr;
        b.slot_table.clear();
        return 0;
    });
    delete bridge;
}

extern "C" int cf_llama_server_slot_create(Bridge *bridge, int64_t slot_id, int64_t sequence_id) {
    return relay(bridge, [&](Bridge &b) {
        if (b.slot_table.find(slot_id) != b.slot_table.end()) return b.refuse("slot already exists");
        if (b.outcome(cf_sequence_create(b.cache, sequence_id)) != 0) return -1;
        try {
            b.slot_table[slot_id] = sequence_id;
        } catch (...) {
            return b.refuse("out of host memory");
        }
        return 0;
    });
}

extern "C" int cf_llama_server_slot_reset_async(Bridge *bridge, int64_t slot_id, void *stream) {
    return relay(bridge, [&](Bridge &b) {
        const auto entry = b.slot_table.find(slot_id);
        if (entry == b.slot_table.end()) return b.refuse("slot does not exist");
        if (b.outcome(cf_sequence_remove_async(b.cache, entry->second, kWholeSequence, kWholeSequence, stream)) != 0) return -1;
        b.slot_table.erase(entry);
        return b.outcome(cf_multisequence_reclaim_async(b.cache, stream));   // the slot's pages go back at once
    });
}

extern "C" int cf_llama_server_cancel_sequence_async(Bridge *bridge, int64_t sequence_id, void *stream) {
    return relay(bridge, [&](Bridge &b) {
        for (auto entry = b.slot_table.begin(); entry != b.slot_table.end();) {   // every slot that names the sequence is forgotten
            if (entry->second == sequence_id) entry = b.slot_table.erase(entry);
            else ++entry;
        }
        return b.outcome(cf_sequence_remove_async(b.cache, sequence_id, kWholeSequence, kWholeSequence, stream));
    });
}

extern "C" int cf_llama_server_sequence_copy_async(Bridge *bridge, int64_t source_sequence, int64_t destination_sequence,
                                                   uint32_t token_begin, uint32_t token_end, void *stream) {
    return relay(bridge, [&](Bridge &b) {
        return b.outcome(cf_sequence_copy_async(b.cache, source_sequence, destination_sequence, token_begin, token_end, stream));
    });
}

extern "C" int cf_llama_server_sequence_remove_async(Bridge *bridge, int64_t sequence_id, int64_t position_begin, int64_t position_end,
                                                     void *stream) {
    return relay(bridge, [&](Bridge &b) {
        return b.outcome(cf_sequence_remove_async(b.cache, sequence_id, position_begin, position_end, stream));
    });
}

extern "C" int cf_llama_server_context_shift_async(Bridge *bridge, int64_t sequence_id, uint32_t position_begin, uint32_t position_end,
                                                   int32_t delta, void *stream) {
    return relay(bridge, [&](Bridge &b) {
        return b.outcome(cf_sequence_shift_async(b.cache, sequence_id, position_begin, position_end, delta, stream));
    });
}

extern "C" int cf_llama_server_batch_attention_async(Bridge *bridge, const cf_sequence_attention_item *items, uint32_t item_count,
                                                     void *stream) {
    return relay(bridge, [&](Bridge &b) { return b.outcome(cf_multisequence_attention_async(b.cache, items, item_count, stream)); });
}

extern "C" int cf_llama_server_audit(const Bridge *bridge) {
    if (bridge == nullptr) return -1;
    std::lock_guard<std::mutex> hold(bridge->lock);
    return cf_multisequence_audit(bridge->cache);
}

extern "C" const char *cf_llama_server_multisequence_last_error(const Bridge *bridge) {
    return bridge != nullptr ? bridge->error.c_str() : "null llama-server multisequence bridge";
}
