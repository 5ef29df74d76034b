// ms_host_cache.cpp — the reference's multi-sequence cache ABI (include/chromofold/multisequence_cache.h:65-112,
// src/multisequence_cache.cpp) and its llama-server runtime ABI (include/chromofold/llama_server_runtime.h:58-86,
// src/llama_server_runtime.cpp), as fronts of this library's device sequence store (ms_resolver.cu). Declared in
// include/chromofold_b200/compat_mscache.h, which says what is kept and what is narrower.
//
// Host code only: every byte of K/V is moved, sealed and attended by the kernels behind cf_ms_cuda_* / cf_b200_ms_*.

#include <algorithm>
#include <cmath>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <stdexcept>
#include <string>
#include <unordered_set>
#include <vector>

#include "chromofold_b200/compat_mscache.h"

static_assert(sizeof(cf_sequence_attention_item) == sizeof(cf_ms_batch_item), "the two batch item layouts are one");

namespace {

struct Speculation {
    cf_speculation_id id = 0;
    uint32_t baseline_tokens = 0;
    bool active = false;
};
struct SequenceState {
    Speculation speculation;
    // Logical position of the first token the device store holds for this sequence. The store keeps a sequence's tokens
    // contiguous from its token 0; a copy of a range that starts later, or a context shift of the whole sequence, only
    // moves this offset (sealed records carry no position).
    uint32_t base = 0;
};

bool valid_config(const cf_multisequence_config &c) {
    return c.layer_count > 0 && c.kv_head_count > 0 && c.query_head_count > 0 && c.head_dim > 0 && c.page_size > 0 &&
           c.gqa_group_size > 0 && c.query_head_count == c.kv_head_count * c.gqa_group_size;
}

}  // namespace

struct cf_multisequence_cache {
    cf_multisequence_config config{};
    mutable std::mutex mutex;
    cf_ms_cuda_resolver *device = nullptr;
    std::map<int64_t, SequenceState> sequences;
    mutable cf_multisequence_counters counters{};
    cf_speculation_id next_speculation_id = 1;
    uint64_t mutations_since_audit = 0;
    std::string last_error;
};

namespace {

struct Unsupported : std::runtime_error {
    using std::runtime_error::runtime_error;
};

void device_check(cf_multisequence_cache *c, int rc) {
    if (rc != 0) throw std::runtime_error(cf_ms_cuda_last_error(c->device));
}

SequenceState &find(cf_multisequence_cache *c, int64_t id, const char *what = "sequence does not exist") {
    auto it = c->sequences.find(id);
    if (it == c->sequences.end()) throw std::runtime_error(what);
    return it->second;
}

// Sealed tokens of the sequence's longest layer.
uint32_t sealed_tokens(cf_multisequence_cache *c, int64_t id) {
    uint32_t most = 0;
    for (uint32_t layer = 0; layer < c->config.layer_count; ++layer) {
        uint32_t sealed = 0, active = 0;
        if (cf_b200_ms_sequence_tokens(c->device, id, layer, &sealed, &active) != 0) throw std::runtime_error("sequence does not exist");
        most = std::max(most, sealed);
    }
    return most;
}

// Longest layer of the sequence, in tokens (sealed + active).
uint32_t total_tokens(cf_multisequence_cache *c, int64_t id) {
    uint32_t total = 0;
    for (uint32_t layer = 0; layer < c->config.layer_count; ++layer) {
        uint32_t sealed = 0, active = 0;
        if (cf_b200_ms_sequence_tokens(c->device, id, layer, &sealed, &active) != 0) throw std::runtime_error("sequence does not exist");
        total = std::max(total, sealed + active);
    }
    return total;
}

void seal_full_tails(cf_multisequence_cache *c, int64_t id, void *stream) {
    for (uint32_t layer = 0; layer < c->config.layer_count; ++layer) {
        uint32_t sealed = 0, active = 0;
        cf_b200_ms_sequence_tokens(c->device, id, layer, &sealed, &active);
        if (active == c->config.page_size) device_check(c, cf_b200_ms_seal_active_async(c->device, id, layer, stream));
    }
}

void update_active_peak(cf_multisequence_cache *c) {
    c->counters.active_sequences = c->sequences.size();
    c->counters.active_sequences_peak = std::max(c->counters.active_sequences_peak, c->counters.active_sequences);
}

// The audit walks every page, so running it after every mutation would make filling a cache quadratic in its size: it
// runs after every mutation while the cache is small, and once per (pages / 64) mutations beyond that.
void maybe_audit(cf_multisequence_cache *c) {
    if (!c->config.enable_invariant_auditor) return;
    uint64_t pages_in_use = 0;
    cf_b200_ms_arena_stats(c->device, &pages_in_use, nullptr, nullptr, nullptr, nullptr);
    if (++c->mutations_since_audit * 64u < pages_in_use) return;
    c->mutations_since_audit = 0;
    ++c->counters.invariant_audits;
    if (cf_ms_cuda_audit(c->device) != 0) {
        ++c->counters.invariant_failures;
        throw std::runtime_error("multisequence invariant audit failed");
    }
}

template <class F>
int guarded(cf_multisequence_cache *c, F &&body) {
    std::lock_guard<std::mutex> guard(c->mutex);
    try {
        body();
        c->last_error.clear();
        return 0;
    } catch (const Unsupported &e) {
        ++c->counters.unsupported_operations;
        c->last_error = e.what();
    } catch (const std::exception &e) {
        c->last_error = e.what();
    }
    return -1;
}

}  // namespace

extern "C" cf_multisequence_cache *cf_multisequence_create(const cf_multisequence_config *config) {
    if (!config || !valid_config(*config)) return nullptr;
    try {
        auto cache = std::make_unique<cf_multisequence_cache>();
        cache->config = *config;
        cf_ms_cuda_config device{};
        device.layer_count = config->layer_count;
        device.kv_head_count = config->kv_head_count;
        device.query_head_count = config->query_head_count;
        device.head_dim = config->head_dim;
        device.page_size = config->page_size;
        device.gqa_group_size = config->gqa_group_size;
        device.use_async_allocator = config->use_async_allocator;
        cache->device = cf_ms_cuda_create(&device);   // no CUDA call yet: device memory is taken on first use
        if (!cache->device) return nullptr;
        return cache.release();
    } catch (...) {
        return nullptr;
    }
}

extern "C" void cf_multisequence_destroy(cf_multisequence_cache *cache, void *stream) {
    if (!cache) return;
    if (cache->device) cf_ms_cuda_destroy(cache->device, stream);
    delete cache;
}

extern "C" int cf_sequence_create(cf_multisequence_cache *c, int64_t id) {
    if (!c) return -1;
    return guarded(c, [&] {
        if (c->sequences.count(id)) throw std::runtime_error("sequence already exists");
        device_check(c, cf_ms_cuda_sequence_create(c->device, id));
        c->sequences.emplace(id, SequenceState{});
        ++c->counters.sequences_created;
        update_active_peak(c);
        maybe_audit(c);
    });
}

extern "C" int cf_sequence_copy_async(cf_multisequence_cache *c, int64_t source, int64_t destination, uint32_t token_begin,
                                      uint32_t token_end, void *stream) {
    if (!c || source == destination || token_end < token_begin) return -1;
    return guarded(c, [&] {
        // src/multisequence_cache.cpp:235-292: the destination gets the sealed pages that lie wholly inside
        // [token_begin, token_end) and the active tail if it lies wholly inside; nothing is an error. A range whose end
        // is not above its begin (the reference's own test passes 0, 0) copies nothing.
        const uint32_t base = find(c, source, "source sequence does not exist").base;
        const uint32_t page = c->config.page_size, total = total_tokens(c, source), sealed = sealed_tokens(c, source);
        const uint64_t lo = token_begin > base ? token_begin - base : 0u;                 // the range in the store's coordinates
        const uint64_t hi = token_end > base ? std::min<uint64_t>(token_end - base, total) : 0u;
        uint64_t keep_end = hi >= total ? total : std::min<uint64_t>(hi / page * page, sealed);
        uint64_t keep_begin = std::min<uint64_t>((lo + page - 1) / page * page, keep_end);
        if (keep_begin > sealed) keep_begin = keep_end;   // the range starts inside the active tail: the tail is not wholly inside
        if (keep_begin >= keep_end) keep_begin = keep_end = 0;
        device_check(c, cf_ms_cuda_copy_sequence_async(c->device, source, destination, stream));
        if ((keep_end < total && cf_b200_ms_truncate_async(c->device, destination, static_cast<uint32_t>(keep_end), stream) != 0) ||
            (keep_begin > 0 && cf_b200_ms_drop_prefix_async(c->device, destination, static_cast<uint32_t>(keep_begin), stream) != 0)) {
            const std::string why = cf_ms_cuda_last_error(c->device);
            cf_ms_cuda_sequence_remove_async(c->device, destination, stream);
            c->sequences.erase(destination);
            update_active_peak(c);
            throw std::runtime_error(why);
        }
        SequenceState fresh;
        fresh.base = base + static_cast<uint32_t>(keep_begin);
        c->sequences[destination] = fresh;
        ++c->counters.sequences_copied;
        update_active_peak(c);
        maybe_audit(c);
    });
}

extern "C" int cf_sequence_remove_async(cf_multisequence_cache *c, int64_t id, int64_t position_begin, int64_t position_end,
                                        void *stream) {
    if (!c || position_end < position_begin) return -1;
    return guarded(c, [&] {
        find(c, id);
        if (position_begin < 0 && position_end < 0) {
            device_check(c, cf_ms_cuda_sequence_remove_async(c->device, id, stream));
            c->sequences.erase(id);
            ++c->counters.sequences_removed;
            update_active_peak(c);
            maybe_audit(c);
            return;
        }
        // src/multisequence_cache.cpp:314-347. A sealed page the range covers goes, one it cuts is an error (an empty range
        // strictly inside a page cuts it); an active tail the range covers goes, one it enters and leaves by its end is
        // cut there, any other overlap is an error (an empty range strictly inside the tail too); a range that meets
        // nothing cached succeeds. Every successful range removal counts as a removal. Narrower here: what goes must be
        // a suffix of the sequence.
        const int64_t base = find(c, id).base;   // positions are logical; the store counts from the sequence's first held token
        const int64_t lo = std::max<int64_t>(position_begin, 0) - base, hi = position_end - base;   // may be negative
        const int64_t page = c->config.page_size, total = total_tokens(c, id), sealed = sealed_tokens(c, id);
        int64_t keep = total;   // tokens that stay
        bool page_kept_after_removed = false;
        for (int64_t p0 = 0; p0 < sealed; p0 += page) {
            const int64_t p1 = std::min(p0 + page, sealed);
            if (hi <= p0 || lo >= p1) {
                if (keep < total) page_kept_after_removed = true;
                continue;
            }
            if (lo > p0 || hi < p1) throw Unsupported("removal inside immutable page is not supported");
            keep = std::min(keep, p0);
        }
        if (total > sealed) {   // the active tail [sealed, total)
            if (lo <= sealed && hi >= total) keep = std::min(keep, sealed);
            else if (lo >= sealed && lo < total && hi >= total) keep = std::min(keep, lo);
            else if (hi > sealed && lo < total) throw Unsupported("non-suffix active-tail removal is not supported");
            else if (keep < total) page_kept_after_removed = true;   // pages went, the tail after them stays
        }
        if (page_kept_after_removed) throw Unsupported("only a suffix of a sequence can be removed");
        if (keep < total && cf_b200_ms_truncate_async(c->device, id, static_cast<uint32_t>(keep), stream) != 0)
            throw Unsupported(cf_ms_cuda_last_error(c->device));
        ++c->counters.sequences_removed;
        maybe_audit(c);
    });
}

extern "C" int cf_sequence_shift_async(cf_multisequence_cache *c, int64_t id, uint32_t position_begin, uint32_t position_end,
                                       int32_t delta, void *) {
    if (!c || position_end < position_begin) return -1;
    return guarded(c, [&] {
        // src/multisequence_cache.cpp:357-380: pages (and the active tail) wholly inside the range move by delta, a page the
        // range cuts is an error. The store holds a sequence's tokens contiguously, so what it can express is a move of
        // everything it holds (the offset changes), of nothing, or by zero; a move of only some of the pages would open
        // a gap or an overlap inside the sequence and is refused as unsupported.
        SequenceState &q = find(c, id);
        const uint32_t page = c->config.page_size, total = total_tokens(c, id), sealed = sealed_tokens(c, id);
        const uint64_t lo = position_begin > q.base ? position_begin - q.base : 0u;
        const uint64_t hi = position_end > q.base ? std::min<uint64_t>(position_end - q.base, total) : 0u;
        // a sealed page the range cuts is an error; an active tail the range cuts simply does not move (:372-377)
        const bool cuts_a_page = (lo < sealed && lo % page != 0) || (hi < sealed && hi % page != 0);
        if (lo < hi && cuts_a_page) throw Unsupported("context shift must align with immutable page boundaries");
        const uint64_t first_page = std::min<uint64_t>((lo + page - 1) / page, sealed / page);
        const uint64_t pages_moved = lo < hi ? std::min<uint64_t>(hi, sealed) / page - std::min(first_page, std::min<uint64_t>(hi, sealed) / page) : 0u;
        const bool has_tail = total > sealed, tail_moves = has_tail && lo < hi && lo <= sealed && hi >= total;
        const bool nothing = pages_moved == 0 && !tail_moves;
        const bool everything = total > 0 && pages_moved == sealed / page && (tail_moves || !has_tail);
        if (!nothing && !everything && delta != 0)
            throw Unsupported("a shift of part of a sequence would leave a gap in its stored tokens");
        if (everything) {
            if (static_cast<int64_t>(q.base) + delta < 0) throw std::runtime_error("context shift produces negative token position");
            q.base = static_cast<uint32_t>(static_cast<int64_t>(q.base) + delta);
        }
        ++c->counters.sequences_shifted;
        maybe_audit(c);
    });
}

extern "C" int cf_sequence_append_async(cf_multisequence_cache *c, int64_t id, uint32_t layer, uint32_t token_begin,
                                        const cf_device_tensor_view *keys, const cf_device_tensor_view *values, void *stream) {
    if (!c || !keys || !values || layer >= c->config.layer_count || cf_device_tensor_validate(keys) != 0 ||
        cf_device_tensor_validate(values) != 0)
        return -1;
    return guarded(c, [&] {
        SequenceState &q = find(c, id);
        // a sequence that holds nothing adopts the position of its first rows (src/multisequence_cache.cpp:423: an empty
        // active page takes the caller's token_begin); the layers of one sequence share that first position here
        if (total_tokens(c, id) == 0) q.base = token_begin;
        if (token_begin < q.base) throw std::runtime_error("non-contiguous sequence append");
        device_check(c, cf_b200_ms_append_active_async(c->device, id, layer, token_begin - q.base, keys, values, stream));
        uint32_t sealed = 0, active = 0;
        cf_b200_ms_sequence_tokens(c->device, id, layer, &sealed, &active);
        if (active == c->config.page_size && !q.speculation.active)   // a full page is sealed on the GPU at once
            device_check(c, cf_b200_ms_seal_active_async(c->device, id, layer, stream));
        maybe_audit(c);
    });
}

extern "C" int cf_multisequence_attention_async(cf_multisequence_cache *c, const cf_sequence_attention_item *items,
                                                uint32_t item_count, void *stream) {
    if (!c || !items || item_count == 0) return -1;
    return guarded(c, [&] {
        std::set<int64_t> observed;
        bool rebased = false;
        for (uint32_t i = 0; i < item_count; ++i) {
            const cf_sequence_attention_item &item = items[i];
            auto it = c->sequences.find(item.sequence_id);
            if (it == c->sequences.end()) throw std::runtime_error("attention item references unknown sequence");
            if (item.layer >= c->config.layer_count || cf_device_tensor_validate(&item.query) != 0 || !item.output)
                throw std::runtime_error("invalid sequence attention item");
            if (item.query_token_begin < it->second.base) throw std::runtime_error("query position lies before the sequence's first token");
            rebased = rebased || it->second.base != 0;
            observed.insert(item.sequence_id);
        }
        ++c->counters.batches_dispatched;
        c->counters.sequences_per_batch_peak = std::max<uint64_t>(c->counters.sequences_per_batch_peak, observed.size());
        if (!rebased) {
            device_check(c, cf_ms_cuda_execute_batch_async(c->device, reinterpret_cast<const cf_ms_batch_item *>(items), item_count, stream));
            return;
        }
        std::vector<cf_sequence_attention_item> local(items, items + item_count);   // logical positions -> the store's
        for (cf_sequence_attention_item &item : local) item.query_token_begin -= c->sequences.at(item.sequence_id).base;
        device_check(c, cf_ms_cuda_execute_batch_async(c->device, reinterpret_cast<const cf_ms_batch_item *>(local.data()), item_count, stream));
    });
}

extern "C" cf_speculation_id cf_sequence_speculation_begin(cf_multisequence_cache *c, int64_t id) {
    if (!c) return 0;
    cf_speculation_id out = 0;
    guarded(c, [&] {
        SequenceState &q = find(c, id);
        if (q.speculation.active) throw std::runtime_error("speculation already active");
        q.speculation = {c->next_speculation_id++, total_tokens(c, id), true};
        ++c->counters.speculative_transactions_started;
        out = q.speculation.id;
    });
    return out;
}

extern "C" int cf_sequence_speculation_commit(cf_multisequence_cache *c, int64_t id, cf_speculation_id speculation_id,
                                              uint32_t accepted_tokens, void *stream) {
    if (!c || speculation_id == 0) return -1;
    return guarded(c, [&] {
        auto it = c->sequences.find(id);
        if (it == c->sequences.end() || !it->second.speculation.active || it->second.speculation.id != speculation_id)
            throw std::runtime_error("invalid speculative transaction");
        const uint32_t baseline = it->second.speculation.baseline_tokens;
        if (total_tokens(c, id) < baseline) throw std::runtime_error("active tail predates speculative baseline");
        if (accepted_tokens > total_tokens(c, id) - baseline)
            throw std::runtime_error("accepted token count exceeds provisional tail");
        device_check(c, cf_b200_ms_truncate_async(c->device, id, baseline + accepted_tokens, stream));
        it->second.speculation = {};
        seal_full_tails(c, id, stream);
        ++c->counters.speculative_transactions_committed;
        maybe_audit(c);
    });
}

extern "C" int cf_sequence_speculation_rollback(cf_multisequence_cache *c, int64_t id, cf_speculation_id speculation_id,
                                                void *stream) {
    if (!c || speculation_id == 0) return -1;
    return guarded(c, [&] {
        auto it = c->sequences.find(id);
        if (it == c->sequences.end() || !it->second.speculation.active || it->second.speculation.id != speculation_id)
            throw std::runtime_error("invalid speculative transaction");
        device_check(c, cf_b200_ms_truncate_async(c->device, id, it->second.speculation.baseline_tokens, stream));
        it->second.speculation = {};
        ++c->counters.speculative_transactions_rolled_back;
        maybe_audit(c);
    });
}

extern "C" int cf_multisequence_reclaim_async(cf_multisequence_cache *c, void *stream) {
    if (!c) return -1;
    return guarded(c, [&] {
        device_check(c, cf_ms_cuda_reclaim_async(c->device, stream));
        maybe_audit(c);
    });
}

extern "C" int cf_multisequence_audit(const cf_multisequence_cache *c) {
    if (!c) return -1;
    std::lock_guard<std::mutex> guard(c->mutex);
    return cf_ms_cuda_audit(c->device);
}

extern "C" int cf_multisequence_get_counters(const cf_multisequence_cache *c, cf_multisequence_counters *out) {
    if (!c || !out) return -1;
    std::lock_guard<std::mutex> guard(c->mutex);
    cf_ms_cuda_counters device{};
    cf_ms_cuda_get_counters(c->device, &device);
    c->counters.pages_reclaimed = device.pages_reclaimed;
    c->counters.pages_pending_reclamation = device.pages_retired - device.pages_reclaimed;
    c->counters.pending_reclamation_bytes = device.pending_reclamation_bytes;
    c->counters.pending_reclamation_bytes_peak = device.pending_reclamation_bytes_peak;
    c->counters.dense_fallback_launches = device.dense_fallback_launches;
    uint64_t shared = 0, references = 0, increments = 0, decrements = 0;
    cf_b200_ms_page_sharing(c->device, &shared, &references, &increments, &decrements);
    c->counters.shared_pages = shared;
    c->counters.shared_page_references = references;
    c->counters.page_ref_increments = increments;
    c->counters.page_ref_decrements = decrements;
    *out = c->counters;
    return 0;
}

extern "C" const char *cf_multisequence_last_error(const cf_multisequence_cache *c) {
    return c ? c->last_error.c_str() : "null multisequence cache";
}

// ---------------------------------------------------------------------------------------------------------------
// llama-server runtime: slots, batches and shutdown over the cache above (src/llama_server_runtime.cpp:44-244).
// ---------------------------------------------------------------------------------------------------------------
struct cf_llama_server_runtime {
    cf_llama_server_config config{};
    cf_multisequence_cache *cache = nullptr;
    mutable std::mutex mutex;
    std::unordered_set<int64_t> live;
    cf_llama_server_stats stats{};
    bool shutting_down = false;
    std::string error;
};

namespace {

int server_fail(cf_llama_server_runtime *r, const char *message) {
    r->error = message && *message ? message : "unknown server runtime error";
    return -1;
}

}  // namespace

extern "C" cf_llama_server_runtime *cf_llama_server_runtime_create(const cf_llama_server_config *c) {
    if (!c || !c->layer_count || !c->query_head_count || !c->kv_head_count || !c->head_dim || !c->page_size || !c->block_size ||
        !c->gqa_group_size || c->query_head_count != c->kv_head_count * c->gqa_group_size || !c->llama_commit || !c->model_sha256)
        return nullptr;
    try {
        auto r = std::make_unique<cf_llama_server_runtime>();
        r->config = *c;
        cf_multisequence_config host{};
        host.layer_count = c->layer_count;
        host.kv_head_count = c->kv_head_count;
        host.query_head_count = c->query_head_count;
        host.head_dim = c->head_dim;
        host.page_size = c->page_size;
        host.gqa_group_size = c->gqa_group_size;
        host.use_async_allocator = 1;
        host.enable_invariant_auditor = 1;
        r->cache = cf_multisequence_create(&host);
        if (!r->cache) return nullptr;
        return r.release();
    } catch (...) {
        return nullptr;
    }
}

extern "C" void cf_llama_server_runtime_destroy(cf_llama_server_runtime *r, void *stream) {
    if (!r) return;
    cf_llama_server_shutdown_async(r, stream);
    if (r->cache) cf_multisequence_destroy(r->cache, stream);
    delete r;
}

extern "C" int cf_llama_server_slot_create(cf_llama_server_runtime *r, int64_t id) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down) return server_fail(r, "server runtime is shutting down");
    if (r->live.count(id)) return server_fail(r, "sequence already exists");
    if (cf_sequence_create(r->cache, id) != 0) return server_fail(r, cf_multisequence_last_error(r->cache));
    r->live.insert(id);
    ++r->stats.http_requests;
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_slot_reset_async(cf_llama_server_runtime *r, int64_t id, void *stream) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (!r->live.count(id)) return server_fail(r, "sequence does not exist");
    if (cf_sequence_remove_async(r->cache, id, -1, -1, stream) != 0) return server_fail(r, cf_multisequence_last_error(r->cache));
    r->live.erase(id);
    ++r->stats.slot_reuses;
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_cancel_async(cf_llama_server_runtime *r, int64_t id, void *stream) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (!r->live.count(id)) return server_fail(r, "sequence does not exist");
    if (cf_ms_cuda_cancel_sequence_async(r->cache->device, id, stream) != 0) return server_fail(r, cf_ms_cuda_last_error(r->cache->device));
    ++r->stats.cancelled_requests;
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_sequence_copy_async(cf_llama_server_runtime *r, int64_t source, int64_t destination,
                                                   uint32_t token_begin, uint32_t token_end, void *stream) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down || !r->live.count(source)) return server_fail(r, "source sequence does not exist");
    if (cf_sequence_copy_async(r->cache, source, destination, token_begin, token_end, stream) != 0)
        return server_fail(r, cf_multisequence_last_error(r->cache));
    r->live.insert(destination);
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_sequence_remove_async(cf_llama_server_runtime *r, int64_t id, int64_t position_begin,
                                                     int64_t position_end, void *stream) {
    if (!r) return -1;
    if (position_begin < 0 && position_end < 0) return cf_llama_server_slot_reset_async(r, id, stream);
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down || !r->live.count(id)) return server_fail(r, "sequence does not exist");
    if (cf_sequence_remove_async(r->cache, id, position_begin, position_end, stream) != 0)
        return server_fail(r, cf_multisequence_last_error(r->cache));
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_sequence_shift_async(cf_llama_server_runtime *r, int64_t id, uint32_t position_begin,
                                                    uint32_t position_end, int32_t delta, void *stream) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down || !r->live.count(id)) return -1;
    if (cf_sequence_shift_async(r->cache, id, position_begin, position_end, delta, stream) != 0)
        return server_fail(r, cf_multisequence_last_error(r->cache));
    ++r->stats.context_shifts;
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_append_layer_async(cf_llama_server_runtime *r, int64_t id, uint32_t layer, uint32_t token_begin,
                                                  const float *key, const float *value, uint32_t token_count, void *stream) {
    if (!r || !key || !value || !token_count) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down || !r->live.count(id)) return -1;
    if (layer >= r->config.layer_count) return server_fail(r, "layer index is out of range");
    const uint64_t row = static_cast<uint64_t>(r->config.kv_head_count) * r->config.head_dim;
    uint32_t done = 0;
    while (done < token_count) {   // page by page: an append never crosses a page boundary
        const uint32_t position = token_begin + done;
        const uint32_t chunk = std::min(token_count - done, r->config.page_size - position % r->config.page_size);
        cf_device_tensor_view k{};
        k.scalar_type = CF_DEVICE_F32;
        k.token_count = chunk;
        k.head_count = r->config.kv_head_count;
        k.head_dim = r->config.head_dim;
        k.element_stride_bytes = 4;
        k.head_stride_bytes = 4ull * r->config.head_dim;
        k.token_stride_bytes = 4ull * row;
        k.device_ordinal = static_cast<int32_t>(r->config.cuda_device);
        cf_device_tensor_view v = k;
        k.data = key + done * row;
        v.data = value + done * row;
        if (cf_sequence_append_async(r->cache, id, layer, position, &k, &v, stream) != 0)
            return server_fail(r, cf_multisequence_last_error(r->cache));
        done += chunk;
    }
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_execute_batch_async(cf_llama_server_runtime *r, const cf_llama_server_batch *batch, void *stream) {
    if (!r || !batch || !batch->attention_items || !batch->attention_item_count) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down) return server_fail(r, "server runtime is shutting down");
    if (r->stats.dense_nodes_scheduled != 0) return server_fail(r, "dense attention node scheduled while the sealed-KV backend is active");
    std::unordered_set<int64_t> ids;
    for (uint32_t i = 0; i < batch->attention_item_count; ++i) {
        if (!r->live.count(batch->attention_items[i].sequence_id)) return server_fail(r, "batch references unknown sequence");
        ids.insert(batch->attention_items[i].sequence_id);
    }
    if (ids.size() > 1) ++r->stats.interleaved_batches;
    if (cf_multisequence_attention_async(r->cache, batch->attention_items, batch->attention_item_count, stream) != 0)
        return server_fail(r, cf_multisequence_last_error(r->cache));
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_shutdown_async(cf_llama_server_runtime *r, void *stream) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down) return r->stats.shutdown_failures ? -1 : 0;
    r->shutting_down = true;
    for (int64_t id : r->live) {
        cf_ms_cuda_cancel_sequence_async(r->cache->device, id, stream);
        cf_sequence_remove_async(r->cache, id, -1, -1, stream);
    }
    r->live.clear();
    cf_multisequence_reclaim_async(r->cache, stream);
    ++r->stats.shutdown_audits;
    if (cf_multisequence_audit(r->cache) != 0) {
        ++r->stats.shutdown_failures;
        return server_fail(r, "shutdown invariant audit failed");
    }
    r->error.clear();
    return 0;
}

extern "C" int cf_llama_server_get_stats(const cf_llama_server_runtime *r, cf_llama_server_stats *out) {
    if (!r || !out) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    *out = r->stats;
    return 0;
}

extern "C" const char *cf_llama_server_last_error(const cf_llama_server_runtime *r) {
    return r ? r->error.c_str() : "runtime is null";
}
