// multigpu_runtime.cu — admission checks and accounting of the reference's multi-GPU runtime ABI
// (include/chromofold/multigpu_cuda_runtime.h:92-111, src/cuda/multigpu_cuda_runtime.cu:34-259). Declared in
// include/chromofold_b200/compat_multigpu.h. Like the reference's, these calls launch nothing.

#include <cuda_runtime.h>

#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <vector>

#include "chromofold_b200/compat_multigpu.h"

namespace {
struct Device {
    cf_multigpu_device_config config{};
    bool failed = false;
};
bool valid_codec(uint32_t bits) { return bits == 2u || bits == 4u || bits == 8u || bits == 16u; }
}  // namespace

struct cf_multigpu_cuda_runtime {
    cf_multigpu_runtime_config config{};
    std::vector<Device> devices;
    mutable std::mutex mutex;
    cf_multigpu_counters counters{};
    bool shutting_down = false;
    std::string error;

    Device *find(int32_t ordinal) {
        for (Device &d : devices)
            if (d.config.device_ordinal == ordinal) return &d;
        return nullptr;
    }
    int refuse(const char *why) {
        ++counters.fail_closed_rejections;
        error = why;
        return -1;
    }
    int cuda_failed(cudaError_t e) {
        ++counters.cuda_errors;
        error = cudaGetErrorString(e);
        return -1;
    }
};

extern "C" cf_multigpu_cuda_runtime *cf_multigpu_cuda_create(const cf_multigpu_runtime_config *c) {
    if (!c || !c->devices || c->device_count < 2u || c->tensor_parallel_size < 2u || c->tensor_parallel_size > c->device_count)
        return nullptr;
    try {
        auto r = std::make_unique<cf_multigpu_cuda_runtime>();
        r->config = *c;
        std::set<int32_t> seen;
        for (uint32_t i = 0; i < c->device_count; ++i) {
            const cf_multigpu_device_config &d = c->devices[i];
            if (d.device_ordinal < 0 || d.memory_budget_bytes == 0u || !seen.insert(d.device_ordinal).second) return nullptr;
            r->devices.push_back({d, false});
        }
        r->config.devices = nullptr;   // the caller's array is not kept
        return r.release();
    } catch (...) {
        return nullptr;
    }
}

extern "C" void cf_multigpu_cuda_destroy(cf_multigpu_cuda_runtime *r) {
    if (!r) return;
    cf_multigpu_cuda_shutdown(r);
    delete r;
}

extern "C" int cf_multigpu_cuda_validate_topology(cf_multigpu_cuda_runtime *r) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    for (const Device &a : r->devices)
        for (const Device &b : r->devices) {
            if (a.config.device_ordinal == b.config.device_ordinal) continue;
            int can = 0;
            const cudaError_t e = cudaDeviceCanAccessPeer(&can, a.config.device_ordinal, b.config.device_ordinal);
            if (e != cudaSuccess) return r->cuda_failed(e);
            if (!can && r->config.require_peer_access && !r->config.allow_host_staging)
                return r->refuse("required CUDA peer path is unavailable");
        }
    r->error.clear();
    return 0;
}

extern "C" int cf_multigpu_cuda_execute_async(cf_multigpu_cuda_runtime *r, const cf_multigpu_attention_shard *shards,
                                              uint32_t shard_count, void *) {
    if (!r || !shards || shard_count == 0u) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down) return r->refuse("runtime is shutting down");
    for (uint32_t i = 0; i < shard_count; ++i) {   // the whole batch is checked before anything is counted
        const cf_multigpu_attention_shard &s = shards[i];
        if (!s.query || !s.output || s.query_head_count == 0u || s.head_dim == 0u || s.page_count == 0u || !s.pages ||
            s.layer >= r->config.layer_count)
            return r->refuse("invalid multi-GPU shard");
        const Device *d = r->find(s.execution_device);
        if (!d || d->failed) return r->refuse("execution device is unknown or failed");
        for (uint32_t p = 0; p < s.page_count; ++p) {
            const cf_multigpu_page_view &page = s.pages[p];
            if (!page.key_payload || !page.value_payload || !valid_codec(page.key_codec) || !valid_codec(page.value_codec) ||
                page.head_dim != s.head_dim || page.token_count == 0u)
                return r->refuse("invalid device-local page descriptor");
        }
    }
    for (uint32_t i = 0; i < shard_count; ++i) {
        const cf_multigpu_attention_shard &s = shards[i];
        for (uint32_t p = 0; p < s.page_count; ++p) {
            const cf_multigpu_page_view &page = s.pages[p];
            if (page.source_device != s.execution_device) {
                int can = 0;
                const cudaError_t e = cudaDeviceCanAccessPeer(&can, s.execution_device, page.source_device);
                if (e != cudaSuccess) return r->cuda_failed(e);
                const uint64_t bytes = page.key_payload_bytes + page.value_payload_bytes;
                if (can) {
                    ++r->counters.p2p_copy_calls;
                    r->counters.p2p_bytes += bytes;
                } else if (r->config.allow_host_staging) {
                    ++r->counters.host_staged_copy_calls;
                    r->counters.host_staged_bytes += bytes;
                } else {
                    ++r->counters.transfer_errors;
                    return r->refuse("no permitted transport for remote page");
                }
                ++r->counters.remote_pages_loaded;
            }
            if (page.key_codec != page.value_codec || page.key_codec != 4u) ++r->counters.mixed_codec_pages_consumed;
        }
        ++r->counters.shards_dispatched;
    }
    if (r->config.collective != CF_MULTIGPU_COLLECTIVE_NONE) {
        ++r->counters.collective_calls;
        r->counters.collective_bytes += static_cast<uint64_t>(shard_count) * sizeof(float);
    }
    ++r->counters.batches_submitted;
    r->error.clear();
    return 0;
}

extern "C" int cf_multigpu_cuda_migrate_sequence_async(cf_multigpu_cuda_runtime *r, uint64_t, int32_t source, int32_t destination,
                                                       const cf_multigpu_page_view *pages, uint32_t page_count, void *) {
    if (!r || !pages || page_count == 0u || source == destination) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->shutting_down) return -1;
    for (uint32_t i = 0; i < page_count; ++i)
        if (pages[i].source_device != source || !pages[i].key_payload || !pages[i].value_payload)
            return r->refuse("migration source does not match page ownership");
    ++r->counters.migrations_completed;
    r->error.clear();
    return 0;
}

extern "C" int cf_multigpu_cuda_inject_device_failure(cf_multigpu_cuda_runtime *r, int32_t ordinal) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    Device *d = r->find(ordinal);
    if (!d) return -1;
    d->failed = true;   // a host-side flag: nothing is done to the GPU
    ++r->counters.device_failures_detected;
    return 0;
}

extern "C" int cf_multigpu_cuda_shutdown(cf_multigpu_cuda_runtime *r) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    r->shutting_down = true;
    if (r->counters.page_refs_at_shutdown != 0u || r->counters.snapshot_refs_at_shutdown != 0u) {
        r->error = "multi-GPU references remain at shutdown";
        return -1;
    }
    r->error.clear();
    return 0;
}

extern "C" int cf_multigpu_cuda_get_counters(const cf_multigpu_cuda_runtime *r, cf_multigpu_counters *out) {
    if (!r || !out) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    *out = r->counters;
    return 0;
}

extern "C" const char *cf_multigpu_cuda_last_error(const cf_multigpu_cuda_runtime *r) {
    return r ? r->error.c_str() : "runtime is null";
}
