// static_workspace.cu — sealed attention for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the point where they need attention: an inference engine
// that handed the whole device heap to its own arena at start-up, a plugin running inside another framework's
// memory budget, or a latency-critical serving thread where an allocator call (and the implicit synchronisation it
// may bring) is forbidden. cf_b200_sealed_attention_async asks such a caller for a split-KV workspace it has no way
// to provide. The entry point below takes the same descriptor but ignores its workspace fields and uses a fixed
// array that is part of the library image instead.
//
// The array lives in every GPU context that loads the library and stays there until the process exits
// (CF_B200_STATIC_WORKSPACE_BYTES per device). All calls on a device share it and it keeps whatever the last call
// left: the plan kernel rewrites the whole header (including the work counter, which must start at zero) at the
// start of every call, and every partial that is read was written earlier in the same call, so nothing stale is
// consumed — but two calls that overlap on the GPU (different streams, no ordering) would race on it. Callers
// must order them.

#include <atomic>
#include <cstdio>
#include <mutex>

#include "attention_params.cuh"

namespace {

static __device__ __align__(256) unsigned char g_static_workspace[CF_B200_STATIC_WORKSPACE_BYTES];

constexpr int kMaxDevices = 64;
std::atomic<void *> g_workspace_address[kMaxDevices] = {};  // device address of the array, per device ordinal
std::mutex g_setup_mutex;                                   // two threads may make the first call on a device at once
thread_local char g_error[200] = "";

cf_status fail(cf_status status, const char *what) {
    std::snprintf(g_error, sizeof g_error, "%s", what);
    return status;
}

}  // namespace

extern "C" const char *cf_b200_sealed_attention_static_error(void) { return g_error; }

extern "C" cf_status cf_b200_sealed_attention_static_async(const cf_b200_sealed_attention_desc *desc, void *stream) {
    g_error[0] = '\0';
    if (desc == nullptr || desc->struct_size != sizeof(cf_b200_sealed_attention_desc) ||
        desc->abi_version != CF_B200_ABI_VERSION)
        return fail(CF_ERR_INVALID_ARGUMENT, "descriptor is null or has the wrong struct_size / abi_version");
    if (desc->kv_head_count == 0 || desc->query_head_count == 0 || desc->head_dim == 0 ||
        desc->query_head_count % desc->kv_head_count != 0 || desc->kv_head_begin >= desc->kv_head_count ||
        desc->kv_head_span > desc->kv_head_count - desc->kv_head_begin || desc->seq_count == 0)
        return fail(CF_ERR_INVALID_ARGUMENT, "head counts, head_dim or seq_count are not usable");

    // Size check first, before any CUDA call: the fixed array must hold at least one partial per sequence.
    const uint32_t span = desc->kv_head_span ? desc->kv_head_span : desc->kv_head_count - desc->kv_head_begin;
    const uint32_t local_q = span * (desc->query_head_count / desc->kv_head_count);
    // The floor is one partial of (head_dim + 2) floats per sequence and query head; a shared-prefix hint sets aside
    // CF_B200_SHARED_CHUNKS_MAX more of those per sequence and query head. The hint is optional by contract, so a batch
    // whose plain partials fit but whose shared-prefix partials do not is served without the hint instead of refused.
    auto fits = [&](bool shared) {
        const cfb::WorkspaceLayout layout =
            cfb::workspace_layout(desc->seq_count, local_q, desc->head_dim, CF_B200_STATIC_WORKSPACE_BYTES, shared);
        return layout.partials_offset < CF_B200_STATIC_WORKSPACE_BYTES && layout.chunk_capacity >= desc->seq_count;
    };
    bool keep_hint = desc->shared_prefix_pages != 0;
    if (keep_hint && !fits(true)) keep_hint = false;
    if (!fits(keep_hint)) {
        const unsigned long long need = static_cast<unsigned long long>(desc->seq_count) * local_q * (desc->head_dim + 2u) * 4ull;
        std::snprintf(g_error, sizeof g_error,
                      "batch too large for the built-in workspace: %u sequences x %u query heads x (head_dim %u + 2) floats = "
                      "%llu bytes of partials at least, the array has %u",
                      desc->seq_count, local_q, desc->head_dim, need, static_cast<unsigned>(CF_B200_STATIC_WORKSPACE_BYTES));
        return CF_ERR_UNSUPPORTED;
    }

    // Set-up, once per device, with that device current: in host code the array's name is only a stand-in, the
    // device address has to be asked for. This first call per device should come before any stream capture.
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
        return fail(CF_ERR_CUDA, "no current CUDA device (or device ordinal beyond 63)");
    void *address = g_workspace_address[device].load(std::memory_order_acquire);
    if (address == nullptr) {
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        address = g_workspace_address[device].load(std::memory_order_relaxed);
        if (address == nullptr) {
            const cudaError_t e = cudaGetSymbolAddress(&address, g_static_workspace);
            if (e != cudaSuccess || address == nullptr) {
                std::snprintf(g_error, sizeof g_error, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
                return CF_ERR_CUDA;
            }
            g_workspace_address[device].store(address, std::memory_order_release);
        }
    }

    cf_b200_sealed_attention_desc with_workspace = *desc;
    with_workspace.workspace = address;
    with_workspace.workspace_bytes = CF_B200_STATIC_WORKSPACE_BYTES;
    if (!keep_hint) with_workspace.shared_prefix_pages = 0;
    const cf_status status = cf_b200_sealed_attention_async(&with_workspace, stream);
    if (status != CF_OK) {
        std::snprintf(g_error, sizeof g_error, "the attention call behind this entry point returned %s",
                      status == CF_ERR_INVALID_ARGUMENT ? "CF_ERR_INVALID_ARGUMENT (the descriptor did not validate)"
                      : status == CF_ERR_UNSUPPORTED    ? "CF_ERR_UNSUPPORTED (the geometry or the requested kernel is not served)"
                                                        : "CF_ERR_CUDA (a launch failed)");
        return status;
    }
    return CF_OK;
}
