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

#include <cstdio>

#include "attention_params.cuh"

namespace {

static __device__ __align__(256) unsigned char g_static_workspace[CF_B200_STATIC_WORKSPACE_BYTES];

constexpr int kMaxDevices = 64;
void *g_workspace_address[kMaxDevices] = {};  // device address of the array, per device ordinal
thread_local char g_error[160] = "";

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
    const cfb::WorkspaceLayout layout =
        cfb::workspace_layout(desc->seq_count, local_q, desc->head_dim, CF_B200_STATIC_WORKSPACE_BYTES,
                              desc->shared_prefix_pages != 0);
    if (layout.partials_offset >= CF_B200_STATIC_WORKSPACE_BYTES || layout.chunk_capacity < desc->seq_count) {
        std::snprintf(g_error, sizeof g_error,
                      "batch too large for the built-in workspace: %u sequences x %u query heads x head_dim %u needs "
                      "more than %u bytes",
                      desc->seq_count, local_q, desc->head_dim, static_cast<unsigned>(CF_B200_STATIC_WORKSPACE_BYTES));
        return CF_ERR_UNSUPPORTED;
    }

    // Set-up, once per device, with that device current: in host code the array's name is only a stand-in, the
    // device address has to be asked for. This first call per device should come before any stream capture.
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
        return fail(CF_ERR_CUDA, "no current CUDA device (or device ordinal beyond 63)");
    if (g_workspace_address[device] == nullptr) {
        void *address = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&address, g_static_workspace);
        if (e != cudaSuccess || address == nullptr) {
            std::snprintf(g_error, sizeof g_error, "cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return CF_ERR_CUDA;
        }
        g_workspace_address[device] = address;
    }

    cf_b200_sealed_attention_desc with_workspace = *desc;
    with_workspace.workspace = g_workspace_address[device];
    with_workspace.workspace_bytes = CF_B200_STATIC_WORKSPACE_BYTES;
    const cf_status status = cf_b200_sealed_attention_async(&with_workspace, stream);
    if (status != CF_OK) return fail(status, "the attention launch rejected the descriptor or a CUDA launch failed");
    return CF_OK;
}
