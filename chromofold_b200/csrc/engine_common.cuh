// engine_common.cuh — pieces shared by the fronts of the reference's device ABIs (device_engine.cu, ms_resolver.cu):
// a grow-only device buffer, typed strided loads and stores, and the row-conversion kernels.
#ifndef CHROMOFOLD_B200_ENGINE_COMMON_CUH
#define CHROMOFOLD_B200_ENGINE_COMMON_CUH

#include <algorithm>
#include <cstdlib>
#include <stdexcept>
#include <string>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "chromofold_b200/compat_device.h"
#include "chromofold_b200/sealed_kv.h"

namespace cfb_engine {

inline void cuda_check(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// The coder the stores behind the reference's device ABIs seal with: nibble-split rANS unless CHROMOFOLD_B200_CODER names
// another (rans | huffman | fixed8 | rans4 | huffman4). The split coders need tiles of a multiple of eight values.
inline uint32_t engine_coder(uint32_t tile_values) {
    uint32_t coder = CF_B200_CODER_RANS_SPLIT4;
    if (const char *env = std::getenv("CHROMOFOLD_B200_CODER")) {
        const std::string name(env);
        if (name == "rans") coder = CF_B200_CODER_RANS;
        else if (name == "huffman") coder = CF_B200_CODER_HUFFMAN;
        else if (name == "fixed8") coder = CF_B200_CODER_FIXED8;
        else if (name == "huffman4") coder = CF_B200_CODER_HUFFMAN_SPLIT4;
    }
    if (tile_values % 8u != 0) {
        if (coder == CF_B200_CODER_RANS_SPLIT4) coder = CF_B200_CODER_RANS;
        if (coder == CF_B200_CODER_HUFFMAN_SPLIT4) coder = CF_B200_CODER_HUFFMAN;
    }
    return coder;
}

inline size_t scalar_bytes(uint32_t type) {
    return type == CF_DEVICE_F16 || type == CF_DEVICE_BF16 ? 2 : type == CF_DEVICE_F32 ? 4 : 0;
}

template <class T>
struct Buffer {  // grow-only device array; growing copies the old contents
    T *ptr = nullptr;
    size_t count = 0;
    Buffer() = default;
    Buffer(const Buffer &) = delete;
    Buffer &operator=(const Buffer &) = delete;
    ~Buffer() { if (ptr) cudaFree(ptr); }
    void ensure(size_t wanted, cudaStream_t s) {
        if (wanted <= count) return;
        const size_t next = std::max(wanted, count * 2);
        T *fresh = nullptr;
        cuda_check(cudaMalloc(reinterpret_cast<void **>(&fresh), next * sizeof(T)), "cudaMalloc");
        cuda_check(cudaMemsetAsync(fresh, 0, next * sizeof(T), s), "cudaMemsetAsync");
        if (ptr) {
            cuda_check(cudaMemcpyAsync(fresh, ptr, count * sizeof(T), cudaMemcpyDeviceToDevice, s), "cudaMemcpyAsync");
            cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
            cudaFree(ptr);
        }
        ptr = fresh;
        count = next;
    }
    size_t bytes() const { return count * sizeof(T); }
};

__device__ __forceinline__ float load_scalar(const void *base, uint64_t byte_offset, uint32_t type) {
    const char *p = static_cast<const char *>(base) + byte_offset;
    if (type == CF_DEVICE_F16) return __half2float(*reinterpret_cast<const __half *>(p));
    if (type == CF_DEVICE_BF16) return __bfloat162float(*reinterpret_cast<const __nv_bfloat16 *>(p));
    return *reinterpret_cast<const float *>(p);
}

__device__ __forceinline__ void store_scalar(void *base, uint64_t byte_offset, uint32_t type, float v) {
    char *p = static_cast<char *>(base) + byte_offset;
    if (type == CF_DEVICE_F16) *reinterpret_cast<__half *>(p) = __float2half_rn(v);
    else if (type == CF_DEVICE_BF16) *reinterpret_cast<__nv_bfloat16 *>(p) = __float2bfloat16_rn(v);
    else *reinterpret_cast<float *>(p) = v;
}

// Strided [token][head][dim] rows of any scalar type -> the engine's fp32 tail [head][capacity][dim], starting at
// tail row `row0` (the job of the reference's convert_to_active, src/cuda/device_kv_dataplane.cu:49-70, with the
// head-major order the sealer and the attention tail reader use).
static __global__ void rows_to_tail_kernel(cf_device_tensor_view view, float *tail, uint32_t capacity, uint32_t row0) {
    const uint64_t count = static_cast<uint64_t>(view.token_count) * view.head_count * view.head_dim;
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t d = i % view.head_dim, h = (i / view.head_dim) % view.head_count;
    const uint32_t t = i / (static_cast<uint64_t>(view.head_dim) * view.head_count);
    const float v = load_scalar(view.data, t * view.token_stride_bytes + h * view.head_stride_bytes + d * view.element_stride_bytes,
                                view.scalar_type);
    tail[(static_cast<uint64_t>(h) * capacity + row0 + t) * view.head_dim + d] = v;
}

// Strided typed view -> contiguous fp32 [token][head][dim]; and back for outputs.
static __global__ void view_to_dense_kernel(cf_device_tensor_view view, float *dense) {
    const uint64_t count = static_cast<uint64_t>(view.token_count) * view.head_count * view.head_dim;
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t d = i % view.head_dim, h = (i / view.head_dim) % view.head_count;
    const uint32_t t = i / (static_cast<uint64_t>(view.head_dim) * view.head_count);
    dense[i] = load_scalar(view.data, t * view.token_stride_bytes + h * view.head_stride_bytes + d * view.element_stride_bytes,
                           view.scalar_type);
}
static __global__ void dense_to_view_kernel(const float *dense, void *out, uint32_t type, uint32_t tokens, uint32_t heads,
                                     uint32_t dim, uint64_t ts, uint64_t hs, uint64_t es) {
    const uint64_t count = static_cast<uint64_t>(tokens) * heads * dim;
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t d = i % dim, h = (i / dim) % heads;
    const uint32_t t = i / (static_cast<uint64_t>(dim) * heads);
    store_scalar(out, t * ts + h * hs + d * es, type, dense[i]);
}

// Room in an engine's attention workspace for the shared-prefix partials of `rows` query rows (the extra region of
// cf_device_common.cuh's layout). The workspace grows for it, once per larger batch size, up to kSharedWorkspaceCap;
// false = no room, the caller then leaves the hint out. Call before the descriptor's workspace pointer is taken.
constexpr uint64_t kSharedWorkspaceCap = 1ull << 30;
inline bool shared_prefix_room(Buffer<uint8_t> &workspace, uint32_t rows, uint32_t kv_heads, uint32_t query_heads, uint32_t head_dim,
                               cudaStream_t s) {
    cf_b200_sealed_attention_desc d{};
    d.kv_head_count = kv_heads;
    d.query_head_count = query_heads;
    d.head_dim = head_dim;
    d.seq_count = rows;
    d.shared_prefix_pages = 1;
    uint64_t bytes = 0;
    if (cf_b200_sealed_attention_workspace_bytes(&d, 65536, &bytes) != CF_OK || bytes + 256 > kSharedWorkspaceCap) return false;
    workspace.ensure(bytes + 256, s);
    return true;
}

inline uint32_t choose_tile_tokens(uint32_t page_size, uint32_t head_dim) {
    // 16-token records at head_dim 128, 96, 64 and 32 are the geometries of the lane-per-block attention kernels
    if ((head_dim == 128 || head_dim == 96 || head_dim == 64 || head_dim == 32) && page_size % 16 == 0) return 16;
    const uint32_t limit = CF_B200_MAX_STREAM_SYMBOLS / head_dim;
    for (uint32_t t = std::min(page_size, limit); t >= 1; --t)
        if (page_size % t == 0) return t;
    return 1;
}


}  // namespace cfb_engine

#endif
