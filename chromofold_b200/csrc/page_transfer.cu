// page_transfer.cu — pack sealed records of an arena into a contiguous transfer image and unpack them into another
// arena, with an FNV-1a checksum per record (the checksum of the reference's page store,
// src/persistent_page_store.cpp:11-15). Declared in include/chromofold_b200/page_transfer.h.
//
// One block per (page, kv head). The copy is 16 bytes per thread per step; the checksum is inherently serial
// (h = (h ^ byte) * prime), so it is cut into 32 independent lanes — lane l hashes the bytes of 16-byte units
// l, l + 32, ... — and the 32 lane hashes are folded in lane order with the same recurrence applied to their
// 8 bytes each. The result is a function of the record bytes only, equal on both sides.

#include <cuda_runtime.h>

#include "chromofold_b200/page_transfer.h"

namespace {

constexpr unsigned long long kFnvBasis = 1469598103934665603ull, kFnvPrime = 1099511628211ull;

__host__ __device__ inline unsigned long long fnv_bytes(unsigned long long h, const uint8_t *p, uint64_t n) {
    for (uint64_t i = 0; i < n; ++i) h = (h ^ p[i]) * kFnvPrime;
    return h;
}

// Checksum of `units` 16-byte units at `record`, computed by warp 0 of the block; valid in every thread afterwards.
__device__ unsigned long long record_checksum(const uint8_t *record, uint32_t units, unsigned long long *s_result) {
    if (threadIdx.x < 32) {
        unsigned long long h = kFnvBasis;
        for (uint32_t u = threadIdx.x; u < units; u += 32) {
            const uint4 v = reinterpret_cast<const uint4 *>(record)[u];
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int b = 0; b < 4; ++b) h = (h ^ ((w[i] >> (8 * b)) & 0xffu)) * kFnvPrime;
        }
        unsigned long long total = kFnvBasis;
        for (int lane = 0; lane < 32; ++lane) {   // fold the lane hashes in lane order
            const unsigned long long x = __shfl_sync(0xffffffffu, h, lane);
#pragma unroll
            for (int b = 0; b < 8; ++b) total = (total ^ ((x >> (8 * b)) & 0xffull)) * kFnvPrime;
        }
        if (threadIdx.x == 0) *s_result = total;
    }
    __syncthreads();
    return *s_result;
}

__global__ void __launch_bounds__(128) pack_kernel(const uint8_t *arena, const uint64_t *page_dir, uint32_t kv_heads,
                                                   const uint32_t *page_ids, cf_b200_transfer_entry *manifest, uint8_t *payload,
                                                   uint64_t capacity_units, unsigned long long *cursor, uint32_t *status) {
    __shared__ unsigned long long s_sum, s_offset;
    const uint32_t page = blockIdx.x, head = blockIdx.y;
    const uint64_t entry = page_dir[static_cast<uint64_t>(page_ids[page]) * kv_heads + head];
    const uint32_t units = static_cast<uint32_t>(CF_B200_DIR_LENGTH_UNITS(entry));
    cf_b200_transfer_entry out{0u, 0u, 0ull};
    if (units != 0) {
        const uint8_t *record = arena + 16ull * CF_B200_DIR_OFFSET_UNITS(entry);
        if (threadIdx.x == 0) s_offset = atomicAdd(cursor, static_cast<unsigned long long>(units));
        const unsigned long long sum = record_checksum(record, units, &s_sum);   // also orders s_offset
        if (s_offset + units <= capacity_units) {
            uint4 *dst = reinterpret_cast<uint4 *>(payload) + s_offset;
            for (uint32_t u = threadIdx.x; u < units; u += blockDim.x) dst[u] = reinterpret_cast<const uint4 *>(record)[u];
            out.offset_units = static_cast<uint32_t>(s_offset);
            out.length_units = units;
            out.checksum = sum;
        } else if (threadIdx.x == 0 && status) {
            atomicOr(status, CF_B200_DEVSTAT_ARENA_FULL);
        }
    }
    if (threadIdx.x == 0) manifest[static_cast<uint64_t>(page) * kv_heads + head] = out;
}

__global__ void __launch_bounds__(128) unpack_kernel(const cf_b200_transfer_entry *manifest, const uint8_t *payload,
                                                     uint64_t payload_units, uint32_t kv_heads, const uint32_t *dst_page_ids,
                                                     uint8_t *arena, uint64_t arena_units, unsigned long long *cursor,
                                                     uint64_t *page_dir, uint32_t *status) {
    __shared__ unsigned long long s_sum, s_offset;
    const uint32_t page = blockIdx.x, head = blockIdx.y;
    const cf_b200_transfer_entry e = manifest[static_cast<uint64_t>(page) * kv_heads + head];
    uint64_t *dir = page_dir + static_cast<uint64_t>(dst_page_ids[page]) * kv_heads + head;
    if (e.length_units == 0) {
        if (threadIdx.x == 0) *dir = 0ull;
        return;
    }
    const bool inside = static_cast<uint64_t>(e.offset_units) + e.length_units <= payload_units && e.length_units <= 0xffffu;
    const uint8_t *record = payload + 16ull * e.offset_units;
    const unsigned long long sum = inside ? record_checksum(record, e.length_units, &s_sum) : 0ull;
    if (!inside || sum != e.checksum) {
        if (threadIdx.x == 0) {
            *dir = 0ull;
            if (status) atomicOr(status, CF_B200_DEVSTAT_CHECKSUM);
        }
        return;
    }
    if (threadIdx.x == 0) s_offset = atomicAdd(cursor, static_cast<unsigned long long>(e.length_units));
    __syncthreads();
    if (s_offset + e.length_units > arena_units) {
        if (threadIdx.x == 0) {
            *dir = 0ull;
            if (status) atomicOr(status, CF_B200_DEVSTAT_ARENA_FULL);
        }
        return;
    }
    uint4 *dst = reinterpret_cast<uint4 *>(arena) + s_offset;
    for (uint32_t u = threadIdx.x; u < e.length_units; u += blockDim.x) dst[u] = reinterpret_cast<const uint4 *>(record)[u];
    __threadfence();   // the record is in place before its directory entry is
    __syncthreads();
    if (threadIdx.x == 0) *dir = CF_B200_DIR_ENTRY(s_offset, e.length_units);
}

}  // namespace

extern "C" cf_status cf_b200_pages_pack_async(const uint8_t *arena, const uint64_t *page_dir, uint32_t kv_head_count,
                                              const uint32_t *page_ids, uint32_t page_count, cf_b200_transfer_entry *manifest,
                                              uint8_t *payload, uint64_t payload_capacity_bytes,
                                              unsigned long long *payload_cursor_units, uint32_t *status, void *stream) {
    if (!arena || !page_dir || !page_ids || !manifest || !payload || !payload_cursor_units || kv_head_count == 0)
        return CF_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(arena) & 15u) || (reinterpret_cast<uintptr_t>(payload) & 15u)) return CF_ERR_INVALID_ARGUMENT;
    if (page_count == 0) return CF_OK;
    if (kv_head_count > 65535u) return CF_ERR_UNSUPPORTED;
    pack_kernel<<<dim3(page_count, kv_head_count), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        arena, page_dir, kv_head_count, page_ids, manifest, payload, payload_capacity_bytes / 16, payload_cursor_units, status);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}

extern "C" cf_status cf_b200_pages_unpack_async(const cf_b200_transfer_entry *manifest, const uint8_t *payload,
                                                uint64_t payload_bytes, uint32_t kv_head_count, const uint32_t *dst_page_ids,
                                                uint32_t page_count, uint8_t *arena, uint64_t arena_units,
                                                unsigned long long *arena_cursor_units, uint64_t *page_dir, uint32_t *status,
                                                void *stream) {
    if (!manifest || !payload || !dst_page_ids || !arena || !arena_cursor_units || !page_dir || kv_head_count == 0)
        return CF_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(arena) & 15u) || (reinterpret_cast<uintptr_t>(payload) & 15u)) return CF_ERR_INVALID_ARGUMENT;
    if (page_count == 0) return CF_OK;
    if (kv_head_count > 65535u) return CF_ERR_UNSUPPORTED;
    unpack_kernel<<<dim3(page_count, kv_head_count), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        manifest, payload, payload_bytes / 16, kv_head_count, dst_page_ids, arena, arena_units, arena_cursor_units, page_dir, status);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}

extern "C" uint64_t cf_b200_record_checksum(const void *record, uint64_t bytes) {
    const uint8_t *p = static_cast<const uint8_t *>(record);
    if (!p) return 0;
    unsigned long long total = kFnvBasis;
    for (uint64_t lane = 0; lane < 32; ++lane) {
        unsigned long long h = kFnvBasis;
        for (uint64_t u = lane; u < bytes / 16; u += 32) h = fnv_bytes(h, p + 16 * u, 16);
        uint8_t le[8];
        for (int b = 0; b < 8; ++b) le[b] = static_cast<uint8_t>(h >> (8 * b));
        total = fnv_bytes(total, le, 8);
    }
    return total;
}

extern "C" uint64_t cf_b200_fnv1a(const void *bytes, uint64_t count) {
    return bytes ? fnv_bytes(kFnvBasis, static_cast<const uint8_t *>(bytes), count) : kFnvBasis;
}
