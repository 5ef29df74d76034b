// production_runtime.cu — the reference's batched decode runtime (include/chromofold/production_attention.h:90-104,
// src/cuda/production_attention.cu:142-246) over the reference's own page descriptors (int4 nibbles + per-block fp32
// scales) and fp32 unsealed tails. Declared in include/chromofold_b200/compat_production.h, which also lists where
// this implementation departs from the reference on purpose (nibble convention, visibility rule).
//
// One launch serves the whole batch. A block owns one (item, kv head, query token); its four warps take every fourth
// token, so a nibble is decoded once for all query heads of the group; the warps' online-softmax states are merged in
// shared memory. The item array travels through a pinned staging ring into a pooled device buffer.

#include <math_constants.h>

#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <set>
#include <utility>
#include <vector>

#include "cf_device_common.cuh"
#include "chromofold_b200/compat_production.h"
#include "engine_common.cuh"

namespace {

using cfb_engine::cuda_check;
using cfb_engine::load_scalar;
using cfb_engine::store_scalar;

constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kPassHeads = 4;   // query heads of one group served per pass over the tokens
constexpr int kRing = 4;
constexpr float kLog2e = 1.4426950408889634f;

struct Shape { uint32_t hq, hkv, dim, group; };

// value = (nibble - 8) * scale[flat / block_size], low nibble first (src/cuda/device_kv_seal_attention.cu:106-118)
__device__ __forceinline__ float nibble_value(const uint8_t *payload, const float *scales, uint64_t flat, uint32_t block) {
    const uint32_t nib = (payload[flat >> 1] >> ((flat & 1u) * 4u)) & 0xfu;
    return static_cast<float>(static_cast<int>(nib) - 8) * scales[flat / block];
}

struct OnlineRow {  // one query head's state in one lane: four channels (lane + 32 j)
    float m, l, acc[4];
    __device__ __forceinline__ void reset() {
        m = -CUDART_INF_F;
        l = acc[0] = acc[1] = acc[2] = acc[3] = 0.0f;
    }
    __device__ __forceinline__ void add(float score, const float (&v)[4]) {
        const float nm = fmaxf(m, score);
        const float so = exp2f(m - nm), w = exp2f(score - nm);  // m = -inf gives so = 0
        l = l * so + w;
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[j] = acc[j] * so + w * v[j];
        m = nm;
    }
};

// With `splits` > 1, block (item, kv head * splits + split, query token) takes every splits-th page of the item (split 0
// also the active tail) and leaves (max, sum, weighted[D]) per query head in `partials`
// [(item * max_tokens + query token) * query heads + head][split][D + 2] for batch_combine_kernel: a batch of a few long
// items then still fills the GPU.
__global__ void __launch_bounds__(kThreads) batch_attention_kernel(const cf_attention_batch_item *items, Shape shape,
                                                                   unsigned long long *byte_counters, uint32_t splits,
                                                                   float *partials) {
    __shared__ float s_m[kWarps][kPassHeads], s_l[kWarps][kPassHeads];
    __shared__ float s_acc[kWarps][kPassHeads][128];
    const cf_attention_batch_item item = items[blockIdx.x];
    const uint32_t kv_head = blockIdx.y / splits, split = blockIdx.y % splits, qtok = blockIdx.z;
    if (qtok >= item.query.token_count) return;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t D = shape.dim, G = shape.group, HKV = shape.hkv;
    const uint32_t qpos = item.query_token_begin + qtok;
    const uint32_t first = cfb::window_begin(qpos, item.causal_window);
    const float scale = item.softmax_scale * kLog2e;
    unsigned long long payload_bytes = 0, scale_bytes = 0;

    for (uint32_t g0 = 0; g0 < G; g0 += kPassHeads) {
        const uint32_t heads = min(static_cast<uint32_t>(kPassHeads), G - g0);
        float q[kPassHeads][4];
#pragma unroll
        for (int g = 0; g < kPassHeads; ++g)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t d = lane + 32u * j;
                q[g][j] = (static_cast<uint32_t>(g) < heads && d < D)
                              ? load_scalar(item.query.data,
                                            qtok * item.query.token_stride_bytes +
                                                (kv_head * G + g0 + g) * item.query.head_stride_bytes +
                                                d * item.query.element_stride_bytes,
                                            item.query.scalar_type) * scale
                              : 0.0f;
            }
        OnlineRow row[kPassHeads];
#pragma unroll
        for (int g = 0; g < kPassHeads; ++g) row[g].reset();
        auto take = [&](const float (&k)[4], const float (&v)[4]) {
#pragma unroll
            for (int g = 0; g < kPassHeads; ++g) {
                if (static_cast<uint32_t>(g) >= heads) break;
                float dot = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) dot += q[g][j] * k[j];
                row[g].add(cfb::warp_sum(dot), v);
            }
        };
        for (uint32_t pi = split; pi < item.sealed_page_count; pi += splits) {
            const cf_device_page_descriptor page = item.sealed_pages[pi];
            if (!page.key_payload || !page.value_payload || !page.key_scales || !page.value_scales) continue;
            if (page.head_dim != D || page.kv_head_count != HKV || page.block_size == 0) continue;
            if (page.token_begin > qpos || page.token_begin + page.token_count <= first) continue;
            if (g0 == 0 && tid == 0) {
                payload_bytes += static_cast<unsigned long long>(page.token_count) * D;   // K + V nibbles of this head
                scale_bytes += 2ull * page.token_count * ((D + page.block_size - 1) / page.block_size) * 4ull;
            }
            for (uint32_t t = warp; t < page.token_count; t += kWarps) {
                const uint32_t absolute = page.token_begin + t;
                if (absolute < first || absolute > qpos) continue;
                const uint64_t flat0 = (static_cast<uint64_t>(t) * HKV + kv_head) * D;
                float k[4], v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t d = lane + 32u * j;
                    k[j] = d < D ? nibble_value(page.key_payload, page.key_scales, flat0 + d, page.block_size) : 0.0f;
                    v[j] = d < D ? nibble_value(page.value_payload, page.value_scales, flat0 + d, page.block_size) : 0.0f;
                }
                take(k, v);
            }
        }
        for (uint32_t t = warp; t < (split == 0 ? item.active_token_count : 0u); t += kWarps) {
            const uint32_t absolute = item.active_token_begin + t;
            if (absolute < first || absolute > qpos) continue;
            const uint64_t flat0 = (static_cast<uint64_t>(t) * HKV + kv_head) * D;
            float k[4], v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t d = lane + 32u * j;
                k[j] = d < D ? item.active_keys[flat0 + d] : 0.0f;
                v[j] = d < D ? item.active_values[flat0 + d] : 0.0f;
            }
            take(k, v);
        }
        __syncthreads();  // the previous pass is done with the shared arrays
#pragma unroll
        for (int g = 0; g < kPassHeads; ++g) {
            if (lane == 0) {
                s_m[warp][g] = row[g].m;
                s_l[warp][g] = row[g].l;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) s_acc[warp][g][lane + 32 * j] = row[g].acc[j];
        }
        __syncthreads();
        for (uint32_t i = tid; i < heads * D; i += kThreads) {
            const uint32_t g = i / D, d = i % D;
            float m = -CUDART_INF_F;
            for (int w = 0; w < kWarps; ++w) m = fmaxf(m, s_m[w][g]);
            float l = 0.0f, a = 0.0f;
            if (m != -CUDART_INF_F)
                for (int w = 0; w < kWarps; ++w) {
                    if (s_m[w][g] == -CUDART_INF_F) continue;
                    const float sw = exp2f(s_m[w][g] - m);
                    l += s_l[w][g] * sw;
                    a += s_acc[w][g][d] * sw;
                }
            if (splits > 1) {
                float *dst = partials + ((static_cast<uint64_t>(blockIdx.x) * gridDim.z + qtok) * shape.hq + kv_head * G + g0 + g) *
                                            splits * (D + 2u) + split * (D + 2u);
                if (d == 0) {
                    dst[0] = m;
                    dst[1] = l;
                }
                dst[2 + d] = a;
            } else {
                store_scalar(item.output,
                             qtok * item.output_token_stride_bytes + (kv_head * G + g0 + g) * item.output_head_stride_bytes +
                                 d * item.output_element_stride_bytes,
                             item.output_type, l > 0.0f ? a / l : 0.0f);
            }
        }
    }
    if (tid == 0 && byte_counters) {
        atomicAdd(&byte_counters[0], payload_bytes);
        atomicAdd(&byte_counters[1], scale_bytes);
    }
}

// CF_ATTENTION_REFERENCE: the plain form the reference's kernel has (production_attention.cu:59-139): one warp per
// (item, query head, query token), tokens in order, lanes over channels; same nibble and visibility rules as above.
// One block per (item, query head, query token): merges the splits' partials and writes the item's strided, typed output.
__global__ void batch_combine_kernel(const cf_attention_batch_item *items, Shape shape, uint32_t splits, const float *partials) {
    __shared__ float weight[32];   // splits <= 32
    __shared__ float total;
    const cf_attention_batch_item item = items[blockIdx.x];
    const uint32_t head = blockIdx.y, qtok = blockIdx.z, D = shape.dim, stride = D + 2u;
    if (qtok >= item.query.token_count) return;
    const float *src = partials + ((static_cast<uint64_t>(blockIdx.x) * gridDim.z + qtok) * shape.hq + head) * splits * stride;
    if (threadIdx.x < 32) {   // one warp: the splits' maxima and sums, in parallel over the splits
        const float ms = threadIdx.x < splits ? src[threadIdx.x * stride] : -CUDART_INF_F;
        const float m = cfb::warp_max(ms);
        const float w = ms == -CUDART_INF_F ? 0.0f : exp2f(ms - m);
        if (threadIdx.x < splits) weight[threadIdx.x] = w;
        const float l = cfb::warp_sum(threadIdx.x < splits ? src[threadIdx.x * stride + 1] * w : 0.0f);
        if (threadIdx.x == 0) total = l;
    }
    __syncthreads();
    const float l = total;
    for (uint32_t d = threadIdx.x; d < D; d += blockDim.x) {
        float a = 0.0f;
#pragma unroll 8
        for (uint32_t s = 0; s < splits; ++s) a += src[s * stride + 2 + d] * weight[s];   // independent loads
        store_scalar(item.output,
                     qtok * item.output_token_stride_bytes + head * item.output_head_stride_bytes + d * item.output_element_stride_bytes,
                     item.output_type, l > 0.0f ? a / l : 0.0f);
    }
}

__global__ void __launch_bounds__(32) plain_attention_kernel(const cf_attention_batch_item *items, Shape shape) {
    const cf_attention_batch_item item = items[blockIdx.x];
    const uint32_t q_head = blockIdx.y, qtok = blockIdx.z, lane = threadIdx.x;
    if (qtok >= item.query.token_count) return;
    const uint32_t D = shape.dim, HKV = shape.hkv, kv_head = q_head / shape.group;
    const uint32_t qpos = item.query_token_begin + qtok;
    const uint32_t first = cfb::window_begin(qpos, item.causal_window);
    float q[4];
    for (int j = 0; j < 4; ++j) {
        const uint32_t d = lane + 32u * j;
        q[j] = d < D ? load_scalar(item.query.data,
                                   qtok * item.query.token_stride_bytes + q_head * item.query.head_stride_bytes +
                                       d * item.query.element_stride_bytes,
                                   item.query.scalar_type)
                     : 0.0f;
    }
    float m = -CUDART_INF_F, l = 0.0f, acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    auto take = [&](const float (&k)[4], const float (&v)[4]) {
        float dot = 0.0f;
        for (int j = 0; j < 4; ++j) dot += q[j] * k[j];
        const float s = cfb::warp_sum(dot) * item.softmax_scale;
        const float nm = fmaxf(m, s);
        const float so = m == -CUDART_INF_F ? 0.0f : expf(m - nm), w = expf(s - nm);
        l = l * so + w;
        for (int j = 0; j < 4; ++j) acc[j] = acc[j] * so + w * v[j];
        m = nm;
    };
    for (uint32_t pi = 0; pi < item.sealed_page_count; ++pi) {
        const cf_device_page_descriptor page = item.sealed_pages[pi];
        if (!page.key_payload || !page.value_payload || !page.key_scales || !page.value_scales) continue;
        if (page.head_dim != D || page.kv_head_count != HKV || page.block_size == 0) continue;
        for (uint32_t t = 0; t < page.token_count; ++t) {
            const uint32_t absolute = page.token_begin + t;
            if (absolute < first || absolute > qpos) continue;
            const uint64_t flat0 = (static_cast<uint64_t>(t) * HKV + kv_head) * D;
            float k[4], v[4];
            for (int j = 0; j < 4; ++j) {
                const uint32_t d = lane + 32u * j;
                k[j] = d < D ? nibble_value(page.key_payload, page.key_scales, flat0 + d, page.block_size) : 0.0f;
                v[j] = d < D ? nibble_value(page.value_payload, page.value_scales, flat0 + d, page.block_size) : 0.0f;
            }
            take(k, v);
        }
    }
    for (uint32_t t = 0; t < item.active_token_count; ++t) {
        const uint32_t absolute = item.active_token_begin + t;
        if (absolute < first || absolute > qpos) continue;
        const uint64_t flat0 = (static_cast<uint64_t>(t) * HKV + kv_head) * D;
        float k[4], v[4];
        for (int j = 0; j < 4; ++j) {
            const uint32_t d = lane + 32u * j;
            k[j] = d < D ? item.active_keys[flat0 + d] : 0.0f;
            v[j] = d < D ? item.active_values[flat0 + d] : 0.0f;
        }
        take(k, v);
    }
    for (int j = 0; j < 4; ++j) {
        const uint32_t d = lane + 32u * j;
        if (d < D)
            store_scalar(item.output,
                         qtok * item.output_token_stride_bytes + q_head * item.output_head_stride_bytes +
                             d * item.output_element_stride_bytes,
                         item.output_type, l > 0.0f ? acc[j] / l : 0.0f);
    }
}

// max |a - b| and sum |a - b| of two fp32 arrays: result[0] = max (as ordered int bits), result[1] = sum
__global__ void compare_kernel(const float *a, const float *b, uint64_t count, float *result) {
    float mx = 0.0f, sum = 0.0f;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const float d = fabsf(a[i] - b[i]);
        mx = d == d ? fmaxf(mx, d) : CUDART_INF_F;  // a NaN counts as an unbounded error
        sum += d == d ? d : CUDART_INF_F;
    }
    mx = cfb::warp_max(mx);
    sum = cfb::warp_sum(sum);
    if ((threadIdx.x & 31u) == 0) {
        atomicMax(reinterpret_cast<int *>(result), __float_as_int(mx));  // non-negative floats order like ints
        atomicAdd(result + 1, sum);
    }
}

struct Slot {
    cf_attention_batch_item *host = nullptr;   // pinned
    cf_attention_batch_item *device = nullptr;
    uint32_t capacity = 0;
    cudaEvent_t done = nullptr;
    bool pending = false;
};

}  // namespace

struct cf_attention_runtime {
    cf_attention_runtime_config config{};
    mutable std::mutex mutex;
    mutable cf_attention_counters counters{};
    std::string error;
    Slot ring[kRing];
    uint32_t next_slot = 0;
    unsigned long long *byte_counters = nullptr;   // device: payload bytes, scale bytes
    cfb_engine::Buffer<float> scratch_a, scratch_b, compare_result;
    uint64_t reserved_bytes = 0;
    float *partials = nullptr;     // split partials of the optimized kernel, grow-only
    uint64_t partial_floats = 0;
    int sm_count = 0;
};

namespace {

void validate_items(const cf_attention_runtime &r, const cf_attention_batch_item *items, uint32_t count, uint32_t *max_tokens,
                    uint64_t *rows) {
    std::set<std::pair<int64_t, uint32_t>> seen;
    *max_tokens = 0;
    *rows = 0;
    for (uint32_t i = 0; i < count; ++i) {
        const cf_attention_batch_item &it = items[i];
        if (it.layer >= r.config.layer_count) throw std::invalid_argument("batch item layer is out of range");
        if (cf_device_tensor_validate(&it.query) != 0) throw std::invalid_argument("batch item query view is invalid");
        if (it.query.head_count != r.config.query_head_count || it.query.head_dim != r.config.head_dim)
            throw std::invalid_argument("batch item query shape does not match the runtime");
        if (!it.output || cfb_engine::scalar_bytes(it.output_type) == 0) throw std::invalid_argument("batch item output is invalid");
        if (it.output_element_stride_bytes < cfb_engine::scalar_bytes(it.output_type))
            throw std::invalid_argument("batch item output stride is too small");
        if (it.sealed_page_count && !it.sealed_pages) throw std::invalid_argument("batch item has pages but no descriptors");
        if (it.active_token_count && (!it.active_keys || !it.active_values))
            throw std::invalid_argument("batch item has active tokens but no active rows");
        if (!std::isfinite(it.softmax_scale)) throw std::invalid_argument("batch item softmax scale is not finite");
        if (!seen.insert({it.sequence_id, it.layer}).second)
            throw std::invalid_argument("two batch items name the same sequence and layer");
        *max_tokens = std::max(*max_tokens, it.query.token_count);
        *rows += it.query.token_count;
    }
}

// Stage the items and return their device copy; the slot is marked busy until `finish` records its event.
Slot &stage(cf_attention_runtime &r, const cf_attention_batch_item *items, uint32_t count, cudaStream_t s) {
    Slot &slot = r.ring[r.next_slot];
    r.next_slot = (r.next_slot + 1) % kRing;
    if (slot.pending) {
        cuda_check(cudaEventSynchronize(slot.done), "wait for a staging slot");
        slot.pending = false;
    }
    if (slot.capacity < count) {
        const uint32_t cap = std::max(count, std::max(64u, slot.capacity * 2));
        if (slot.host) cudaFreeHost(slot.host);
        if (slot.device) cudaFree(slot.device);
        slot.host = nullptr;
        slot.device = nullptr;
        r.reserved_bytes -= static_cast<uint64_t>(slot.capacity) * sizeof(cf_attention_batch_item);
        slot.capacity = 0;
        cuda_check(cudaMallocHost(reinterpret_cast<void **>(&slot.host), cap * sizeof(cf_attention_batch_item)), "pinned item buffer");
        cuda_check(cudaMalloc(reinterpret_cast<void **>(&slot.device), cap * sizeof(cf_attention_batch_item)), "device item buffer");
        slot.capacity = cap;
        r.reserved_bytes += static_cast<uint64_t>(cap) * sizeof(cf_attention_batch_item);
        ++r.counters.allocation_count;
        ++r.counters.pool_misses;
    } else {
        ++r.counters.pool_hits;
    }
    if (!slot.done) cuda_check(cudaEventCreateWithFlags(&slot.done, cudaEventDisableTiming), "event");
    std::memcpy(slot.host, items, count * sizeof(cf_attention_batch_item));
    cuda_check(cudaMemcpyAsync(slot.device, slot.host, count * sizeof(cf_attention_batch_item), cudaMemcpyHostToDevice, s),
               "upload batch items");
    r.counters.peak_reserved_bytes = std::max(r.counters.peak_reserved_bytes, r.reserved_bytes);
    r.counters.peak_live_bytes = std::max<uint64_t>(r.counters.peak_live_bytes, count * sizeof(cf_attention_batch_item));
    return slot;
}

void finish(Slot &slot, cudaStream_t s) {
    cuda_check(cudaEventRecord(slot.done, s), "record staging event");
    slot.pending = true;
}

void launch(cf_attention_runtime &r, bool optimized, const cf_attention_batch_item *device_items, uint32_t count,
            uint32_t max_tokens, cudaStream_t s) {
    const Shape shape{r.config.query_head_count, r.config.kv_head_count, r.config.head_dim, r.config.gqa_group_size};
    if (optimized) {
        if (!r.byte_counters) {
            cuda_check(cudaMalloc(reinterpret_cast<void **>(&r.byte_counters), 16), "byte counters");
            cuda_check(cudaMemsetAsync(r.byte_counters, 0, 16, s), "byte counters");
        }
        // split the pages of every item over enough blocks to fill the GPU when the batch alone does not
        if (r.sm_count == 0) {
            int device = 0;
            cuda_check(cudaGetDevice(&device), "cudaGetDevice");
            cuda_check(cudaDeviceGetAttribute(&r.sm_count, cudaDevAttrMultiProcessorCount, device), "SM count");
        }
        const uint64_t blocks = static_cast<uint64_t>(count) * shape.hkv * max_tokens;
        const uint32_t splits = static_cast<uint32_t>(std::min<uint64_t>(32, std::max<uint64_t>(1, (2ull * r.sm_count + blocks - 1) / blocks)));
        if (splits > 1) {
            const uint64_t floats = static_cast<uint64_t>(count) * max_tokens * shape.hq * splits * (shape.dim + 2u);
            if (r.partial_floats < floats) {
                if (r.partials) {
                    cuda_check(cudaStreamSynchronize(s), "drain before the partials grow");
                    cudaFree(r.partials);
                    r.partials = nullptr;
                    r.reserved_bytes -= r.partial_floats * 4;
                }
                cuda_check(cudaMalloc(reinterpret_cast<void **>(&r.partials), floats * 4), "split partials");
                r.partial_floats = floats;
                r.reserved_bytes += floats * 4;
                ++r.counters.allocation_count;
            }
        }
        batch_attention_kernel<<<dim3(count, shape.hkv * splits, max_tokens), kThreads, 0, s>>>(device_items, shape, r.byte_counters, splits,
                                                                                             r.partials);
        if (splits > 1) batch_combine_kernel<<<dim3(count, shape.hq, max_tokens), 128, 0, s>>>(device_items, shape, splits, r.partials);
        ++r.counters.optimized_launches;
    } else {
        plain_attention_kernel<<<dim3(count, shape.hq, max_tokens), 32, 0, s>>>(device_items, shape);
        ++r.counters.reference_launches;
    }
    cuda_check(cudaGetLastError(), "attention launch");
}

template <class F>
int guarded(cf_attention_runtime *r, F &&body) {
    try {
        body();
        r->error.clear();
        return 0;
    } catch (const std::invalid_argument &e) {
        r->error = e.what();
    } catch (const std::exception &e) {
        ++r->counters.cuda_errors;
        r->error = e.what();
    } catch (...) {
        r->error = "unknown error";
    }
    return -1;
}

}  // namespace

extern "C" cf_attention_runtime *cf_attention_runtime_create(const cf_attention_runtime_config *config) {
    if (!config || !config->layer_count || !config->query_head_count || !config->kv_head_count || !config->head_dim) return nullptr;
    if (config->query_head_count != config->kv_head_count * config->gqa_group_size) return nullptr;
    if (config->head_dim > 128) return nullptr;   // CF_KV_MAX_HEAD_DIM, include/chromofold/chromofold.h:22
    if (config->mode != CF_ATTENTION_REFERENCE && config->mode != CF_ATTENTION_OPTIMIZED) return nullptr;
    try {
        auto r = std::make_unique<cf_attention_runtime>();
        r->config = *config;
        return r.release();   // no CUDA call: device memory is taken on first use
    } catch (...) {
        return nullptr;
    }
}

extern "C" void cf_attention_runtime_destroy(cf_attention_runtime *r, void *stream) {
    if (!r) return;
    bool touched = r->byte_counters != nullptr;
    for (const Slot &slot : r->ring) touched = touched || slot.host != nullptr;
    if (touched) cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    for (Slot &slot : r->ring) {
        if (slot.pending) cudaEventSynchronize(slot.done);
        if (slot.done) cudaEventDestroy(slot.done);
        if (slot.host) cudaFreeHost(slot.host);
        if (slot.device) cudaFree(slot.device);
    }
    if (r->byte_counters) cudaFree(r->byte_counters);
    if (r->partials) cudaFree(r->partials);
    delete r;
}

extern "C" int cf_attention_execute_async(cf_attention_runtime *r, const cf_attention_batch_item *items, uint32_t count,
                                          void *stream) {
    if (!r || !items || !count) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> guard(r->mutex);
    return guarded(r, [&] {
        uint32_t max_tokens = 0;
        uint64_t rows = 0;
        validate_items(*r, items, count, &max_tokens, &rows);
        if (max_tokens == 0) return;
        Slot &slot = stage(*r, items, count, s);
        launch(*r, r->config.mode == CF_ATTENTION_OPTIMIZED, slot.device, count, max_tokens, s);
        finish(slot, s);
        if (rows > count) ++r->counters.prefill_launches;
        else ++r->counters.decode_launches;
        if (count > 1) {
            ++r->counters.grouped_batches;
            r->counters.grouped_items += count;
            r->counters.kernel_launches_avoided += count - 1;
        }
        for (uint32_t i = 0; i < count; ++i)
            r->counters.descriptor_bytes_read += static_cast<uint64_t>(items[i].sealed_page_count) * sizeof(cf_device_page_descriptor);
    });
}

extern "C" int cf_attention_compare_async(cf_attention_runtime *r, const cf_attention_batch_item *items, uint32_t count,
                                          float max_abs_error, float mean_abs_error, void *stream) {
    if (!r || !items || !count || !(max_abs_error > 0.0f) || !(mean_abs_error > 0.0f)) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> guard(r->mutex);
    return guarded(r, [&] {
        uint32_t max_tokens = 0;
        uint64_t rows = 0;
        validate_items(*r, items, count, &max_tokens, &rows);
        if (rows == 0) return;
        const uint64_t row_values = static_cast<uint64_t>(r->config.query_head_count) * r->config.head_dim;
        const uint64_t values = rows * row_values;
        r->scratch_a.ensure(values, s);
        r->scratch_b.ensure(values, s);
        r->compare_result.ensure(2, s);
        cuda_check(cudaMemsetAsync(r->compare_result.ptr, 0, 8, s), "clear comparison");
        for (int pass = 0; pass < 2; ++pass) {   // the same items, outputs redirected to dense fp32 scratch rows
            std::vector<cf_attention_batch_item> redirected(items, items + count);
            uint64_t row = 0;
            for (cf_attention_batch_item &it : redirected) {
                it.output = (pass ? r->scratch_b.ptr : r->scratch_a.ptr) + row * row_values;
                it.output_type = CF_DEVICE_F32;
                it.output_element_stride_bytes = 4;
                it.output_head_stride_bytes = 4ull * r->config.head_dim;
                it.output_token_stride_bytes = 4ull * row_values;
                row += it.query.token_count;
            }
            Slot &slot = stage(*r, redirected.data(), count, s);
            launch(*r, pass == 1, slot.device, count, max_tokens, s);
            finish(slot, s);
        }
        compare_kernel<<<148, 256, 0, s>>>(r->scratch_a.ptr, r->scratch_b.ptr, values, r->compare_result.ptr);
        cuda_check(cudaGetLastError(), "comparison launch");
        float result[2] = {0.0f, 0.0f};
        cuda_check(cudaMemcpyAsync(result, r->compare_result.ptr, 8, cudaMemcpyDeviceToHost, s), "read comparison");
        cuda_check(cudaStreamSynchronize(s), "wait for comparison");
        const float mean = result[1] / static_cast<float>(values);
        if (!(result[0] <= max_abs_error) || !(mean <= mean_abs_error)) {
            ++r->counters.numerical_failures;
            throw std::invalid_argument("optimized and reference outputs differ: max " + std::to_string(result[0]) + ", mean " +
                                        std::to_string(mean));
        }
    });
}

extern "C" int cf_attention_invalidate_graphs(cf_attention_runtime *r) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    ++r->counters.graph_invalidations;   // this runtime keeps no captured graphs: one launch per batch already
    return 0;
}

extern "C" int cf_attention_get_counters(const cf_attention_runtime *r, cf_attention_counters *counters) {
    if (!r || !counters) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (r->byte_counters) {   // device-side byte counts of the launches that have completed so far
        unsigned long long host[2] = {0, 0};
        if (cudaMemcpy(host, r->byte_counters, 16, cudaMemcpyDeviceToHost) == cudaSuccess) {
            r->counters.compressed_payload_bytes_read = host[0];
            r->counters.scale_bytes_read = host[1];
        }
    }
    *counters = r->counters;
    return 0;
}

extern "C" const char *cf_attention_last_error(const cf_attention_runtime *r) {
    return r ? r->error.c_str() : "runtime is null";
}
