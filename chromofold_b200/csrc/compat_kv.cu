// compat_kv.cu — the reference's CUDA entry points for this path, re-implemented for sm_100a
// (declared in include/chromofold_b200/compat_kv.h):
//   cf_kv_validate_paged_attention_desc / cf_kv_paged_attention_async   (src/cuda/paged_kv_attention.cu:280-327)
//   cf_rans_decode_async                                                (src/cuda/rans.cu:38-50)
// The descriptors are the reference's (one 104-byte descriptor per page and kv head, per-page LUTs, K per-channel and
// V per-token fp32 scales), so this path keeps their cost; it is split over the pages of a kv head to fill the GPU
// and runs faster than the reference's kernels on the same descriptors, but the sealed-KV entry points are the fast path.

#include <mutex>
#include <algorithm>
#include <math_constants.h>

#include "cf_device_common.cuh"
#include "chromofold_b200/compat_kv.h"

namespace cfb {
// Implemented in flat_rans_decode.cu
cudaError_t launch_flat_rans_decode(const uint8_t *data, const int32_t *byte_off, const uint32_t *state0, const int32_t *slot2sym,
                                    const int32_t *freq, const int32_t *cum, uint32_t groups, int32_t *out, cudaStream_t stream);
namespace {

constexpr int kThreads = 128;
constexpr uint32_t kBatchSymbols = 4096;   // symbols of one stream decoded to shared memory at a time
constexpr uint32_t kMaxGroup = 16;
constexpr float kLog2e = 1.4426950408889634f;

// Decode coded block `b` of a page stream and hand every symbol whose flat index lies in [lo, hi) to `emit`.
template <class Emit>
__device__ void decode_block_range(const uint32_t *words, const int32_t *offsets, const int32_t *lut, uint32_t maxlen,
                                   uint32_t fixed_bits, uint32_t block_size, uint32_t b, uint32_t total, uint32_t lo,
                                   uint32_t hi, Emit emit) {
    const uint32_t first = b * block_size;
    const uint32_t last = min(first + block_size, total);
    if (fixed_bits) {  // symbol i sits at bit i * fixed_bits, never crossing a word (kv_gpu_fixture.cpp:36-40)
        const uint32_t mask = (1u << fixed_bits) - 1u;
        uint32_t i = max(first, lo);
        const uint32_t end = min(last, hi);
        while (i < end) {   // one load per word, every symbol of the word that is wanted
            const uint32_t bit = i * fixed_bits;
            const uint32_t w = words[bit >> 5];
            uint32_t pos = bit & 31u;
            do {
                emit(i, (w >> ((32u - fixed_bits) - pos)) & mask);
                ++i;
                pos += fixed_bits;
            } while (pos + fixed_bits <= 32u && i < end);
        }
        return;
    }
    uint32_t bit = static_cast<uint32_t>(offsets[b]);
    for (uint32_t i = first; i < min(last, hi); ++i) {  // block_huffman_device.cuh:12-19, two words at a time
        const uint32_t w = bit >> 5, off = bit & 31u;
        uint32_t window = words[w] << off;
        if (off + maxlen > 32u) window |= words[w + 1] >> (32u - off);
        const uint32_t entry = static_cast<uint32_t>(lut[window >> (32u - maxlen)]);
        if (i >= lo) emit(i, entry & 0xffu);
        bit += entry >> 8;
    }
}

struct Smem {
    uint32_t off_ksym, off_vsym, off_q, off_qk, off_acc, off_scores, off_ml, off_alpha, off_scan, off_match, off_tokens, total;
};
__host__ __device__ inline Smem smem_layout(uint32_t group, uint32_t head_dim, uint32_t batch_tokens) {
    Smem s;
    s.off_ksym = 0;
    s.off_vsym = kBatchSymbols;
    s.off_q = 2 * kBatchSymbols;
    s.off_qk = s.off_q + group * head_dim * 4;
    s.off_acc = s.off_qk + group * head_dim * 4;
    s.off_scores = s.off_acc + group * head_dim * 4;
    s.off_ml = s.off_scores + group * batch_tokens * 4;
    s.off_alpha = s.off_ml + group * 8 + 16;         // per query head: factor of the running sums in the current update
    s.off_scan = s.off_alpha + group * 4 + 16;       // per-thread match counts of the descriptor scan
    s.off_match = s.off_scan + kThreads * 4;            // indices of this kv head's descriptors, in order (uint16)
    s.off_tokens = s.off_match + 2 * 4096;              // their token counts (uint32); a call names at most 4096 descriptors
    s.total = s.off_tokens + 4 * 4096 + 16;
    return s;
}

// One block per (query row, kv head, split): all query heads of the group share every decoded symbol.
// Split-KV: with `splits` > 1 block z of a (query row, kv head) takes every splits-th token batch of its head's pages (split 0 also the
// active tail) and leaves (max, sum, weighted[D]) per query head in `partials`, merged by compat_combine_kernel.
// The partials live in a fixed array inside the library image (this ABI has no workspace argument and its calls must
// not allocate): kCompatSlots slots, handed out in turn; a slot is reused only after the call that used it last has
// finished on the device (an event per slot, waited for on the new call's stream).
constexpr uint32_t kCompatSlots = 4;
constexpr uint32_t kCompatSlotFloats = 512u * 1024u;   // 2 MiB per slot
constexpr uint32_t kCompatMaxSplits = 64;
__device__ float g_compat_partials[kCompatSlots * kCompatSlotFloats];

__global__ void __launch_bounds__(kThreads) compat_paged_attention_kernel(cf_kv_paged_attention_desc desc,
                                                                          uint32_t batch_tokens, uint32_t splits,
                                                                          float *partials) {
    extern __shared__ __align__(16) uint8_t smem[];
    const uint32_t G = desc.gqa_group_size, D = desc.head_dim;
    const Smem lay = smem_layout(G, D, batch_tokens);
    uint8_t *ksym = smem + lay.off_ksym;
    uint8_t *vsym = smem + lay.off_vsym;
    float *q = reinterpret_cast<float *>(smem + lay.off_q);        // q * softmax_scale * log2(e)
    float *qk = reinterpret_cast<float *>(smem + lay.off_qk);      // q scaled by the page's per-channel K scales
    float *acc = reinterpret_cast<float *>(smem + lay.off_acc);
    float *scores = reinterpret_cast<float *>(smem + lay.off_scores);
    float *ml = reinterpret_cast<float *>(smem + lay.off_ml);
    float *alpha_s = reinterpret_cast<float *>(smem + lay.off_alpha);

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t query_row = blockIdx.x, kv_head = blockIdx.y, split = blockIdx.z;
    uint32_t batches_of_head = 0;   // token batches of this kv head's pages met so far: batch n belongs to split n % splits
    const uint32_t query_token = desc.query_token_begin + query_row;
    const uint32_t first_token = window_begin(query_token, desc.causal_window);

    for (uint32_t i = tid; i < G * D; i += kThreads) {
        const uint32_t head = kv_head * G + i / D;
        q[i] = desc.queries[(static_cast<uint64_t>(query_row) * desc.query_head_count + head) * D + i % D] *
               (desc.softmax_scale * kLog2e);
        acc[i] = 0.0f;
    }
    if (tid < G) {
        ml[2 * tid] = -CUDART_INF_F;
        ml[2 * tid + 1] = 0.0f;
    }
    __syncthreads();

    // Online-softmax update from scores[g][0..count). First the weights, once: warp w takes query heads w, w + 4, ...,
    // its lanes the tokens; scores[g][t] becomes exp2(s - max) * scale_of(t) (the V scale of the token rides on the
    // weight) and (max, sum) move on. Then thread d adds its channel: acc[g][d] = acc * alpha + sum_t weight * value.
    auto update = [&](uint32_t count, auto raw_value_of, auto scale_of) {
        for (uint32_t g = warp; g < G; g += kThreads / 32) {
            float *row = scores + g * batch_tokens;
            const float m_old = ml[2 * g], l_old = ml[2 * g + 1];
            float pm = -CUDART_INF_F;
            for (uint32_t t = lane; t < count; t += 32) pm = fmaxf(pm, row[t]);
            const float m_new = fmaxf(m_old, warp_max(pm));
            float lsum = 0.0f;
            for (uint32_t t = lane; t < count; t += 32) {
                const float sc = row[t];
                const float w = sc == -CUDART_INF_F ? 0.0f : exp2f(sc - m_new);   // m_new is finite whenever sc is
                lsum += w;
                row[t] = w * scale_of(t);
            }
            lsum = warp_sum(lsum);
            if (lane == 0) {
                const float alpha = m_old == -CUDART_INF_F ? 0.0f : exp2f(m_old - m_new);   // nothing visible so far: 0 * 0
                ml[2 * g] = m_new;
                ml[2 * g + 1] = m_new == -CUDART_INF_F ? l_old : l_old * alpha + lsum;
                alpha_s[g] = m_new == -CUDART_INF_F ? 1.0f : alpha;
            }
        }
        __syncthreads();
        if (tid < D) {
            for (uint32_t g = 0; g < G; ++g) {
                const float *row = scores + g * batch_tokens;
                float a0 = 0.0f, a1 = 0.0f;
                uint32_t t = 0;
                for (; t + 1 < count; t += 2) {
                    a0 += row[t] * raw_value_of(t, tid);
                    a1 += row[t + 1] * raw_value_of(t + 1, tid);
                }
                if (t < count) a0 += row[t] * raw_value_of(t, tid);
                acc[g * D + tid] = acc[g * D + tid] * alpha_s[g] + (a0 + a1);
            }
        }
        __syncthreads();
    };

    // The descriptors of this kv head, found by all threads at once (a serial walk over up to 4096 descriptors in global
    // memory would cost one memory latency each): thread t looks at a contiguous run and the runs' matches are
    // concatenated in order.
    uint32_t *scan = reinterpret_cast<uint32_t *>(smem + lay.off_scan);
    uint16_t *match = reinterpret_cast<uint16_t *>(smem + lay.off_match);
    uint32_t *match_tokens = reinterpret_cast<uint32_t *>(smem + lay.off_tokens);
    const uint32_t run = (desc.page_count + kThreads - 1) / kThreads;
    const uint32_t run_begin = min(tid * run, desc.page_count), run_end = min(run_begin + run, desc.page_count);
    uint32_t mine = 0;
    for (uint32_t pi = run_begin; pi < run_end; ++pi) mine += desc.pages[pi].kv_head == kv_head && desc.pages[pi].head_dim == D;
    scan[tid] = mine;
    __syncthreads();
    uint32_t before = 0, matches = 0;
    for (uint32_t t = 0; t < kThreads; ++t) {
        const uint32_t n = scan[t];
        before += t < tid ? n : 0u;
        matches += n;
    }
    for (uint32_t pi = run_begin; pi < run_end; ++pi)
        if (desc.pages[pi].kv_head == kv_head && desc.pages[pi].head_dim == D) {
            match[before] = static_cast<uint16_t>(pi);
            match_tokens[before++] = desc.pages[pi].token_count;
        }
    __syncthreads();

    for (uint32_t mi = 0; mi < matches; ++mi) {
        // Two fields decide whether any token batch of the page is this split's; only then is the descriptor read whole.
        // Every block counts the batches of every page of the head the same way, whether it works on them or not.
        const uint32_t page_batches = (match_tokens[mi] + batch_tokens - 1) / batch_tokens;
        const uint32_t first_mine = (split + splits - batches_of_head % splits) % splits;   // offset of this split's next batch
        if (first_mine >= page_batches) {
            batches_of_head += page_batches;
            continue;
        }
        const cf_kv_device_page page = desc.pages[match[mi]];
        if (page.token_begin > query_token || page.token_begin + page.token_count <= first_token) {
            batches_of_head += page_batches;
            continue;
        }
        const uint32_t total = page.token_count * D;
        const int zp = static_cast<int>(page.zero_point);
        bool scaled = false;   // the page's K scales are folded into the queries when its first batch comes up
        for (uint32_t t0 = 0; t0 < page.token_count; t0 += batch_tokens) {
            if (batches_of_head++ % splits != split) continue;
            if (!scaled) {
                __syncthreads();   // the previous page's readers of qk are done
                for (uint32_t i = tid; i < G * D; i += kThreads) qk[i] = q[i] * page.k_scales[i % D];
                scaled = true;
            }
            const uint32_t count = min(batch_tokens, page.token_count - t0);
            const uint32_t lo = t0 * D, hi = (t0 + count) * D;
            const uint32_t b_first = lo / page.block_size, b_last = (hi - 1) / page.block_size;
            __syncthreads();
            for (uint32_t job = tid; job < 2 * (b_last - b_first + 1); job += kThreads) {
                const uint32_t b = b_first + (job >> 1);
                if (job & 1)
                    decode_block_range(page.v_words, page.v_block_offsets, page.v_lut, page.v_max_code_length,
                                       page.fixed_code_length, page.block_size, b, total, lo, hi,
                                       [&](uint32_t i, uint32_t s) { vsym[i - lo] = static_cast<uint8_t>(s); });
                else
                    decode_block_range(page.k_words, page.k_block_offsets, page.k_lut, page.k_max_code_length,
                                       page.fixed_code_length, page.block_size, b, total, lo, hi,
                                       [&](uint32_t i, uint32_t s) { ksym[i - lo] = static_cast<uint8_t>(s); });
            }
            __syncthreads();
            for (uint32_t t = warp; t < count; t += kThreads / 32) {   // a warp per token: its codes are read once for all heads
                const uint32_t token = page.token_begin + t0 + t;
                const bool visible = token >= first_token && token <= query_token;
                float k[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t d = lane + 32u * j;
                    k[j] = visible && d < D ? static_cast<float>(static_cast<int>(ksym[t * D + d]) - zp) : 0.0f;
                }
                for (uint32_t g = 0; g < G; ++g) {
                    float dot = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const uint32_t d = lane + 32u * j;
                        if (d < D) dot += qk[g * D + d] * k[j];
                    }
                    dot = warp_sum(dot);
                    if (lane == 0) scores[g * batch_tokens + t] = visible ? dot : -CUDART_INF_F;
                }
            }
            __syncthreads();
            update(count, [&](uint32_t t, uint32_t d) { return static_cast<float>(static_cast<int>(vsym[t * D + d]) - zp); },
                   [&](uint32_t t) { return page.v_scales[t0 + t]; });
        }
    }

    // dense fp32 tail [active_token_count][kv_head_count][head_dim] (paged_kv_attention.cu:154-166)
    const uint32_t tail_tokens = split == 0 ? desc.active_token_count : 0u;
    for (uint32_t t0 = 0; t0 < tail_tokens; t0 += batch_tokens) {
        const uint32_t count = min(batch_tokens, tail_tokens - t0);
        __syncthreads();
        for (uint32_t pair = warp; pair < G * count; pair += kThreads / 32) {
            const uint32_t g = pair / count, t = pair % count;
            const uint32_t token = desc.active_token_begin + t0 + t;
            float s = -CUDART_INF_F;
            if (token >= first_token && token <= query_token) {
                const float *row = desc.active_k + (static_cast<uint64_t>(t0 + t) * desc.kv_head_count + kv_head) * D;
                float dot = 0.0f;
                for (uint32_t d = lane; d < D; d += 32) dot += q[g * D + d] * row[d];
                s = warp_sum(dot);
            }
            if (lane == 0) scores[g * batch_tokens + t] = s;
        }
        __syncthreads();
        update(count,
               [&](uint32_t t, uint32_t d) { return desc.active_v[(static_cast<uint64_t>(t0 + t) * desc.kv_head_count + kv_head) * D + d]; },
               [&](uint32_t) { return 1.0f; });
    }

    if (splits > 1) {
        for (uint32_t i = tid; i < G * D; i += kThreads) {
            const uint32_t g = i / D;
            float *dst = partials + ((static_cast<uint64_t>(query_row) * desc.query_head_count + kv_head * G + g) * splits + split) * (D + 2u);
            if (i % D == 0) {
                dst[0] = ml[2 * g];
                dst[1] = ml[2 * g + 1];
            }
            dst[2 + i % D] = acc[i];
        }
        return;
    }
    for (uint32_t i = tid; i < G * D; i += kThreads) {
        const uint32_t g = i / D;
        const float l = ml[2 * g + 1];
        desc.output[(static_cast<uint64_t>(query_row) * desc.query_head_count + kv_head * G + g) * D + i % D] =
            l > 0.0f ? acc[i] / l : 0.0f;  // no visible token: zeros (paged_kv_attention.cu:170-173)
    }
}

// One block per (query row, query head): merges the splits' partials (cf_online_softmax_merge rule, scores in log2 units).
__global__ void compat_combine_kernel(float *output, const float *partials, uint32_t query_heads, uint32_t head_dim, uint32_t splits) {
    __shared__ float weight[kCompatMaxSplits];
    __shared__ float total;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * query_heads + blockIdx.y;
    const uint32_t stride = head_dim + 2u;
    const float *src = partials + row * splits * stride;
    if (threadIdx.x < 32) {   // one warp: the splits' maxima and sums, in parallel over the splits
        float m = -CUDART_INF_F;
        for (uint32_t s = threadIdx.x; s < splits; s += 32) m = fmaxf(m, src[s * stride]);
        m = warp_max(m);
        float l = 0.0f;
        for (uint32_t s = threadIdx.x; s < splits; s += 32) {
            const float ms = src[s * stride];
            const float w = ms == -CUDART_INF_F ? 0.0f : exp2f(ms - m);
            weight[s] = w;
            l += src[s * stride + 1] * w;
        }
        l = warp_sum(l);
        if (threadIdx.x == 0) total = l;
    }
    __syncthreads();
    const float l = total;
    for (uint32_t d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float a = 0.0f;
#pragma unroll 8
        for (uint32_t s = 0; s < splits; ++s) a += src[s * stride + 2 + d] * weight[s];   // independent loads
        output[row * head_dim + d] = l > 0.0f ? a / l : 0.0f;   // no visible token: zeros
    }
}

// One thread per coded block (rans.cu:28-36), recurrence of rans.cu:20-23.
__global__ void compat_rans_decode_kernel(const uint8_t *data, const int32_t *byte_off, const uint32_t *state0,
                                          const int32_t *slot2sym, const int32_t *freq, const int32_t *cum, int block,
                                          int n, int32_t *out, int first_block) {
    const int b = first_block + blockIdx.x * blockDim.x + threadIdx.x;
    const long long base = static_cast<long long>(b) * block;
    if (base >= n) return;
    const int count = static_cast<int>(min(static_cast<long long>(block), n - base));
    uint32_t x = state0[b];
    const uint8_t *bytes = data + byte_off[b];
    for (int j = 0; j < count; ++j) {
        const uint32_t slot = x & (CF_B200_RANS_M - 1u);
        const int s = __ldg(slot2sym + slot);
        x = static_cast<uint32_t>(__ldg(freq + s)) * (x >> CF_B200_RANS_PROB_BITS) + slot - static_cast<uint32_t>(__ldg(cum + s));
        while (x < kRansL) x = (x << 8) | *bytes++;
        out[base + j] = s;
    }
}

// ---- flat (non-paged) windowed attention over block-Huffman K / V: the reference's M6 entry points -------------------
// (src/cuda/fused_kv_attention.cu:26-161). One block per query row. Both entry points run the SAME arithmetic in the
// same order — scores by one thread per window row, serial over channels; output by one thread per channel, serial
// over window rows — so the fused result equals the decode-then-dense result bit for bit, as the reference promises
// for its own pair. The fused kernel decodes the window's rows to symbols in shared memory (never to global memory).
constexpr int kFlatThreads = 128;

// Bit position of flat element `flat`: its block's offset plus a skip-decode inside the block (fused_kv_attention.cu:16-23).
__device__ uint32_t flat_row_position(const uint32_t *words, const int32_t *boff, const int32_t *lut, int maxlen, int block,
                                      long flat) {
    const int b = static_cast<int>(flat / block);
    uint32_t bit = static_cast<uint32_t>(boff[b]);
    const int skip = static_cast<int>(flat - static_cast<long>(b) * block);
    for (int i = 0; i < skip; ++i) {
        const uint32_t w = bit >> 5, off = bit & 31u;
        uint32_t window = words[w] << off;
        if (off + maxlen > 32u) window |= words[w + 1] >> (32u - off);
        bit += static_cast<uint32_t>(lut[window >> (32u - maxlen)]) >> 8;
    }
    return bit;
}

template <class Emit>
__device__ void flat_decode_row(const uint32_t *words, const int32_t *lut, int maxlen, uint32_t bit, int dim, Emit emit) {
    for (int c = 0; c < dim; ++c) {
        const uint32_t w = bit >> 5, off = bit & 31u;
        uint32_t window = words[w] << off;
        if (off + maxlen > 32u) window |= words[w + 1] >> (32u - off);
        const uint32_t e = static_cast<uint32_t>(lut[window >> (32u - maxlen)]);
        emit(c, static_cast<int>(e & 0xffu));
        bit += e >> 8;
    }
}

struct FlatArgs {
    const uint32_t *kw, *vw;
    const int32_t *kb, *kl, *vb, *vl;
    int kmax, vmax;
    const float *kscale, *vscale, *Q, *Kd, *Vd;
    float *out;
    int seq, dim, nq, window, block, zero;
    float sscale;
};

template <bool kFused>
__global__ void __launch_bounds__(kFlatThreads) flat_attention_kernel(FlatArgs a) {
    extern __shared__ __align__(16) uint8_t smem[];
    float *q = reinterpret_cast<float *>(smem);                        // [dim]
    float *sc = q + CF_KV_MAX_HEAD_DIM;                                 // [window]
    uint8_t *ksym = reinterpret_cast<uint8_t *>(sc + CF_KV_MAX_WINDOW); // [window][dim]   (fused only)
    uint8_t *vsym = ksym + static_cast<size_t>(a.window) * a.dim;
    __shared__ float s_inv;
    const int i = blockIdx.x, tid = threadIdx.x;
    const int lo = max(0, i - a.window + 1), nk = i - lo + 1;
    for (int c = tid; c < a.dim; c += kFlatThreads) q[c] = a.Q[static_cast<long>(i) * a.dim + c];
    if (kFused) {
        for (int job = tid; job < 2 * nk; job += kFlatThreads) {
            const int jj = job >> 1, j = lo + jj;
            if (job & 1) {
                const uint32_t bit = flat_row_position(a.vw, a.vb, a.vl, a.vmax, a.block, static_cast<long>(j) * a.dim);
                flat_decode_row(a.vw, a.vl, a.vmax, bit, a.dim, [&](int c, int s) { vsym[jj * a.dim + c] = static_cast<uint8_t>(s); });
            } else {
                const uint32_t bit = flat_row_position(a.kw, a.kb, a.kl, a.kmax, a.block, static_cast<long>(j) * a.dim);
                flat_decode_row(a.kw, a.kl, a.kmax, bit, a.dim, [&](int c, int s) { ksym[jj * a.dim + c] = static_cast<uint8_t>(s); });
            }
        }
    }
    __syncthreads();
    auto k_at = [&](int jj, int c) {
        return kFused ? static_cast<float>(static_cast<int>(ksym[jj * a.dim + c]) - a.zero) * a.kscale[c]
                      : a.Kd[static_cast<long>(lo + jj) * a.dim + c];
    };
    auto v_at = [&](int jj, int c) {
        return kFused ? static_cast<float>(static_cast<int>(vsym[jj * a.dim + c]) - a.zero) * a.vscale[lo + jj]
                      : a.Vd[static_cast<long>(lo + jj) * a.dim + c];
    };
    for (int jj = tid; jj < nk; jj += kFlatThreads) {
        float s = 0.0f;
        for (int c = 0; c < a.dim; ++c) s += q[c] * k_at(jj, c);
        sc[jj] = s * a.sscale;
    }
    __syncthreads();
    if (tid == 0) {  // serial max and sum: the order is part of the bit-identity contract
        float mx = -1e30f;
        for (int jj = 0; jj < nk; ++jj) mx = fmaxf(mx, sc[jj]);
        float sum = 0.0f;
        for (int jj = 0; jj < nk; ++jj) {
            sc[jj] = expf(sc[jj] - mx);
            sum += sc[jj];
        }
        s_inv = 1.0f / sum;
    }
    __syncthreads();
    for (int c = tid; c < a.dim; c += kFlatThreads) {
        float acc = 0.0f;
        for (int jj = 0; jj < nk; ++jj) acc += (sc[jj] * s_inv) * v_at(jj, c);
        a.out[static_cast<long>(i) * a.dim + c] = acc;
    }
}

// Decode-then-dense stage 1: one thread per row writes dequantised fp32 rows (fused_kv_attention.cu:69-81).
__global__ void flat_decode_dense_kernel(const uint32_t *words, const int32_t *boff, const int32_t *lut, int maxlen, int block,
                                         int seq, int dim, int zero, const float *scale, int per_token, float *dense) {
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= seq) return;
    const uint32_t bit = flat_row_position(words, boff, lut, maxlen, block, static_cast<long>(j) * dim);
    flat_decode_row(words, lut, maxlen, bit, dim, [&](int c, int s) {
        dense[static_cast<long>(j) * dim + c] = static_cast<float>(s - zero) * (per_token ? scale[j] : scale[c]);
    });
}

cf_status flat_validate(const void *kw, const void *kb, const void *kl, int kmax, const void *vw, const void *vb,
                        const void *vl, int vmax, const void *kscale, const void *vscale, const void *Q, const void *out,
                        int seq, int dim, int nq, int window, int block, float sscale) {  // fused_kv_attention.cu:115-126
    if (!kw || !kb || !kl || !vw || !vb || !vl || !kscale || !vscale || !Q || !out) return CF_ERR_INVALID_ARGUMENT;
    if (seq <= 0 || dim <= 0 || nq < 0 || nq > seq || window <= 0 || block <= 0 || kmax <= 0 || vmax <= 0)
        return CF_ERR_INVALID_ARGUMENT;
    if (!(sscale == sscale) || sscale - sscale != 0.0f) return CF_ERR_INVALID_ARGUMENT;
    if (dim > CF_KV_MAX_HEAD_DIM || window > CF_KV_MAX_WINDOW || kmax > 24 || vmax > 24) return CF_ERR_UNSUPPORTED;
    return CF_OK;
}

bool finite_float(float v) { return v == v && v - v == 0.0f; }

}  // namespace
}  // namespace cfb

extern "C" cf_status cf_kv_validate_paged_attention_desc(const cf_kv_paged_attention_desc *d) {
    if (!d || d->struct_size != sizeof(cf_kv_paged_attention_desc) || d->abi_version != CF_KV_CUDA_ABI_VERSION ||
        !d->queries || !d->output || d->query_count == 0 || d->query_head_count == 0 || d->kv_head_count == 0 ||
        d->gqa_group_size == 0 || d->head_dim == 0 || d->head_dim > CF_KV_MAX_HEAD_DIM || !cfb::finite_float(d->softmax_scale))
        return CF_ERR_INVALID_ARGUMENT;
    if (d->query_head_count != d->kv_head_count * d->gqa_group_size || d->page_count > CF_KV_CUDA_MAX_PAGES_PER_LAUNCH ||
        (d->page_count != 0 && !d->pages) || (d->active_token_count != 0 && (!d->active_k || !d->active_v)))
        return CF_ERR_INVALID_ARGUMENT;
    if (d->query_token_begin > UINT32_MAX - d->query_count || d->active_token_begin > UINT32_MAX - d->active_token_count)
        return CF_ERR_INVALID_ARGUMENT;
    return CF_OK;
}

namespace {
// Slots of the partials array, per device: whose turn it is and when the slot's last user is done.
struct CompatSlots {
    std::mutex lock;
    bool made = false;
    cudaEvent_t done[cfb::kCompatSlots] = {};
    float *base = nullptr;
    uint32_t next = 0;
    int sm_count = 0;
};
CompatSlots g_compat_slots[64];
}  // namespace

// The pages of a kv head are dealt out to enough splits to fill the GPU: a decode step has only kv_head_count
// (query row, kv head) pairs.
extern "C" cf_status cf_kv_paged_attention_async(const cf_kv_paged_attention_desc *d, void *stream) {
    const cf_status valid = cf_kv_validate_paged_attention_desc(d);
    if (valid != CF_OK) return valid;
    if (d->gqa_group_size > cfb::kMaxGroup) return CF_ERR_UNSUPPORTED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const uint32_t batch_tokens = cfb::kBatchSymbols / d->head_dim;
    const cfb::Smem lay = cfb::smem_layout(d->gqa_group_size, d->head_dim, batch_tokens);
    if (cudaFuncSetAttribute(cfb::compat_paged_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(lay.total)) != cudaSuccess)
        return CF_ERR_CUDA;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return CF_ERR_CUDA;
    uint32_t splits = 1, slot = 0;
    CompatSlots *slots = device >= 0 && device < 64 ? &g_compat_slots[device] : nullptr;
    cudaStreamCaptureStatus capture = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &capture) != cudaSuccess) return CF_ERR_CUDA;
    if (capture != cudaStreamCaptureStatusNone) slots = nullptr;   // a captured call keeps to one launch and no events
    if (slots) {
        std::lock_guard<std::mutex> guard(slots->lock);
        if (!slots->made) {   // first call on this device: events, the array's address, the SM count
            for (cudaEvent_t &e : slots->done)
                if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return CF_ERR_CUDA;
            if (cudaGetSymbolAddress(reinterpret_cast<void **>(&slots->base), cfb::g_compat_partials) != cudaSuccess ||
                cudaDeviceGetAttribute(&slots->sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
                return CF_ERR_CUDA;
            slots->made = true;
        }
        const uint64_t pairs = static_cast<uint64_t>(d->query_count) * d->kv_head_count;
        const uint64_t room = cfb::kCompatSlotFloats / (static_cast<uint64_t>(d->query_count) * d->query_head_count * (d->head_dim + 2u));
        const uint64_t wanted = (2ull * slots->sm_count + pairs - 1) / pairs;
        splits = static_cast<uint32_t>(std::max<uint64_t>(1, std::min({wanted, room, static_cast<uint64_t>(cfb::kCompatMaxSplits)})));
        if (splits > 1) {
            slot = slots->next++ % cfb::kCompatSlots;
            if (cudaStreamWaitEvent(s, slots->done[slot], 0) != cudaSuccess) return CF_ERR_CUDA;   // the slot's last user
        }
    }
    float *partials = splits > 1 ? slots->base + static_cast<size_t>(slot) * cfb::kCompatSlotFloats : nullptr;
    cfb::compat_paged_attention_kernel<<<dim3(d->query_count, d->kv_head_count, splits), cfb::kThreads, lay.total, s>>>(
        *d, batch_tokens, splits, partials);
    if (splits > 1) {
        cfb::compat_combine_kernel<<<dim3(d->query_count, d->query_head_count), 128, 0, s>>>(d->output, partials, d->query_head_count,
                                                                                          d->head_dim, splits);
        if (cudaEventRecord(slots->done[slot], s) != cudaSuccess) return CF_ERR_CUDA;
    }
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}

extern "C" cf_status cf_rans_decode_async(const uint8_t *data, const int32_t *byte_off, const uint32_t *state0,
                                          const int32_t *slot2sym, const int32_t *freq, const int32_t *cum, int block,
                                          int n, int32_t *out, void *stream) {
    if (!data || !byte_off || !state0 || !slot2sym || !freq || !cum || !out) return CF_ERR_INVALID_ARGUMENT;
    if (block <= 0 || n < 0) return CF_ERR_INVALID_ARGUMENT;
    if (n == 0) return CF_OK;
    const int blocks = (n + block - 1) / block;
    int first_block = 0;
    if (block == 64 && blocks > 64) {   // whole groups of 64 blocks: the lane-per-block decoder (flat_rans_decode.cu)
        const uint32_t groups = static_cast<uint32_t>(blocks - 1) / 64u;
        if (cfb::launch_flat_rans_decode(data, byte_off, state0, slot2sym, freq, cum, groups, out, static_cast<cudaStream_t>(stream)) !=
            cudaSuccess)
            return CF_ERR_CUDA;
        first_block = static_cast<int>(groups * 64u);
    }
    cfb::compat_rans_decode_kernel<<<(blocks - first_block + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        data, byte_off, state0, slot2sym, freq, cum, block, n, out, first_block);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}

extern "C" cf_status cf_kv_attn_fused_async(const uint32_t *kw, const int32_t *kb, const int32_t *kl, int kmax,
                                            const uint32_t *vw, const int32_t *vb, const int32_t *vl, int vmax,
                                            const float *kscale, const float *vscale, const float *Q, float *out, int seq,
                                            int dim, int nq, int window, int block, int zero, float sscale, void *stream) {
    const cf_status valid = cfb::flat_validate(kw, kb, kl, kmax, vw, vb, vl, vmax, kscale, vscale, Q, out, seq, dim, nq, window,
                                               block, sscale);
    if (valid != CF_OK) return valid;
    if (nq == 0) return CF_OK;
    const cfb::FlatArgs a{kw, vw, kb, kl, vb, vl, kmax, vmax, kscale, vscale, Q, nullptr, nullptr, out,
                          seq, dim, nq, window, block, zero, sscale};
    const size_t smem = (CF_KV_MAX_HEAD_DIM + CF_KV_MAX_WINDOW) * sizeof(float) + 2 * static_cast<size_t>(window) * dim;
    if (cudaFuncSetAttribute(cfb::flat_attention_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
        return CF_ERR_CUDA;
    cfb::flat_attention_kernel<true><<<nq, cfb::kFlatThreads, smem, static_cast<cudaStream_t>(stream)>>>(a);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}

extern "C" cf_status cf_kv_attn_dense_async(const uint32_t *kw, const int32_t *kb, const int32_t *kl, int kmax,
                                            const uint32_t *vw, const int32_t *vb, const int32_t *vl, int vmax,
                                            const float *kscale, const float *vscale, const float *Q, float *Kd, float *Vd,
                                            float *out, int seq, int dim, int nq, int window, int block, int zero,
                                            float sscale, void *stream) {
    const cf_status valid = cfb::flat_validate(kw, kb, kl, kmax, vw, vb, vl, vmax, kscale, vscale, Q, out, seq, dim, nq, window,
                                               block, sscale);
    if (valid != CF_OK) return valid;
    if (!Kd || !Vd) return CF_ERR_INVALID_ARGUMENT;
    if (nq == 0) return CF_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cfb::flat_decode_dense_kernel<<<(seq + 63) / 64, 64, 0, s>>>(kw, kb, kl, kmax, block, seq, dim, zero, kscale, 0, Kd);
    cfb::flat_decode_dense_kernel<<<(seq + 63) / 64, 64, 0, s>>>(vw, vb, vl, vmax, block, seq, dim, zero, vscale, 1, Vd);
    const cfb::FlatArgs a{kw, vw, kb, kl, vb, vl, kmax, vmax, kscale, vscale, Q, Kd, Vd, out,
                          seq, dim, nq, window, block, zero, sscale};
    const size_t smem = (CF_KV_MAX_HEAD_DIM + CF_KV_MAX_WINDOW) * sizeof(float);
    cfb::flat_attention_kernel<false><<<nq, cfb::kFlatThreads, smem, s>>>(a);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}
