// sealed_attention.cu — decode-step attention over sealed pages: planning, the any-geometry kernel, the split-KV
// combine, the decode probe, and the C entry points.
//
// The arithmetic follows the reference's paged attention (src/cuda/paged_kv_attention.cu:41-176): dequantise inside
// the dot product, one online softmax over every page and the tail, output = weighted / sum. What differs is the
// execution: sequences are cut into chunks of pages, each (chunk, kv head) unit is processed independently for all
// query heads of the group at once (a K/V code is decoded once, not once per query head), and the partial
// (max, sum, weighted) triples are merged with the rule of cf_online_softmax_merge (src/runtime/kv_runtime.cpp:219-243).

#include <atomic>
#include <math_constants.h>

#include "attention_params.cuh"

static std::atomic<unsigned long long> g_shared_prefix_launches{0};

namespace cfb {

namespace {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kPlanThreads = 1024;
constexpr uint32_t kPlanCache = 2048;   // batch entries whose page ranges the plan kernel keeps in shared memory
constexpr int kGenericThreads = 128;
constexpr uint32_t kGenericMaxGroup = 16;

// ---------------------------------------------------------------------------------------------------------------
// Plan: how many chunks each sequence gets. One block.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t visible_pages(const AttentionParams &p, uint32_t seq, uint32_t *first_page,
                                                  uint32_t shared_pages = 0) {
    const uint32_t slot = slot_of(p, seq);
    const uint32_t sealed = p.seq_sealed_tokens[slot];
    const uint32_t tail = p.tail_tokens ? p.tail_tokens[slot] : 0u;
    const uint32_t qpos = query_position(p, seq, sealed, tail);
    const uint32_t pages = min((sealed + p.page_tokens - 1u) / p.page_tokens, qpos / p.page_tokens + 1u);
    const uint32_t first = min(max(window_begin(qpos, p.causal_window) / p.page_tokens, shared_pages), pages);
    if (first_page) *first_page = first;
    return pages - first;
}

// Shared-prefix hint, part one: block s compares the first `shared_prefix_pages` ids of entry s's page-table row with the
// first entry's and leaves the result (1 = differs) in the entry's cell of the chunk-prefix array, which the plan kernel
// reads before it overwrites the array with the real prefix sums.
__global__ void __launch_bounds__(256) verify_prefix_kernel(AttentionParams p) {
    const uint32_t s = blockIdx.x;
    const uint32_t *row0 = p.page_table + static_cast<uint64_t>(slot_of(p, 0)) * p.page_table_stride;
    const uint32_t *row = p.page_table + static_cast<uint64_t>(slot_of(p, s)) * p.page_table_stride;
    int bad = 0;
    for (uint32_t pg = threadIdx.x; pg < p.shared_prefix_pages; pg += blockDim.x) bad |= row[pg] != row0[pg];
    bad = __syncthreads_or(bad);
    if (threadIdx.x == 0) chunk_prefix(p)[s] = bad ? 1u : 0u;
}

__global__ void __launch_bounds__(kPlanThreads) plan_kernel(AttentionParams p) {
    __shared__ uint32_t scan[kPlanThreads];
    __shared__ uint32_t warp_totals[kPlanThreads / 32];
    __shared__ uint32_t s_visible[kPlanCache], s_first[kPlanCache];
    __shared__ uint32_t s_total;
    static_assert(kPlanThreads == 1024, "the block scan below is 32 warps of 32 lanes");
    const uint32_t tid = threadIdx.x;
    const uint32_t per_thread = (p.seq_count + kPlanThreads - 1) / kPlanThreads;
    const uint32_t begin = min(tid * per_thread, p.seq_count);
    const uint32_t end = min(begin + per_thread, p.seq_count);
    PlanHeader *hdr = plan_header(p);
    uint32_t *prefix = chunk_prefix(p);

    // Shared prefix: taken only if every listed sequence has the pages sealed and its page-table row starts with the
    // same ids as the first sequence's (compared by verify_prefix_kernel, result per entry in prefix[]). The pages are
    // then cut into chunks for the shared-prefix kernel and left out of the per-sequence chunks below.
    uint32_t shared = p.shared_prefix_pages;
    if (shared) {
        int bad = 0;
        for (uint32_t s = begin; s < end; ++s) {   // the pages must be sealed and wholly visible to the entry's query token
            const uint32_t slot = slot_of(p, s), sealed = p.seq_sealed_tokens[slot];
            const uint32_t qpos = query_position(p, s, sealed, p.tail_tokens ? p.tail_tokens[slot] : 0u);
            if (sealed / p.page_tokens < shared || qpos + 1u < shared * p.page_tokens || prefix[s] != 0u) bad = 1;
        }
        if (__syncthreads_or(bad)) {
            shared = 0;
            if (tid == 0) raise_status(p, CF_B200_DEVSTAT_PREFIX_MISMATCH);
        }
    }
    uint32_t shared_ctas = 0, shared_rounds = 0;
    if (shared) {   // an even split of the prefix's rounds over the CTAs of the shared-prefix kernel (SharedSplit)
        const uint32_t row_tiles = (p.seq_count * p.group + 127u) / 128u;
        shared_rounds = (shared + 7u) / 8u;
        shared_ctas = shared_split_ctas(shared_rounds, p.kv_head_span * row_tiles, p.sm_count, CF_B200_SHARED_CHUNKS_MAX);
        if (shared_ctas == 0u) shared = 0;   // no CTA to take it: the pages stay with the per-sequence chunks
    }

    // The visible page range of every batch entry is needed by each pass below; it costs a chain of dependent loads
    // (slot, sealed tokens, tail tokens, query position), so batches of up to kPlanCache entries keep it in shared memory.
    const bool cached = p.seq_count <= kPlanCache;
    if (cached) {
        for (uint32_t s = tid; s < p.seq_count; s += kPlanThreads) {
            uint32_t first_page;
            s_visible[s] = visible_pages(p, s, &first_page, shared);
            s_first[s] = first_page;
        }
        __syncthreads();
    }
    auto visible_of = [&](uint32_t s, uint32_t *first_page) {
        if (!cached) return visible_pages(p, s, first_page, shared);
        if (first_page) *first_page = s_first[s];
        return s_visible[s];
    };

    uint32_t pages_per_unit = p.min_pages_per_unit;
    uint32_t overflow = 0;
    uint32_t local = 0;  // chunks of this thread's sequences at the current pages_per_unit
    if (pages_per_unit == 0u) {
        // The library's choice. Units are equal-sized and handed out dynamically to W resident warps, so a launch lasts
        // about ceil(units / W) rounds of one unit each; a unit costs its pages plus a start-up worth about three
        // quarters of a page. Warp w scores the candidate 4 + w pages per unit over all sequences; the cheapest that
        // fits the workspace wins (ties: the larger unit, fewer partials to merge). A launch too small to give every
        // warp a unit comes out at 4.
        const uint32_t warp = tid >> 5, lane = tid & 31u, candidate = 4u + warp;
        uint64_t units = 0;
        for (uint32_t s = lane; s < p.seq_count; s += 32u) units += (visible_of(s, nullptr) + candidate - 1u) / candidate;
        for (int o = 16; o > 0; o >>= 1) units += __shfl_xor_sync(0xffffffffu, units, o);
        const uint32_t pass_heads = p.group <= 4u ? 4u : p.query_type == CF_B200_F32 ? 4u : 8u;
        const uint64_t warps = 16ull * (p.sm_count ? p.sm_count : 148u);
        const uint64_t rounds = (units * p.kv_head_span * ((p.group + pass_heads - 1u) / pass_heads) + warps - 1ull) / warps;
        uint64_t cost = rounds * (4ull * candidate + 3ull);
        if (units > p.layout.chunk_capacity || units == 0) cost = ~0ull;
        if (lane == 0) reinterpret_cast<unsigned long long *>(scan)[warp] = cost;   // 32 x 8 bytes of the scan array
        __syncthreads();
        if (tid == 0) {
            uint32_t best = 16u;
            unsigned long long best_cost = ~0ull;
            for (uint32_t w = 0; w < kPlanThreads / 32; ++w) {
                const unsigned long long c = reinterpret_cast<unsigned long long *>(scan)[w];
                if (c <= best_cost && c != ~0ull) {
                    best_cost = c;
                    best = 4u + w;
                }
            }
            s_total = best;
        }
        __syncthreads();
        pages_per_unit = s_total;
        __syncthreads();
    }
    for (int attempt = 0; attempt < 32; ++attempt) {
        local = 0;
        for (uint32_t s = begin; s < end; ++s) local += (visible_of(s, nullptr) + pages_per_unit - 1u) / pages_per_unit;
        // inclusive scan over the block: inside each warp with shuffles, then over the 32 warp totals
        uint32_t incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint32_t up = __shfl_up_sync(0xffffffffu, incl, o);
            if ((tid & 31u) >= static_cast<uint32_t>(o)) incl += up;
        }
        __syncthreads();                          // the previous use of warp_totals is over
        if ((tid & 31u) == 31u) warp_totals[tid >> 5] = incl;
        __syncthreads();
        if (tid < 32u) {
            uint32_t v = warp_totals[tid];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t up = __shfl_up_sync(0xffffffffu, v, o);
                if (tid >= static_cast<uint32_t>(o)) v += up;
            }
            warp_totals[tid] = v;
            if (tid == 31u) s_total = v;
        }
        __syncthreads();
        scan[tid] = incl + ((tid >> 5) ? warp_totals[(tid >> 5) - 1u] : 0u);
        __syncthreads();
        if (s_total <= p.layout.chunk_capacity) break;
        if (attempt == 31 || pages_per_unit >= (1u << 30)) { overflow = 1; break; }
        pages_per_unit <<= 1;
    }
    // Chunk prefix per sequence, and every chunk's start-up record (the attention kernel's warps read that record, not
    // the prefix). Few sequences with many chunks each: a warp per sequence writes the records side by side; many
    // sequences with few chunks: every thread writes those of its own sequences.
    uint32_t running = scan[tid] - local;
    ChunkInfo *info = chunk_info(p);
    const bool by_warp = !overflow && s_total >= 8ull * p.seq_count;
    for (uint32_t s = begin; s < end; ++s) {
        prefix[s] = overflow ? 0u : running;
        uint32_t first_page;
        const uint32_t chunks = (visible_of(s, &first_page) + pages_per_unit - 1u) / pages_per_unit;
        if (!overflow && !by_warp && chunks) {
            const uint32_t slot = slot_of(p, s), sealed = p.seq_sealed_tokens[slot];
            const uint32_t qpos = query_position(p, s, sealed, p.tail_tokens ? p.tail_tokens[slot] : 0u);
            for (uint32_t k = 0; k < chunks; ++k) {
                uint4 *dst = reinterpret_cast<uint4 *>(info + running + k);
                dst[0] = make_uint4(s, slot, sealed, qpos);
                dst[1] = make_uint4(first_page + k * pages_per_unit, row_of(p, s), 0u, 0u);
            }
        }
        running += chunks;
    }
    if (by_warp) {
        __syncthreads();   // prefix[] is complete
        for (uint32_t s = tid >> 5; s < p.seq_count; s += kPlanThreads / 32) {
            const uint32_t c0 = prefix[s], c1 = s + 1u < p.seq_count ? prefix[s + 1u] : s_total;
            if (c1 == c0) continue;
            uint32_t first_page;
            visible_of(s, &first_page);
            const uint32_t slot = slot_of(p, s), sealed = p.seq_sealed_tokens[slot];
            const uint32_t qpos = query_position(p, s, sealed, p.tail_tokens ? p.tail_tokens[slot] : 0u);
            const uint32_t row = row_of(p, s);
            for (uint32_t c = c0 + (tid & 31u); c < c1; c += 32u) {
                uint4 *dst = reinterpret_cast<uint4 *>(info + c);
                dst[0] = make_uint4(s, slot, sealed, qpos);
                dst[1] = make_uint4(first_page + (c - c0) * pages_per_unit, row, 0u, 0u);
            }
        }
    }
    if (tid == 0) {
        prefix[p.seq_count] = overflow ? 0u : s_total;
        hdr->chunk_count = overflow ? 0u : s_total;
        hdr->pages_per_unit = pages_per_unit;
        hdr->next_unit = 0;
        hdr->chunk_capacity = static_cast<uint32_t>(min(p.layout.chunk_capacity, static_cast<uint64_t>(0xffffffffu)));
        hdr->overflow = overflow;
        hdr->shared_pages = overflow ? 0u : shared;
        hdr->shared_ctas = overflow ? 0u : shared_ctas;
        hdr->shared_rounds = shared_rounds;
        if (overflow) raise_status(p, CF_B200_DEVSTAT_WORKSPACE);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Query load helper.
// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ float load_query(const AttentionParams &p, uint32_t seq, uint32_t q_head, uint32_t d) {
    const uint64_t i = (static_cast<uint64_t>(seq) * p.query_head_count + q_head) * p.head_dim + d;
    return p.query_type == CF_B200_F16 ? __half2float(reinterpret_cast<const __half *>(p.queries)[i])
                                       : reinterpret_cast<const float *>(p.queries)[i];
}

// ---------------------------------------------------------------------------------------------------------------
// Any-geometry attention kernel: one CTA per (chunk, kv head) unit. Each page record is copied to shared memory,
// both streams are decoded to symbols there (one thread per block), then scores and the online-softmax update
// are computed from shared memory. Built for coverage of every legal geometry, not for speed.
// ---------------------------------------------------------------------------------------------------------------
struct GenericSmem {
    uint32_t record_bytes, sym_bytes;
    uint32_t off_record, off_ksym, off_vsym, off_q, off_acc, off_scores, off_ml, total;
};

__host__ __device__ inline GenericSmem generic_smem(uint32_t symbols, uint32_t group, uint32_t head_dim,
                                                    uint32_t page_tokens) {
    GenericSmem s;
    s.record_bytes = 16u + 2u * align_up_u32(symbols, 16u) + 32u;
    s.sym_bytes = align_up_u32(symbols, 16u);
    s.off_record = 0;
    s.off_ksym = s.off_record + s.record_bytes;
    s.off_vsym = s.off_ksym + s.sym_bytes;
    s.off_q = s.off_vsym + s.sym_bytes;
    s.off_acc = s.off_q + group * head_dim * 4u;
    s.off_scores = s.off_acc + group * head_dim * 4u;
    s.off_ml = s.off_scores + group * page_tokens * 4u;
    s.total = s.off_ml + group * 8u + 16u;
    return s;
}

__global__ void __launch_bounds__(kGenericThreads) generic_attention_kernel(AttentionParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ uint32_t s_unit;
    const GenericSmem lay = generic_smem(p.symbols, p.group, p.head_dim, p.page_tokens);
    uint8_t *record = smem + lay.off_record;
    uint8_t *ksym = smem + lay.off_ksym;
    uint8_t *vsym = smem + lay.off_vsym;
    float *q = reinterpret_cast<float *>(smem + lay.off_q);
    float *acc = reinterpret_cast<float *>(smem + lay.off_acc);
    float *scores = reinterpret_cast<float *>(smem + lay.off_scores);
    float *ml = reinterpret_cast<float *>(smem + lay.off_ml);  // [group][2]: running max, running sum

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t D = p.head_dim, T = p.page_tokens, G = p.group;
    PlanHeader *hdr = plan_header(p);
    const uint32_t *prefix = chunk_prefix(p);
    const uint32_t unit_count = hdr->chunk_count * p.kv_head_span;
    const uint32_t pages_per_unit = hdr->pages_per_unit;
    const uint32_t max_part_units = align_up_u32(p.symbols, 16u) / 16u;

    for (;;) {
        __syncthreads();
        if (tid == 0) s_unit = atomicAdd(&hdr->next_unit, 1u);
        __syncthreads();
        const uint32_t unit = s_unit;
        if (unit >= unit_count) break;
        const uint32_t chunk = unit / p.kv_head_span;
        const uint32_t head_local = unit % p.kv_head_span;
        const uint32_t kv_head = p.kv_head_begin + head_local;
        const uint32_t seq = sequence_of_chunk(prefix, p.seq_count, chunk);
        const uint32_t slot = slot_of(p, seq);
        const uint32_t sealed = p.seq_sealed_tokens[slot];
        const uint32_t tail = p.tail_tokens ? p.tail_tokens[slot] : 0u;
        const uint32_t qpos = query_position(p, seq, sealed, tail);
        const uint32_t first_token = window_begin(qpos, p.causal_window);
        uint32_t first_page;
        const uint32_t vis = visible_pages(p, seq, &first_page);
        const uint32_t page_begin = first_page + (chunk - prefix[seq]) * pages_per_unit;
        const uint32_t page_end = min(page_begin + pages_per_unit, first_page + vis);

        for (uint32_t i = tid; i < G * D; i += kGenericThreads) {
            q[i] = load_query(p, row_of(p, seq), kv_head * G + i / D, i % D) * (p.softmax_scale * kLog2e);
            acc[i] = 0.0f;
        }
        if (tid < G) {
            ml[2 * tid] = -CUDART_INF_F;
            ml[2 * tid + 1] = 0.0f;
        }

        for (uint32_t page = page_begin; page < page_end; ++page) {
            __syncthreads();
            const uint32_t page_id = p.page_table[static_cast<uint64_t>(slot) * p.page_table_stride + page];
            const uint64_t entry = p.page_dir[static_cast<uint64_t>(page_id) * p.kv_head_count + kv_head];
            const uint32_t units = static_cast<uint32_t>(CF_B200_DIR_LENGTH_UNITS(entry));
            if (units == 0 || units > 1u + 2u * max_part_units) {
                if (tid == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
                continue;
            }
            const uint4 *src = reinterpret_cast<const uint4 *>(p.arena + 16ull * CF_B200_DIR_OFFSET_UNITS(entry));
            for (uint32_t i = tid; i < units; i += kGenericThreads) reinterpret_cast<uint4 *>(record)[i] = src[i];
            __syncthreads();
            const cf_b200_record_header h = *reinterpret_cast<const cf_b200_record_header *>(record);
            if (h.version != CF_B200_FORMAT_VERSION || h.codebook_id != p.codebook_id ||
                1u + h.k_part_units + h.v_part_units != units || h.k_part_units > max_part_units ||
                h.v_part_units > max_part_units || h.token_count == 0 || h.token_count > T || h.k_coder > CF_B200_CODER_MAX ||
                h.v_coder > CF_B200_CODER_MAX) {
                if (tid == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
                continue;
            }
            const uint8_t *k_part = record + 16;
            const uint8_t *v_part = record + 16 + 16u * h.k_part_units;
            const uint32_t k_bytes = 16u * h.k_part_units, v_bytes = 16u * h.v_part_units;
            int bad_table = 0;
            for (uint32_t b = tid; b < 2u * p.nblocks; b += kGenericThreads)
                bad_table |= b < p.nblocks ? !part_block_start_ok(k_part, k_bytes, h.k_coder, p.nblocks, b, p.symbols)
                                           : !part_block_start_ok(v_part, v_bytes, h.v_coder, p.nblocks, b - p.nblocks, p.symbols);
            if (__syncthreads_or(bad_table)) {   // a block starts outside its part
                if (tid == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
                continue;
            }
            for (uint32_t b = tid; b < 2u * p.nblocks; b += kGenericThreads) {
                if (b < p.nblocks) {
                    uint8_t *dst = ksym + b * p.block_size;
                    decode_part_block(k_part, k_bytes, h.k_coder, p.nblocks, b, p.block_size, p.symbols, p.k_tables,
                                      [&](int j, uint32_t s) { dst[j] = static_cast<uint8_t>(s); });
                } else {
                    const uint32_t vb = b - p.nblocks;
                    uint8_t *dst = vsym + vb * p.block_size;
                    decode_part_block(v_part, v_bytes, h.v_coder, p.nblocks, vb, p.block_size, p.symbols, p.v_tables,
                                      [&](int j, uint32_t s) { dst[j] = static_cast<uint8_t>(s); });
                }
            }
            __syncthreads();
            const float k_scale = __half2float(__ushort_as_half(h.k_scale_f16));
            const float v_scale = __half2float(__ushort_as_half(h.v_scale_f16));
            // scores[g][t], one warp per (g, t)
            for (uint32_t pair = warp; pair < G * T; pair += kGenericThreads / 32) {
                const uint32_t g = pair / T, t = pair % T;
                const uint32_t token = page * T + t;
                float s = -CUDART_INF_F;
                if (t < h.token_count && token >= first_token && token < sealed && token <= qpos) {
                    float dot = 0.0f;
                    for (uint32_t d = lane; d < D; d += 32)
                        dot += q[g * D + d] * static_cast<float>(static_cast<int>(ksym[t * D + d]) - kZero);
                    s = warp_sum(dot) * k_scale;
                }
                if (lane == 0) scores[g * T + t] = s;
            }
            __syncthreads();
            // online softmax update: thread d owns channel d of every group member
            float new_m[kGenericMaxGroup], new_l[kGenericMaxGroup];
            for (uint32_t g = 0; g < G; ++g) {
                const float m_old = ml[2 * g], l_old = ml[2 * g + 1];
                float pm = -CUDART_INF_F;
                for (uint32_t t = 0; t < T; ++t) pm = fmaxf(pm, scores[g * T + t]);
                const float m_new = fmaxf(m_old, pm);
                new_m[g] = m_new;
                new_l[g] = l_old;
                if (m_new == -CUDART_INF_F) continue;
                const float alpha = m_old == -CUDART_INF_F ? 0.0f : exp2f(m_old - m_new);
                float lsum = 0.0f, a = 0.0f;
                for (uint32_t t = 0; t < T; ++t) {
                    const float s = scores[g * T + t];
                    const float w = s == -CUDART_INF_F ? 0.0f : exp2f(s - m_new);
                    lsum += w;
                    if (tid < D) a += w * static_cast<float>(static_cast<int>(vsym[tid * T + t]) - kZero);
                }
                new_l[g] = l_old * alpha + lsum;
                if (tid < D) acc[g * D + tid] = acc[g * D + tid] * alpha + a * v_scale;
            }
            __syncthreads();
            if (tid == 0) {
                for (uint32_t g = 0; g < G; ++g) {
                    ml[2 * g] = new_m[g];
                    ml[2 * g + 1] = new_l[g];
                }
            }
        }
        __syncthreads();
        for (uint32_t i = tid; i < G * D; i += kGenericThreads) {
            const uint32_t g = i / D, d = i % D;
            float *dst = partial_ptr(p, chunk, head_local * G + g);
            dst[2 + d] = acc[i];
            if (d == 0) {
                dst[0] = ml[2 * g];
                dst[1] = ml[2 * g + 1];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Combine: merge the chunk partials of one (sequence, query head) with the unsealed tail and write the output.
// ---------------------------------------------------------------------------------------------------------------
#ifndef CFB_COMBINE_THREADS
#define CFB_COMBINE_THREADS 128   // = the largest head_dim: thread d owns output channel d; more threads only wait
#endif
constexpr int kCombineThreads = CFB_COMBINE_THREADS;
constexpr int kCombineWarps = kCombineThreads / 32;

__global__ void __launch_bounds__(kCombineThreads) combine_kernel(AttentionParams p) {
    extern __shared__ float tail_scores[];  // [tail_capacity]
    __shared__ float s_m[kCombineWarps], s_l[kCombineWarps];
    __shared__ float s_acc[kCombineWarps][128];
    const uint32_t seq = blockIdx.x;
    const uint32_t local_q = blockIdx.y;
    const uint32_t G = p.group, D = p.head_dim;
    const uint32_t kv_head = p.kv_head_begin + local_q / G;
    const uint32_t q_head = kv_head * G + local_q % G;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t slot = slot_of(p, seq);
    const uint32_t sealed = p.seq_sealed_tokens[slot];
    const uint32_t C = p.tail_capacity;  // rows per (slot, kv head) in the tails
    const uint32_t tail = p.tail_tokens ? min(p.tail_tokens[slot], C) : 0u;
    const uint32_t qpos = query_position(p, seq, sealed, p.tail_tokens ? p.tail_tokens[slot] : 0u);
    const uint32_t first_token = window_begin(qpos, p.causal_window);
    const uint32_t *prefix = chunk_prefix(p);
    const uint32_t c0 = prefix[seq], c1 = prefix[seq + 1];
    const uint32_t row = row_of(p, seq);   // of the query and output tensors

    // tail scores (binary16 rows, one warp per token)
    for (uint32_t t = warp; t < tail; t += kCombineThreads / 32) {
        const uint64_t tail_row = ((static_cast<uint64_t>(slot) * p.kv_head_count + kv_head) * C + t) * D;
        float dot = 0.0f;
        for (uint32_t d = lane; d < D; d += 32) dot += load_query(p, row, q_head, d) * load_tail(p.tail_k, p.tail_type, tail_row + d);
        dot = warp_sum(dot);
        if (lane == 0)
            tail_scores[t] = (sealed + t >= first_token && sealed + t <= qpos) ? dot * p.softmax_scale * kLog2e : -CUDART_INF_F;
    }
    __syncthreads();

    // Chunk partials: every warp merges its share of the chunks in one pass (running max, rescale on the way), four
    // channels per lane, so that many independent loads are in flight; the warps' results meet in shared memory.
    {
        float wm = -CUDART_INF_F, wl = 0.0f, wa[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t c = c0 + warp; c < c1; c += kCombineWarps) {
            const float *part = partial_ptr(p, c, local_q);
            const float pm = part[0], pl = part[1];
            float pa[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) pa[j] = lane + 32u * j < D ? part[2 + lane + 32u * j] : 0.0f;
            if (pm == -CUDART_INF_F) continue;
            const float nm = fmaxf(wm, pm);
            const float so = exp2f(wm - nm), sn = exp2f(pm - nm);  // wm = -inf gives so = 0
            wl = wl * so + pl * sn;
#pragma unroll
            for (int j = 0; j < 4; ++j) wa[j] = wa[j] * so + pa[j] * sn;
            wm = nm;
        }
        // the shared prefix's partials, same rule: one per CTA of the shared-prefix kernel that met the row's head-tile
        const PlanHeader *hdr = plan_header(p);
        uint32_t cells = 0;
        if (hdr->shared_pages != 0u && hdr->shared_ctas != 0u) {
            const uint32_t row_tiles = (p.seq_count * G + 127u) / 128u;
            const SharedSplit split = {hdr->shared_rounds, p.kv_head_span * row_tiles, hdr->shared_ctas};
            const uint64_t first = static_cast<uint64_t>((local_q / G) * row_tiles + (seq * G + local_q % G) / 128u) * split.rounds;
            cells = min(split.cta_of(first + split.rounds - 1u) - split.cta_of(first) + 1u, CF_B200_SHARED_CHUNKS_MAX);
        }
        for (uint32_t c = warp; c < cells; c += kCombineWarps) {
            const float *part = shared_partial_ptr(p, c, seq, local_q);
            const float pm = part[0], pl = part[1];
            float pa[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) pa[j] = lane + 32u * j < D ? part[2 + lane + 32u * j] : 0.0f;
            if (pm == -CUDART_INF_F) continue;
            const float nm = fmaxf(wm, pm);
            const float so = exp2f(wm - nm), sn = exp2f(pm - nm);
            wl = wl * so + pl * sn;
#pragma unroll
            for (int j = 0; j < 4; ++j) wa[j] = wa[j] * so + pa[j] * sn;
            wm = nm;
        }
        if (lane == 0) {
            s_m[warp] = wm;
            s_l[warp] = wl;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) s_acc[warp][lane + 32 * j] = wa[j];
    }
    __syncthreads();
    float m = -CUDART_INF_F;
    for (int w = 0; w < kCombineWarps; ++w) m = fmaxf(m, s_m[w]);
    for (uint32_t t = 0; t < tail; ++t) m = fmaxf(m, tail_scores[t]);

    float l = 0.0f, a = 0.0f;
    if (m != -CUDART_INF_F) {
        for (int w = 0; w < kCombineWarps; ++w) {
            if (s_m[w] == -CUDART_INF_F) continue;
            const float sw = exp2f(s_m[w] - m);
            l += s_l[w] * sw;
            if (tid < D) a += s_acc[w][tid] * sw;
        }
        for (uint32_t t = 0; t < tail; ++t) {
            const float s = tail_scores[t];
            if (s == -CUDART_INF_F) continue;
            const float w = exp2f(s - m);
            l += w;
            if (tid < D)
                a += w * load_tail(p.tail_v, p.tail_type, ((static_cast<uint64_t>(slot) * p.kv_head_count + kv_head) * C + t) * D + tid);
        }
    }
    if (tid < D) {
        const float out = l > 0.0f ? a / l : 0.0f;  // no visible token: zeros (paged_kv_attention.cu:170-173)
        const uint64_t i = (static_cast<uint64_t>(row) * p.query_head_count + q_head) * D + tid;
        if (p.output_type == CF_B200_F16) reinterpret_cast<__half *>(p.output)[i] = __float2half_rn(out);
        else reinterpret_cast<float *>(p.output)[i] = out;
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Decode probe: write the symbols of whole records to global memory.
// ---------------------------------------------------------------------------------------------------------------
__global__ void decode_pages_kernel(AttentionParams p, const uint32_t *page_ids, uint8_t *k_out, uint8_t *v_out) {
    const uint32_t page = blockIdx.x, kv_head = blockIdx.y;
    const uint64_t entry = p.page_dir[static_cast<uint64_t>(page_ids[page]) * p.kv_head_count + kv_head];
    if (CF_B200_DIR_LENGTH_UNITS(entry) == 0) {
        if (threadIdx.x == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
        return;
    }
    const uint8_t *record = p.arena + 16ull * CF_B200_DIR_OFFSET_UNITS(entry);
    const cf_b200_record_header h = *reinterpret_cast<const cf_b200_record_header *>(record);
    if (h.version != CF_B200_FORMAT_VERSION || h.k_coder > CF_B200_CODER_MAX || h.v_coder > CF_B200_CODER_MAX) {
        if (threadIdx.x == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
        return;
    }
    const uint8_t *k_part = record + 16;
    const uint8_t *v_part = record + 16 + 16u * h.k_part_units;
    const uint64_t base = (static_cast<uint64_t>(page) * p.kv_head_count + kv_head) * p.symbols;
    for (uint32_t b = threadIdx.x; b < 2u * p.nblocks; b += blockDim.x) {
        if (b < p.nblocks) {
            uint8_t *dst = k_out + base + b * p.block_size;
            decode_part_block(k_part, 16u * h.k_part_units, h.k_coder, p.nblocks, b, p.block_size, p.symbols, p.k_tables,
                              [&](int j, uint32_t s) { dst[j] = static_cast<uint8_t>(s); });
        } else {
            const uint32_t vb = b - p.nblocks;
            uint8_t *dst = v_out + base + vb * p.block_size;
            decode_part_block(v_part, 16u * h.v_part_units, h.v_coder, p.nblocks, vb, p.block_size, p.symbols, p.v_tables,
                              [&](int j, uint32_t s) { dst[j] = static_cast<uint8_t>(s); });
        }
    }
}

bool finite_float(float v) { return v == v && v - v == 0.0f; }

// Test hooks (cf_b200_test_wait_expiry): a lowered wait bound and one page whose copy is armed but never issued.
std::atomic<uint32_t> g_test_wait_polls{0}, g_test_skip_copy_page{0};

bool fill_params(const cf_b200_sealed_attention_desc *d, AttentionParams *p) {
    p->kv_head_count = d->kv_head_count;
    p->query_head_count = d->query_head_count;
    p->head_dim = d->head_dim;
    p->page_tokens = d->page_tokens;
    p->block_size = d->block_size;
    p->kv_head_begin = d->kv_head_begin;
    p->kv_head_span = d->kv_head_span ? d->kv_head_span : d->kv_head_count - d->kv_head_begin;
    p->group = d->query_head_count / d->kv_head_count;
    p->symbols = d->head_dim * d->page_tokens;
    p->nblocks = (p->symbols + d->block_size - 1) / d->block_size;
    p->codebook_id = d->codebook_id;
    p->arena = d->arena;
    p->page_dir = d->page_dir;
    p->page_table = d->page_table;
    p->seq_sealed_tokens = d->seq_sealed_tokens;
    p->seq_slots = d->seq_slots;
    p->page_table_stride = d->page_table_stride;
    p->seq_count = d->seq_count;
    p->k_tables = d->k_tables;
    p->v_tables = d->v_tables;
    p->tail_k = d->tail_k;
    p->tail_v = d->tail_v;
    p->tail_tokens = d->tail_tokens;
    p->tail_type = d->tail_type == CF_B200_F32 ? CF_B200_F32 : CF_B200_F16;
    p->query_positions = d->query_positions;
    p->row_map = d->row_map;
    p->tail_capacity = d->tail_capacity ? d->tail_capacity : d->page_tokens;
    p->queries = d->queries;
    p->output = d->output;
    p->query_type = d->query_type;
    p->output_type = d->output_type;
    p->softmax_scale = d->softmax_scale;
    p->causal_window = d->causal_window;
    p->workspace = static_cast<uint8_t *>(d->workspace);
    p->layout = workspace_layout(d->seq_count, p->kv_head_span * p->group, d->head_dim, d->workspace_bytes,
                                 d->shared_prefix_pages != 0);
    p->min_pages_per_unit = d->min_pages_per_unit;
    p->shared_prefix_pages = 0;   // the launch code sets it when the lanes kernels serve the call
    p->sm_count = 0;
    p->decode_probe = d->kernel == CF_B200_KERNEL_DECODE_PROBE ? 1u : d->kernel == CF_B200_KERNEL_DECODE_DUMP ? 2u : 0u;
    p->dump_pages = p->decode_probe == 2u ? d->reserved0 : 1u;
    const uint32_t polls = g_test_wait_polls.load(std::memory_order_relaxed);
    p->wait_polls = polls ? polls : kDefaultWaitPolls;
    p->skip_copy_page = g_test_skip_copy_page.load(std::memory_order_relaxed);
    p->status = d->status;
    p->pool_k = nullptr;
    p->pool_v = nullptr;
    return true;
}

}  // namespace

cudaError_t launch_plan(const AttentionParams &p, cudaStream_t stream) {
    if (p.shared_prefix_pages) verify_prefix_kernel<<<p.seq_count, 256, 0, stream>>>(p);
    plan_kernel<<<1, kPlanThreads, 0, stream>>>(p);
    return cudaPeekAtLastError();
}

cudaError_t launch_combine(const AttentionParams &p, cudaStream_t stream) {
    const dim3 grid(p.seq_count, p.kv_head_span * p.group);
    combine_kernel<<<grid, kCombineThreads, max(p.tail_capacity, 1u) * sizeof(float), stream>>>(p);
    return cudaPeekAtLastError();
}

cudaError_t launch_generic_attention(const AttentionParams &p, cudaStream_t stream) {
    static LauncherState table[64];
    cudaError_t e;
    LauncherState *state = launcher_state(table, &e);
    if (!state) return e;
    const int sm_count = state->sm_count;
    const GenericSmem lay = generic_smem(p.symbols, p.group, p.head_dim, p.page_tokens);
    e = cudaFuncSetAttribute(generic_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(lay.total));
    if (e != cudaSuccess) return e;
    generic_attention_kernel<<<sm_count * 4, kGenericThreads, lay.total, stream>>>(p);
    return cudaPeekAtLastError();
}

}  // namespace cfb

using cfb::AttentionParams;

extern "C" cf_status cf_b200_sealed_attention_validate(const cf_b200_sealed_attention_desc *d) {
    if (d == nullptr || d->struct_size != sizeof(cf_b200_sealed_attention_desc) || d->abi_version != CF_B200_ABI_VERSION)
        return CF_ERR_INVALID_ARGUMENT;
    if (d->kv_head_count == 0 || d->query_head_count == 0 || d->head_dim == 0 || d->page_tokens == 0 ||
        d->block_size == 0 || d->query_head_count % d->kv_head_count != 0 || !cfb::finite_float(d->softmax_scale))
        return CF_ERR_INVALID_ARGUMENT;
    if (d->kv_head_begin >= d->kv_head_count || d->kv_head_span > d->kv_head_count - d->kv_head_begin)
        return CF_ERR_INVALID_ARGUMENT;
    if (d->queries == nullptr || d->output == nullptr || d->workspace == nullptr || d->seq_sealed_tokens == nullptr ||
        d->k_tables == nullptr || d->v_tables == nullptr)
        return CF_ERR_INVALID_ARGUMENT;
    if (d->seq_count == 0) return CF_ERR_INVALID_ARGUMENT;
    if (d->page_table_stride != 0 && (d->page_table == nullptr || d->page_dir == nullptr || d->arena == nullptr))
        return CF_ERR_INVALID_ARGUMENT;
    if (d->tail_tokens != nullptr && (d->tail_k == nullptr || d->tail_v == nullptr)) return CF_ERR_INVALID_ARGUMENT;
    if ((d->query_type != CF_B200_F16 && d->query_type != CF_B200_F32) ||
        (d->output_type != CF_B200_F16 && d->output_type != CF_B200_F32) || d->kernel > CF_B200_KERNEL_DECODE_DUMP ||
        (d->tail_type != 0 && d->tail_type != CF_B200_F16 && d->tail_type != CF_B200_F32))
        return CF_ERR_INVALID_ARGUMENT;
    if ((reinterpret_cast<uintptr_t>(d->arena) & 15u) != 0 || (reinterpret_cast<uintptr_t>(d->workspace) & 255u) != 0)
        return CF_ERR_INVALID_ARGUMENT;
    // format limits
    if (d->head_dim > CF_KV_MAX_HEAD_DIM || d->head_dim * d->page_tokens > CF_B200_MAX_STREAM_SYMBOLS ||
        d->block_size < 16 || d->block_size > 1024 || d->query_head_count / d->kv_head_count > cfb::kGenericMaxGroup)
        return CF_ERR_UNSUPPORTED;
    const uint32_t span = d->kv_head_span ? d->kv_head_span : d->kv_head_count - d->kv_head_begin;
    const cfb::WorkspaceLayout w = cfb::workspace_layout(d->seq_count, span * (d->query_head_count / d->kv_head_count),
                                                         d->head_dim, d->workspace_bytes, d->shared_prefix_pages != 0);
    if (w.chunk_capacity < d->seq_count) return CF_ERR_INVALID_ARGUMENT;  // at least one chunk per sequence
    if (d->shared_prefix_pages > d->page_table_stride) return CF_ERR_INVALID_ARGUMENT;
    // reserved0 has one use: the number of page ids the dump buffer of CF_B200_KERNEL_DECODE_DUMP covers
    if ((d->kernel == CF_B200_KERNEL_DECODE_DUMP) != (d->reserved0 != 0)) return CF_ERR_INVALID_ARGUMENT;
    return CF_OK;
}

extern "C" cf_status cf_b200_sealed_attention_workspace_bytes(const cf_b200_sealed_attention_desc *d,
                                                              uint64_t total_pages, uint64_t *out_bytes) {
    if (d == nullptr || out_bytes == nullptr || d->kv_head_count == 0 || d->query_head_count == 0 ||
        d->query_head_count % d->kv_head_count != 0 || d->head_dim == 0)
        return CF_ERR_INVALID_ARGUMENT;
    const uint32_t span = d->kv_head_span ? d->kv_head_span : d->kv_head_count - d->kv_head_begin;
    const uint32_t local_q = span * (d->query_head_count / d->kv_head_count);
    const uint32_t ppu = d->min_pages_per_unit ? d->min_pages_per_unit : cfb::default_pages_per_unit(total_pages, span);
    const uint64_t chunks = total_pages / ppu + d->seq_count + 1;  // each sequence may round up once
    const cfb::WorkspaceLayout w = cfb::workspace_layout(d->seq_count, local_q, d->head_dim, 0, d->shared_prefix_pages != 0);
    *out_bytes = w.partials_offset + chunks * (w.partial_stride_floats * 4ull * local_q + sizeof(cfb::ChunkInfo)) + 64ull;
    return CF_OK;
}

extern "C" cf_status cf_b200_sealed_attention_stages_async(const cf_b200_sealed_attention_desc *d, uint32_t stages,
                                                           void *stream) {
    return cfb::sealed_attention_stages(d, stages, stream, false);
}

// output_on_peer: the one exception to "every pointer is the current device's" — the multi-GPU scheduler lets the
// combine kernel store its output rows straight into the root GPU's tensor (plain coalesced stores over a peer mapping
// the scheduler has enabled and checked). Everything that is READ stays local.
cf_status cfb::sealed_attention_stages(const cf_b200_sealed_attention_desc *d, uint32_t stages, void *stream, bool output_on_peer) {
    const cf_status valid = cf_b200_sealed_attention_validate(d);
    if (valid != CF_OK) return valid;
    if (stages == 0 || stages > 7u) return CF_ERR_INVALID_ARGUMENT;
    if (!cfb::on_current_device(d->arena) || !cfb::on_current_device(d->workspace) || !cfb::on_current_device(d->queries) ||
        !cfb::on_current_device(d->row_map) || (!output_on_peer && !cfb::on_current_device(d->output)))
        return CF_ERR_INVALID_ARGUMENT;   // memory of another GPU: the call must be made with that GPU current
    AttentionParams p;
    cfb::fill_params(d, &p);
    const bool lanes_ok = cfb::lanes_kernel_supports(p);
    const bool probe = d->kernel == CF_B200_KERNEL_DECODE_PROBE || d->kernel == CF_B200_KERNEL_DECODE_DUMP;
    if ((d->kernel == CF_B200_KERNEL_LANES || probe) && !lanes_ok) return CF_ERR_UNSUPPORTED;
    if (d->kernel == CF_B200_KERNEL_DECODE_DUMP && (stages & CF_B200_STAGE_COMBINE)) return CF_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool use_lanes = d->kernel == CF_B200_KERNEL_LANES || probe ||
                           (d->kernel == CF_B200_KERNEL_AUTO && lanes_ok);
    // the shared-prefix kernel works on rows of 128 = whole query groups and on pages every query token sees in full
    if (use_lanes && p.block_size == 64 && p.head_dim == 128 && d->row_map == nullptr && p.decode_probe != 1u && d->shared_prefix_pages && d->causal_window == 0 && 128u % p.group == 0) {
        static cfb::LauncherState table[64];
        cudaError_t e;
        const cfb::LauncherState *state = cfb::launcher_state(table, &e);
        if (!state) return CF_ERR_CUDA;
        p.shared_prefix_pages = d->shared_prefix_pages;
        p.sm_count = static_cast<uint32_t>(state->sm_count);
    }
    if ((stages & CF_B200_STAGE_PLAN) && cfb::launch_plan(p, s) != cudaSuccess) return CF_ERR_CUDA;
    if (stages & CF_B200_STAGE_ATTENTION) {
        if (p.shared_prefix_pages) {
            if (cfb::launch_prefix_attention(p, s) != cudaSuccess) return CF_ERR_CUDA;
            g_shared_prefix_launches.fetch_add(1, std::memory_order_relaxed);
        }
        const cudaError_t e = use_lanes ? cfb::launch_lanes_attention(p, s) : cfb::launch_generic_attention(p, s);
        if (e != cudaSuccess) return CF_ERR_CUDA;
    }
    if ((stages & CF_B200_STAGE_COMBINE) && cfb::launch_combine(p, s) != cudaSuccess) return CF_ERR_CUDA;
    return CF_OK;
}

extern "C" cf_status cf_b200_test_wait_expiry(uint32_t skip_copy_page_id, uint32_t wait_polls) {
    cfb::g_test_skip_copy_page.store(skip_copy_page_id, std::memory_order_relaxed);
    cfb::g_test_wait_polls.store(wait_polls, std::memory_order_relaxed);
    return CF_OK;
}

extern "C" unsigned long long cf_b200_shared_prefix_launches(void) {
    return g_shared_prefix_launches.load(std::memory_order_relaxed);
}

extern "C" cf_status cf_b200_sealed_attention_async(const cf_b200_sealed_attention_desc *d, void *stream) {
    return cf_b200_sealed_attention_stages_async(
        d, CF_B200_STAGE_PLAN | CF_B200_STAGE_ATTENTION | CF_B200_STAGE_COMBINE, stream);
}

extern "C" cf_status cf_b200_decode_pages_async(const cf_b200_sealed_attention_desc *d, const uint32_t *page_ids,
                                                uint32_t page_count, uint8_t *k_symbols, uint8_t *v_symbols,
                                                void *stream) {
    if (d == nullptr || d->struct_size != sizeof(cf_b200_sealed_attention_desc) ||
        d->abi_version != CF_B200_ABI_VERSION || page_ids == nullptr || k_symbols == nullptr || v_symbols == nullptr ||
        d->arena == nullptr || d->page_dir == nullptr || d->k_tables == nullptr || d->v_tables == nullptr ||
        d->kv_head_count == 0 || d->head_dim == 0 || d->page_tokens == 0 || d->block_size == 0)
        return CF_ERR_INVALID_ARGUMENT;
    if (d->head_dim * d->page_tokens > CF_B200_MAX_STREAM_SYMBOLS || d->block_size < 16 || d->block_size > 1024)
        return CF_ERR_UNSUPPORTED;
    if (page_count == 0) return CF_OK;
    AttentionParams p{};
    p.kv_head_count = d->kv_head_count;
    p.head_dim = d->head_dim;
    p.page_tokens = d->page_tokens;
    p.block_size = d->block_size;
    p.symbols = d->head_dim * d->page_tokens;
    p.nblocks = (p.symbols + d->block_size - 1) / d->block_size;
    p.arena = d->arena;
    p.page_dir = d->page_dir;
    p.k_tables = d->k_tables;
    p.v_tables = d->v_tables;
    p.status = d->status;
    cfb::decode_pages_kernel<<<dim3(page_count, d->kv_head_count), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        p, page_ids, k_symbols, v_symbols);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}
