// dense_attention.cu — the comparison kernel: the same decode-step attention over UNCOMPRESSED binary16 pages.
//
// Same page table, same chunk planning, same split-KV partials and combine as the sealed path; only the read
// differs (the fairness rule of the reference's own dense comparison, tests/latency_bench.cu and
// product/kv-crossover-campaign.json:35-40). It answers "what would this GPU do with plain fp16 KV".
//
// Pool layout: [page_id][kv_head][16 tokens][128 channels] binary16, one 4 KiB tile per (page, kv head) for K and
// one for V. Inside a 256-byte token row the sixteen 16-byte chunks are stored XOR-swizzled,
//     physical chunk = logical chunk ^ f(token),  f(token) = (((token ^ (token >> 2)) & 1) << 2) | ((token >> 1) & 1)
// so that after a linear bulk copy the fragment reads below touch every shared-memory bank once.
//
// One warp owns one (chunk, kv head) unit; a page (K tile + V tile, 8 KiB) arrives by two bulk async copies on
// one mbarrier, double buffered. S = Q K^T and O = P V run on mma.sync m16n8k16 with the query group in the rows
// (up to 8 query heads per kv head).

#include <math_constants.h>

#include "attention_params.cuh"

namespace cfb {
namespace {

constexpr int kWarps = 12;
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kTileBytes = 4096;
constexpr uint32_t kStageBytes = 2 * kTileBytes;
constexpr uint32_t kWarpBytes = 2 * kStageBytes + 64;
constexpr uint32_t kSmemBytes = kWarps * kWarpBytes;
constexpr uint32_t kWaitSpins = 1u << 22;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitSpins; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_addr(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    asm volatile(  // rows 8..15 of A are zero: the query group fills rows 0..7 only
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%5}, {%7,%8}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t swizzle_of(uint32_t token) {
    return (((token ^ (token >> 2)) & 1u) << 2) | ((token >> 1) & 1u);
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

__global__ void __launch_bounds__(kThreads, 1) dense_attention_kernel(AttentionParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint8_t *warp_mem = smem + warp * kWarpBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(warp_mem + 2 * kStageBytes);
    if (lane == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    PlanHeader *hdr = plan_header(p);
    const uint32_t *prefix = chunk_prefix(p);
    const uint32_t unit_count = hdr->chunk_count * p.kv_head_span;
    const uint32_t pages_per_unit = hdr->pages_per_unit;
    const uint32_t G = p.group, g = lane >> 2, t = lane & 3u;
    const float scale = p.softmax_scale * kLog2e;
    uint32_t phase_bits = 0u;

    for (;;) {
        uint32_t unit = 0;
        if (lane == 0) unit = atomicAdd(&hdr->next_unit, 1u);
        unit = __shfl_sync(0xffffffffu, unit, 0);
        if (unit >= unit_count) break;
        const uint32_t chunk = unit / p.kv_head_span;
        const uint32_t head_local = unit % p.kv_head_span;
        const uint32_t kv_head = p.kv_head_begin + head_local;
        const uint32_t seq = sequence_of_chunk(prefix, p.seq_count, chunk);
        const uint32_t slot = slot_of(p, seq);
        const uint32_t sealed = p.seq_sealed_tokens[slot];
        const uint32_t qpos = query_position(p, seq, sealed, 0u);
        const uint32_t first_token = window_begin(qpos, p.causal_window);
        const uint32_t pages = min((sealed + 15u) / 16u, qpos / 16u + 1u);
        const uint32_t first_page = min(first_token / 16u, pages);
        const uint32_t page_begin = first_page + (chunk - prefix[seq]) * pages_per_unit;
        const uint32_t page_end = min(page_begin + pages_per_unit, pages);
        const uint32_t n_pages = page_end > page_begin ? page_end - page_begin : 0u;
        const uint32_t *table_row = p.page_table + static_cast<uint64_t>(slot) * p.page_table_stride;

        // Q fragments: row g = query head g of the group; this lane's channels are chunks t, t+4, t+8, t+12
        uint4 qf[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            qf[i] = make_uint4(0u, 0u, 0u, 0u);
            if (g < G)
                qf[i] = *reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(p.queries) +
                                                         (static_cast<uint64_t>(seq) * p.query_head_count + kv_head * G + g) * 128u +
                                                         8u * (t + 4u * i));
        }
        float acc[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
        float m_run = -CUDART_INF_F, l_run = 0.0f;

        auto issue = [&](uint32_t st, uint32_t page) {
            if (lane == 0) {
                const uint64_t tile = (static_cast<uint64_t>(table_row[page]) * p.kv_head_count + kv_head) * (kTileBytes / 2);
                mbar_expect_tx(&bars[st], kStageBytes);
                bulk_load(warp_mem + st * kStageBytes, p.pool_k + tile, kTileBytes, &bars[st]);
                bulk_load(warp_mem + st * kStageBytes + kTileBytes, p.pool_v + tile, kTileBytes, &bars[st]);
            }
        };
        __syncwarp();
        if (n_pages) issue(0, page_begin);
        bool alive = true;
        for (uint32_t i = 0; i < n_pages; ++i) {
            const uint32_t st = i & 1u;
            if (i + 1 < n_pages) {
                __syncwarp();
                issue(st ^ 1u, page_begin + i + 1);
            }
            if (!mbar_wait(&bars[st], (phase_bits >> st) & 1u)) {
                if (lane == 0) raise_status(p, CF_B200_DEVSTAT_WAIT_EXPIRED);
                alive = false;
                break;
            }
            phase_bits ^= 1u << st;
            const uint8_t *k_tile = warp_mem + st * kStageBytes;
            const uint8_t *v_tile = k_tile + kTileBytes;

            // S = Q K^T for tokens g and 8 + g
            float s[2][4];
#pragma unroll
            for (int cg = 0; cg < 2; ++cg) {
                s[cg][0] = s[cg][1] = s[cg][2] = s[cg][3] = 0.0f;
                const uint32_t row = 8u * cg + g;
                const uint8_t *krow = k_tile + row * 256u;
                const uint32_t f = swizzle_of(row);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint4 kv = *reinterpret_cast<const uint4 *>(krow + (((t + 4u * c) ^ f) << 4));
                    mma_16816(s[cg], qf[c].x, qf[c].y, kv.x, kv.y);
                    mma_16816(s[cg], qf[c].z, qf[c].w, kv.z, kv.w);
                }
            }
            // online softmax: this lane holds head g, tokens 2t, 2t+1, 8+2t, 9+2t
            float sv[4];
            float mx = -CUDART_INF_F;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t token = (page_begin + i) * 16u + 8u * (e >> 1) + 2u * t + (e & 1);
                const bool visible = token >= first_token && token < sealed && token <= qpos;
                sv[e] = visible ? s[e >> 1][e & 1] * scale : -CUDART_INF_F;
                mx = fmaxf(mx, sv[e]);
            }
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run, mx);
            const float m_safe = m_new == -CUDART_INF_F ? 0.0f : m_new;
            const float alpha = exp2f(m_run - m_safe);
            float pv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) pv[e] = exp2f(sv[e] - m_safe);
            l_run = l_run * alpha + (pv[0] + pv[1]) + (pv[2] + pv[3]);
            m_run = m_new;
            const uint32_t pa0 = pack_half2(pv[0], pv[1]), pa2 = pack_half2(pv[2], pv[3]);

            // O = O * alpha + P V ; this lane supplies channels 16g .. 16g+15 of tokens 2t, 2t+1, 8+2t, 9+2t
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                uint4 rows[4];
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const uint32_t token = 8u * (r >> 1) + 2u * t + (r & 1);
                    rows[r] = *reinterpret_cast<const uint4 *>(v_tile + token * 256u + (((2u * g + hf) ^ swizzle_of(token)) << 4));
                }
                const uint32_t *r0 = reinterpret_cast<const uint32_t *>(&rows[0]);
                const uint32_t *r1 = reinterpret_cast<const uint32_t *>(&rows[1]);
                const uint32_t *r2 = reinterpret_cast<const uint32_t *>(&rows[2]);
                const uint32_t *r3 = reinterpret_cast<const uint32_t *>(&rows[3]);
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    const int j = hf * 8 + jj;
                    const uint32_t sel = (jj & 1) ? 0x7632u : 0x5410u;
                    const uint32_t b0 = __byte_perm(r0[jj >> 1], r1[jj >> 1], sel);
                    const uint32_t b1 = __byte_perm(r2[jj >> 1], r3[jj >> 1], sel);
                    acc[j][0] *= alpha;
                    acc[j][1] *= alpha;
                    mma_16816(acc[j], pa0, pa2, b0, b1);
                }
            }
        }
        if (!alive) {
            mbar_wait(&bars[0], phase_bits & 1u);
            mbar_wait(&bars[1], (phase_bits >> 1) & 1u);
            return;
        }
        float l = l_run;
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (g < G) {
            float *dst = partial_ptr(p, chunk, head_local * G + g);
            if (t == 0) {
                dst[0] = m_run;
                dst[1] = l;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                dst[2 + 16u * (2u * t) + j] = acc[j][0];
                dst[2 + 16u * (2u * t + 1u) + j] = acc[j][1];
            }
        }
        __syncwarp();
    }
}

}  // namespace

cudaError_t launch_dense_attention(const AttentionParams &p, cudaStream_t stream) {
    static LauncherState table[64];
    cudaError_t e;
    LauncherState *state = launcher_state(table, &e);
    if (!state) return e;
    if (!state->configured) {
        e = cudaFuncSetAttribute(dense_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(kSmemBytes));
        if (e != cudaSuccess) return e;
        state->configured = true;
    }
    dense_attention_kernel<<<state->sm_count, kThreads, kSmemBytes, stream>>>(p);
    return cudaPeekAtLastError();
}

}  // namespace cfb

extern "C" cf_status cf_b200_dense_attention_async(const cf_b200_dense_attention_desc *d, void *stream) {
    if (d == nullptr || d->struct_size != sizeof(cf_b200_dense_attention_desc) || d->abi_version != CF_B200_ABI_VERSION)
        return CF_ERR_INVALID_ARGUMENT;
    if (d->pool_k == nullptr || d->pool_v == nullptr || d->page_table == nullptr || d->seq_sealed_tokens == nullptr ||
        d->queries == nullptr || d->output == nullptr || d->workspace == nullptr || d->seq_count == 0 ||
        d->kv_head_count == 0 || d->query_head_count == 0 || d->query_head_count % d->kv_head_count != 0 ||
        (reinterpret_cast<uintptr_t>(d->workspace) & 255u) != 0 || (reinterpret_cast<uintptr_t>(d->pool_k) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(d->pool_v) & 15u) != 0)
        return CF_ERR_INVALID_ARGUMENT;
    if (d->head_dim != 128 || d->page_tokens != 16 || d->query_head_count / d->kv_head_count > 8) return CF_ERR_UNSUPPORTED;
    cfb::AttentionParams p{};
    p.kv_head_count = d->kv_head_count;
    p.query_head_count = d->query_head_count;
    p.head_dim = d->head_dim;
    p.page_tokens = d->page_tokens;
    p.block_size = 64;
    p.kv_head_begin = 0;
    p.kv_head_span = d->kv_head_count;
    p.group = d->query_head_count / d->kv_head_count;
    p.page_table = d->page_table;
    p.seq_sealed_tokens = d->seq_sealed_tokens;
    p.seq_slots = d->seq_slots;
    p.page_table_stride = d->page_table_stride;
    p.seq_count = d->seq_count;
    p.queries = d->queries;
    p.output = d->output;
    p.query_type = CF_B200_F16;
    p.output_type = CF_B200_F32;
    p.softmax_scale = d->softmax_scale;
    p.causal_window = d->causal_window;
    p.workspace = static_cast<uint8_t *>(d->workspace);
    p.layout = cfb::workspace_layout(d->seq_count, d->query_head_count, d->head_dim, d->workspace_bytes);
    p.min_pages_per_unit = d->min_pages_per_unit ? d->min_pages_per_unit : 16u;
    p.tail_capacity = d->page_tokens;
    p.pool_k = static_cast<const __half *>(d->pool_k);
    p.pool_v = static_cast<const __half *>(d->pool_v);
    if (p.layout.chunk_capacity < d->seq_count) return CF_ERR_INVALID_ARGUMENT;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (cfb::launch_plan(p, s) != cudaSuccess) return CF_ERR_CUDA;
    if (cfb::launch_dense_attention(p, s) != cudaSuccess) return CF_ERR_CUDA;
    if (cfb::launch_combine(p, s) != cudaSuccess) return CF_ERR_CUDA;
    return CF_OK;
}
