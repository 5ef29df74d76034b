// sealed_attention_prefix.cu — attention over a SHARED sealed prefix: pages that every sequence of the batch
// references (one copy in the arena, the same page ids at the head of every page-table row; the reference's
// shared-page semantics, src/multisequence_cache.cpp:235-292). Geometry: head_dim 128, page_tokens 16, block 64.
//
// The per-sequence kernel would decode such a page once per sequence. Here a page is decoded once per row tile and
// the contraction against all the query rows that share it runs on the tensor cores:
//
//   * rows = (sequence, query head of the kv head's group), 128 rows per CTA, 16 per warp (8 warps);
//     a unit is (prefix chunk, kv head, row tile).
//   * Round of 8 pages: warp w receives page j+w as one bulk async copy (mbarrier, bounded wait), decodes it with the
//     lane-per-block decoders and writes the symbols as int8 tiles to shared memory, K as [token][channel] with the
//     16-byte chunks of a row rotated by a per-token amount, V as [channel][token] — the layouts from which every
//     mma B fragment is one conflict-free 32-bit load. The next round's copy is issued as soon as the warp has
//     decoded, so it lands while the tensor-core phase runs.
//   * Then every warp runs S = Q K^T (Q fragments in registers), an online softmax over two pages at a time, and
//     O += P V for its 16 rows over the 8 decoded pages. Symbols become exact binary16 codes with byte permutes on
//     the way into the fragments; the page's K scale multiplies S, its V scale (relative to the step's first page)
//     multiplies P; P is fed as fp16 plus its rounding residue, so P V is accurate to fp32 level.
//   * Each unit writes (max, sum, weighted[128]) per row to the shared-prefix partials; the combine kernel merges
//     them with the per-sequence partials of the private pages and the tail.
//
// The contraction's k-order is permuted (channels 4t..4t+3 sit at k = 2t, 2t+1, 2t+8, 2t+9; S columns 2t+e of the
// two n-tiles are tokens 4t+e and 4t+2+e) so that A and B fragments come from contiguous bytes.

#include "lanes_decoders.cuh"

namespace cfb {
namespace {

using namespace lanes;

constexpr int kPvInFlight = 4;   // independent accumulators between an mma and the next one on the same accumulator
constexpr int kPWarps = 8;
constexpr int kPThreads = kPWarps * 32;
constexpr uint32_t kTileBytes = 4096;                       // K int8 [16][128] + V int8 [128][16]
constexpr uint32_t kOffStages = kTableBytes;
constexpr uint32_t kOffTiles = kOffStages + kPWarps * kStageBytes;
constexpr uint32_t kOffMeta = kOffTiles + kPWarps * kTileBytes;   // per page of the round: k scale, v scale, token count
constexpr uint32_t kOffBars = kOffMeta + kPWarps * 16;
constexpr uint32_t kPrefixSmem = kOffBars + kPWarps * 8;

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}

// Rotation (in 16-byte chunks) of token `tok`'s K row: the eight tokens of either n-tile get eight different values.
__device__ __forceinline__ uint32_t k_rotation(uint32_t tok) { return ((tok >> 2) << 1) | (tok & 1u); }

// Decode one record into the warp's tile. K quad q of lane l = token l/2, channels 64(l&1)+4q..+3; V quad q of lane l
// = stream positions 64l+4q..+3 of the token-minor V stream = [channel][token] bytes as they are.
template <class KLane, class VLane>
__device__ __forceinline__ void decode_to_tile(KLane &k, VLane &v, uint8_t *tile, uint32_t lane) {
    const uint32_t tok = lane >> 1, rot = k_rotation(tok);
    uint4 *k_row = reinterpret_cast<uint4 *>(tile + tok * 128u);
    uint4 *v_out = reinterpret_cast<uint4 *>(tile + 2048u + lane * 64u);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t kq[4], vq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if constexpr (KLane::kWholeQuads || VLane::kWholeQuads) {
                kq[j] = k.quad();
                vq[j] = v.quad();
            } else {
                k.reload();
                v.reload();
                uint32_t ke[4], ve[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    ke[i] = k.symbol();
                    ve[i] = v.symbol();
                }
                kq[j] = pack_low_bytes(ke[0], ke[1], ke[2], ke[3]);
                vq[j] = pack_low_bytes(ve[0], ve[1], ve[2], ve[3]);
            }
        }
        k_row[(4u * (lane & 1u) + c + rot) & 7u] = make_uint4(kq[0], kq[1], kq[2], kq[3]);
        v_out[c] = make_uint4(vq[0], vq[1], vq[2], vq[3]);
    }
}

template <class KLane>
__device__ __forceinline__ void decode_k_to_tile(KLane &k, uint8_t *tile, uint32_t lane) {
    const uint32_t tok = lane >> 1, rot = k_rotation(tok);
    uint4 *k_row = reinterpret_cast<uint4 *>(tile + tok * 128u);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t kq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) kq[j] = k.quad();
        k_row[(4u * (lane & 1u) + c + rot) & 7u] = make_uint4(kq[0], kq[1], kq[2], kq[3]);
    }
}

template <class VLane>
__device__ __forceinline__ void decode_v_to_tile(VLane &v, uint8_t *tile, uint32_t lane) {
    uint4 *v_out = reinterpret_cast<uint4 *>(tile + 2048u + lane * 64u);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t vq[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) vq[j] = v.quad();
        v_out[c] = make_uint4(vq[0], vq[1], vq[2], vq[3]);
    }
}

__global__ void __launch_bounds__(kPThreads, 1) prefix_attention_kernel(AttentionParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t *k_slot = reinterpret_cast<const uint32_t *>(smem);
    const uint32_t *v_slot = k_slot + 4096;
    const uint16_t *k_lut = reinterpret_cast<const uint16_t *>(v_slot + 4096);
    const uint16_t *v_lut = k_lut + 4096;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3u;
    uint8_t *stage = smem + kOffStages + warp * kStageBytes;
    uint8_t *tiles = smem + kOffTiles;
    float *meta = reinterpret_cast<float *>(smem + kOffMeta);   // [page of the round][4]: k scale, v scale, tokens, -
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + kOffBars) + warp;

    PlanHeader *hdr = plan_header(p);
    __shared__ uint32_t s_unit;
    const uint32_t shared_pages = hdr->shared_pages, chunks = hdr->shared_chunks, per_chunk = hdr->shared_pages_per_chunk;
    if (shared_pages == 0 || chunks == 0) return;   // uniform: nothing shared, or the plan refused the hint

    load_tables(smem, p, tid, kPThreads);
    if (lane == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    uint32_t phase = 0;
    bool expired = false;   // a bounded wait ran out: its copy may still be in flight when the kernel ends

    const uint32_t G = p.group;
    const uint32_t rows_total = p.seq_count * G;
    const uint32_t row_tiles = (rows_total + 127u) / 128u;
    const uint32_t unit_count = chunks * p.kv_head_span * row_tiles;
    const uint32_t *table_row = p.page_table + static_cast<uint64_t>(slot_of(p, 0)) * p.page_table_stride;

    for (;;) {
        __syncthreads();   // everyone has read the previous s_unit
        if (tid == 0) s_unit = atomicAdd(&hdr->next_shared_unit, 1u);
        __syncthreads();
        const uint32_t unit = s_unit;
        if (unit >= unit_count) break;
        const uint32_t tile_index = unit % row_tiles;
        const uint32_t head_local = (unit / row_tiles) % p.kv_head_span;
        const uint32_t chunk = unit / (row_tiles * p.kv_head_span);
        const uint32_t kv_head = p.kv_head_begin + head_local;
        const uint32_t page_begin = chunk * per_chunk, page_end = min(page_begin + per_chunk, shared_pages);

        // this lane's two rows: row g and row g+8 of the warp's sixteen
        const uint32_t row0 = tile_index * 128u + warp * 16u + g, row1 = row0 + 8u;
        const bool live0 = row0 < rows_total, live1 = row1 < rows_total;
        // Q as A fragments, k-step s: (a0, a2) = channels 16s+4t..+3 of row g, (a1, a3) the same of row g+8
        uint32_t qa[8][4];
        {
            const __half *qbase = reinterpret_cast<const __half *>(p.queries);
            const __half *q0 = qbase + (static_cast<uint64_t>(live0 ? row0 / G : 0u) * p.query_head_count + kv_head * G + (live0 ? row0 % G : 0u)) * 128u;
            const __half *q1 = qbase + (static_cast<uint64_t>(live1 ? row1 / G : 0u) * p.query_head_count + kv_head * G + (live1 ? row1 % G : 0u)) * 128u;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const uint2 x = live0 ? *reinterpret_cast<const uint2 *>(q0 + 16 * s + 4 * t) : make_uint2(0u, 0u);
                const uint2 y = live1 ? *reinterpret_cast<const uint2 *>(q1 + 16 * s + 4 * t) : make_uint2(0u, 0u);
                qa[s][0] = x.x;
                qa[s][1] = y.x;
                qa[s][2] = x.y;
                qa[s][3] = y.y;
            }
        }
        float o[16][4];
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f;
        float m0 = -CUDART_INF_F, m1 = -CUDART_INF_F, l0 = 0.0f, l1 = 0.0f;
        float v_unit = 1.0f;   // O is kept in units of the V scale of the step's first present page

        auto dir_entry = [&](uint32_t page) -> uint64_t {
            return p.page_dir[static_cast<uint64_t>(table_row[page]) * p.kv_head_count + kv_head];
        };
        auto entry_ok = [&](uint64_t entry) {
            const uint32_t units16 = static_cast<uint32_t>(CF_B200_DIR_LENGTH_UNITS(entry));
            return units16 != 0 && units16 * 16u <= kStageBytes - 32u;
        };
        auto issue = [&](uint64_t entry) {
            if (lane == 0 && entry_ok(entry)) {
                const uint32_t bytes = static_cast<uint32_t>(CF_B200_DIR_LENGTH_UNITS(entry)) * 16u;
                mbar_expect_tx(bar, bytes);
                bulk_load(stage, p.arena + 16ull * CF_B200_DIR_OFFSET_UNITS(entry), bytes, bar);
            }
        };

        uint64_t entry = page_begin + warp < page_end ? dir_entry(page_begin + warp) : 0ull;
        __syncthreads();   // the previous unit's tiles and stages are free
        issue(entry);

        for (uint32_t round = page_begin; round < page_end; round += kPWarps) {
            // ---- decode: warp w takes page round + w ----
            const uint32_t my_page = round + warp;
            uint8_t *tile = tiles + warp * kTileBytes;
            float k_scale = 0.0f, v_scale = 0.0f;
            uint32_t token_count = 0;
            if (my_page < page_end) {
                if (!entry_ok(entry)) {
                    if (lane == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
                } else if (!mbar_wait(bar, phase & 1u)) {
                    if (lane == 0) raise_status(p, CF_B200_DEVSTAT_WAIT_EXPIRED);
                    expired = true;
                } else {
                    phase ^= 1u;
                    const uint4 hv = *reinterpret_cast<const uint4 *>(stage);
                    if (!record_header_ok(hv, entry, p.codebook_id)) {
                        if (lane == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
                    } else {
                        const uint32_t k_units = hv.x & 0xffffu;
                        const uint32_t k_coder = hv.y & 0xffu, v_coder = (hv.y >> 8) & 0xffu;
                        const uint8_t *k_part = stage + 16, *v_part = k_part + 16u * k_units;
                        token_count = hv.y >> 16;
                        k_scale = __half2float(__ushort_as_half(static_cast<unsigned short>(hv.z & 0xffffu))) * (p.softmax_scale * kLog2e);
                        v_scale = __half2float(__ushort_as_half(static_cast<unsigned short>(hv.z >> 16)));
                        if (k_coder == CF_B200_CODER_RANS && v_coder == CF_B200_CODER_RANS) {
                            RansLane k, v;
                            k.open(k_part, lane, k_slot);
                            v.open(v_part, lane, v_slot);
                            decode_to_tile(k, v, tile, lane);
                        } else if (k_coder == CF_B200_CODER_HUFFMAN && v_coder == CF_B200_CODER_HUFFMAN) {
                            HuffLane k, v;
                            k.open(k_part, lane, k_lut);
                            v.open(v_part, lane, v_lut);
                            decode_to_tile(k, v, tile, lane);
                        } else if (k_coder == CF_B200_CODER_FIXED8 && v_coder == CF_B200_CODER_FIXED8) {
                            FixedLane k, v;
                            k.open(k_part, lane);
                            v.open(v_part, lane);
                            decode_to_tile(k, v, tile, lane);
                        } else {
                            if (k_coder == CF_B200_CODER_RANS) { RansLane k; k.open(k_part, lane, k_slot); decode_k_to_tile(k, tile, lane); }
                            else if (k_coder == CF_B200_CODER_HUFFMAN) { HuffLane k; k.open(k_part, lane, k_lut); decode_k_to_tile(k, tile, lane); }
                            else { FixedLane k; k.open(k_part, lane); decode_k_to_tile(k, tile, lane); }
                            if (v_coder == CF_B200_CODER_RANS) { RansLane v; v.open(v_part, lane, v_slot); decode_v_to_tile(v, tile, lane); }
                            else if (v_coder == CF_B200_CODER_HUFFMAN) { HuffLane v; v.open(v_part, lane, v_lut); decode_v_to_tile(v, tile, lane); }
                            else { FixedLane v; v.open(v_part, lane); decode_v_to_tile(v, tile, lane); }
                        }
                    }
                }
            }
            if (lane == 0) {
                meta[4 * warp] = k_scale;
                meta[4 * warp + 1] = v_scale;
                meta[4 * warp + 2] = __uint_as_float(token_count);   // 0: the page contributes nothing
            }
            __syncwarp();   // every lane is done with the stage
            entry = my_page + kPWarps < page_end ? dir_entry(my_page + kPWarps) : 0ull;
            if (my_page + kPWarps < page_end) issue(entry);
            __syncthreads();   // tiles of the round are complete

            // ---- tensor-core phase: this warp's 16 rows against the round's pages, two pages per softmax step ----
            const uint32_t in_round = min(static_cast<uint32_t>(kPWarps), page_end - round);
            for (uint32_t pg = 0; pg < in_round; pg += 2) {
                float s[2][2][4];   // [page of the pair][n-tile][fragment]
                float ks[2], vs[2];
                uint32_t tc[2];
                if (__float_as_uint(meta[4 * pg + 2]) == 0u && (pg + 1 >= in_round || __float_as_uint(meta[4 * pg + 6]) == 0u))
                    continue;   // neither page of the pair is present (uniform across the block)
                const uint32_t *krow[2][2];
                uint32_t krot[2];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const bool present = pg + h < in_round;
                    ks[h] = present ? meta[4 * (pg + h)] : 0.0f;
                    vs[h] = present ? meta[4 * (pg + h) + 1] : 0.0f;
                    tc[h] = present ? __float_as_uint(meta[4 * (pg + h) + 2]) : 0u;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        s[h][nt][0] = s[h][nt][1] = s[h][nt][2] = s[h][nt][3] = 0.0f;
                        const uint32_t tok = 4u * (g >> 1) + (g & 1u) + 2u * nt;   // the token of column n = g
                        krow[h][nt] = reinterpret_cast<const uint32_t *>(tiles + (pg + h) * kTileBytes + tok * 128u) + t;
                        krot[nt] = k_rotation(tok);
                    }
                }
#pragma unroll
                for (int ss = 0; ss < 8; ++ss)   // k-steps outside: consecutive mma feed different accumulators
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        if (tc[h] == 0u) continue;   // uniform across the warp
#pragma unroll
                        for (int nt = 0; nt < 2; ++nt) {
                            uint32_t b0, b1;
                            quad_to_half2(krow[h][nt][4u * ((ss + krot[nt]) & 7u)], b0, b1);
                            mma_16816(s[h][nt], qa[ss][0], qa[ss][1], qa[ss][2], qa[ss][3], b0, b1);
                        }
                    }
                // scores, masks, row maxima (row g: fragments 0,1; row g+8: fragments 2,3; columns 2t+e)
                float r0 = -CUDART_INF_F, r1 = -CUDART_INF_F;
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const uint32_t tok = 4u * t + 2u * nt + e;
                            const bool vis = tok < tc[h];
                            s[h][nt][e] = vis ? s[h][nt][e] * ks[h] : -CUDART_INF_F;
                            s[h][nt][2 + e] = vis ? s[h][nt][2 + e] * ks[h] : -CUDART_INF_F;
                            r0 = fmaxf(r0, s[h][nt][e]);
                            r1 = fmaxf(r1, s[h][nt][2 + e]);
                        }
                r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 1));
                r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, 2));
                r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 1));
                r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, 2));
                const float n0 = fmaxf(m0, r0), n1 = fmaxf(m1, r1);
                const float z0 = n0 == -CUDART_INF_F ? 0.0f : n0, z1 = n1 == -CUDART_INF_F ? 0.0f : n1;
                const float v_ref = tc[0] ? vs[0] : vs[1];
                const float v_ratio = v_unit / v_ref;
                v_unit = v_ref;
                const float a0 = exp2f(m0 - z0), a1 = exp2f(m1 - z1);
                const float beta0 = a0 * v_ratio, beta1 = a1 * v_ratio;
                const float vr[2] = {tc[0] ? vs[0] / v_ref : 0.0f, tc[1] ? vs[1] / v_ref : 0.0f};
                m0 = n0;
                m1 = n1;
                float sum0 = 0.0f, sum1 = 0.0f;
                uint32_t pa[2][2][4];   // [page][hi | residue][A fragment registers]
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    float pr[2][4];
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 2; ++e) {
                            const float w0 = exp2f(s[h][nt][e] - z0), w1 = exp2f(s[h][nt][2 + e] - z1);
                            sum0 += w0;
                            sum1 += w1;
                            pr[nt][e] = w0 * vr[h];       // the page's V scale relative to the step's unit rides on P
                            pr[nt][2 + e] = w1 * vr[h];
                        }
                    // A fragment: a0 = row g, k 2t,2t+1 = tile 0; a1 = row g+8 of tile 0; a2, a3 = the same of tile 1
                    pa[h][0][0] = pack_half2(pr[0][0], pr[0][1]);
                    pa[h][0][1] = pack_half2(pr[0][2], pr[0][3]);
                    pa[h][0][2] = pack_half2(pr[1][0], pr[1][1]);
                    pa[h][0][3] = pack_half2(pr[1][2], pr[1][3]);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const __half2 hi = *reinterpret_cast<const __half2 *>(&pa[h][0][i]);
                        const float2 back = __half22float2(hi);
                        const int nt = i >> 1, base = (i & 1) * 2;
                        pa[h][1][i] = pack_half2(pr[nt][base] - back.x, pr[nt][base + 1] - back.y);
                    }
                }
                l0 = l0 * a0 + sum0;
                l1 = l1 * a1 + sum1;
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    o[j][0] *= beta0;
                    o[j][1] *= beta0;
                    o[j][2] *= beta1;
                    o[j][3] *= beta1;
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    if (tc[h] == 0u) continue;
                    const uint32_t *vt = reinterpret_cast<const uint32_t *>(tiles + (pg + h) * kTileBytes + 2048u);
#pragma unroll
                    for (int j0 = 0; j0 < 16; j0 += kPvInFlight) {   // channels 8j + g, tokens 4t..4t+3
                        uint32_t b0[kPvInFlight], b1[kPvInFlight];
#pragma unroll
                        for (int j = 0; j < kPvInFlight; ++j) quad_to_half2(vt[(8u * (j0 + j) + g) * 4u + t], b0[j], b1[j]);
#pragma unroll
                        for (int j = 0; j < kPvInFlight; ++j) mma_16816(o[j0 + j], pa[h][0][0], pa[h][0][1], pa[h][0][2], pa[h][0][3], b0[j], b1[j]);
#pragma unroll
                        for (int j = 0; j < kPvInFlight; ++j) mma_16816(o[j0 + j], pa[h][1][0], pa[h][1][1], pa[h][1][2], pa[h][1][3], b0[j], b1[j]);
                    }
                }
            }
            __syncthreads();   // the round's tiles may be overwritten
        }

        // ---- partials of the unit: one (max, sum, weighted[128]) per row ----
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const uint32_t row = r ? row1 : row0;
            if (!(r ? live1 : live0)) continue;
            float *dst = shared_partial_ptr(p, chunk, row / G, head_local * G + row % G);
            if (t == 0) {
                dst[0] = r ? m1 : m0;
                dst[1] = r ? l1 : l0;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j)
                *reinterpret_cast<float2 *>(dst + 2 + 8 * j + 2 * t) = make_float2(o[j][2 * r] * v_unit, o[j][2 * r + 1] * v_unit);
        }
    }
    // A copy is issued only for a page the loop goes on to wait for, so nothing is in flight here unless a wait ran
    // out; then the copy gets one more bounded chance to land before the block's shared memory goes away.
    if (expired) mbar_wait(bar, phase & 1u);
}

}  // namespace

cudaError_t launch_prefix_attention(const AttentionParams &p, cudaStream_t stream) {
    static int sm_count = 0;
    static bool configured = false;
    if (!configured) {
        int device = 0;
        cudaError_t e = cudaGetDevice(&device);
        if (e != cudaSuccess) return e;
        e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(prefix_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPrefixSmem));
        if (e != cudaSuccess) return e;
        configured = true;
    }
    prefix_attention_kernel<<<sm_count, kPThreads, kPrefixSmem, stream>>>(p);
    return cudaPeekAtLastError();
}

}  // namespace cfb
