// sealed_attention_lanes.cu — the hot kernel: decode-step attention over sealed pages for the geometry
// head_dim 128, page_tokens 16, block_size 64 (32 blocks per stream). Query groups larger than 4 heads per kv head are
// served four heads at a time (the unit is then decoded once per sub-group). Blocks of 128 and 256 symbols (16 and 8
// blocks per stream) run the same kernel behind a staging step, see stage_blocks below.
//
// What it computes is what src/cuda/paged_kv_attention.cu:183-276 computes for one query token; how it runs is new:
//
//   * One WARP owns one (chunk, kv head) unit. A page record arrives in shared memory as ONE bulk async copy
//     (cp.async.bulk + mbarrier), double buffered per warp. Coding tables (rANS slot table, Huffman LUT) are loaded
//     once per CTA. No thread ever reads page bytes from global memory directly.
//   * Lane l decodes block l of the K stream and block l of the V stream, interleaved so that the two independent
//     decoder chains overlap. Symbols never leave registers: four symbols are packed into one register, turned
//     into two fp16 pairs with byte permutes (bias 1024, exact), and fed straight into mma.sync fragments.
//       K block l = token l/2, channels 64*(l&1)..+63  -> A operand of S = K * Q^T   (16 mma per page)
//       V block l = channels 4l..4l+3, all 16 tokens   -> B operand of O^T = P' * V  (16 mma per page)
//     The query group is the other operand, laid out with zeros so that every lane's private slice of the
//     contraction lands in its own output column/row. Tensor cores do the whole contraction for the group;
//     a code is decoded once for all query heads (the reference re-decodes per query head,
//     paged_kv_attention.cu:205-207).
//   * Online softmax per page in fp32; partial (max, sum, weighted) per unit goes to the split-KV workspace and is
//     merged by the combine kernel (cf_online_softmax_merge rule, src/runtime/kv_runtime.cpp:219-243).
//   * Every wait on a copy is bounded; on expiry the warp raises CF_B200_DEVSTAT_WAIT_EXPIRED and leaves.

#include <math_constants.h>

#include <atomic>
#include <type_traits>

#include "lanes_decoders.cuh"

namespace cfb {
namespace {

using namespace lanes;

#ifndef CFB_LANES_WARPS
#define CFB_LANES_WARPS 16
#endif
#ifndef CFB_LANES_WARPS2
#define CFB_LANES_WARPS2 16
#endif
// Warps per CTA (one CTA per SM): the four-head kernel and the kernels whose query rows live in shared memory (they
// need 2.3 KB more per warp) are sized separately.
// The kernels for larger blocks (NB = 16 or 8 blocks per stream) keep a 5 KB symbol tile per warp instead of a second
// record stage: a record is free for the next copy as soon as it has been decoded into the tile.
#ifndef CFB_LANES_WARPS_BIG
#define CFB_LANES_WARPS_BIG 16
#endif
template <int NG, int NB = 32> constexpr int kWarpsOf = NB != 32 ? (NG == 1 ? CFB_LANES_WARPS_BIG : 14) : NG == 1 ? CFB_LANES_WARPS : CFB_LANES_WARPS2;
template <int NG, int NB = 32> constexpr int kThreadsOf = kWarpsOf<NG, NB> * 32;
// Per-warp running state of one unit; NG = number of four-head query groups served by one decode pass.
// kDim = head_dim: a lane holds kDim / 8 quads of each stream (K: kDim / 2 channels of one token; V: kDim / 32 channels,
// every token).
template <int NG, int kDim = 128>
struct UnitState {
    float score[NG][4];      // S fragments of the current page
    float acc[NG][kDim / 32][4];   // O fragments: [group][channel of the lane's V block][fragment register]
    uint32_t vq[kDim / 8];   // V symbols of the current page, [channel*4 + token quad]
    float m0[NG], m1[NG], l0[NG], l1[NG];  // running max / partial sum of the lane's two heads of each group
    uint32_t *dump;          // kDump only: where this lane's quads of the current record go (K at +0, V at +512 words)
};

// What the kernel does with the symbols: attention; or (measurement) fold them into a checksum; or (test) store
// every quad the lane decoders yield to global memory, so that they can be compared symbol for symbol.
constexpr int kAttend = 0, kFold = 1, kDump = 2;
// The softmax weights go to the tensor cores as binary16 (value + rounding residue) scaled by this power of two.
constexpr float kWeightScale = 32768.0f;

// Where a lane finds its B fragments of S = K * Q^T (column n = parity*4 + head; zero where the lane's slice of the
// contraction belongs to the other token of the pair).
//   QRegs: held in registers, one group of four heads.
//   QSmem: the query rows of up to eight heads sit in the warp's shared memory as [head][half][64 channels] with a
//   row stride of 36 words, which puts the eight rows one load touches into different banks; a lane reads two words
//   of row (head g&3 of the group, half t&1), or of a zero row when the column is not its own.
template <int kQuads>
struct QRegsT {
    uint32_t bq[kQuads][2];
    template <int GRP>
    __device__ __forceinline__ void get(int q, uint32_t &b0, uint32_t &b1) const {
        b0 = bq[q][0];
        b1 = bq[q][1];
    }
};
using QRegs = QRegsT<16>;
struct QSmem {
    uint32_t addr, group_stride;  // byte address of the lane's row for group 0; distance to the row for group 1 (0 on the zero row)
    template <int GRP>
    __device__ __forceinline__ void get(int q, uint32_t &b0, uint32_t &b1) const {
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr + GRP * group_stride + 8u * q));
    }
};

template <int NG, int kDim, class QSrc>
__device__ __forceinline__ void score_quad(UnitState<NG, kDim> &u, const QSrc &qs, int q, uint32_t kq) {
    uint32_t lo, hi, b0, b1;
    quad_to_half2(kq, lo, hi);
    qs.template get<0>(q, b0, b1);
    mma_16816(u.score[0], lo, 0u, hi, 0u, b0, b1);
    if constexpr (NG == 2) {
        qs.template get<1>(q, b0, b1);
        mma_16816(u.score[1], lo, 0u, hi, 0u, b0, b1);
    }
}

// kFold: the symbols are only folded into a checksum (u.vq[0]) — the decode work of the kernel without its attention.
// kDump: lane l's quad q of a stream holds the symbols 64 l + 4 q .. + 3 of that stream, first symbol in byte 0.
template <int kMode = kAttend, class KLane, class VLane, int NG, class QSrc>
__device__ __forceinline__ void decode_fused(KLane &k, VLane &v, UnitState<NG> &u, const QSrc &qs) {
    if constexpr (KLane::kWholeQuads || VLane::kWholeQuads) {
#pragma unroll
        for (int q = 0; q < 16; ++q) {
            const uint32_t kq = k.quad(q);
            if constexpr (kMode == kFold) {
                u.vq[0] ^= kq ^ v.quad(q);
            } else if constexpr (kMode == kDump) {
                u.dump[q] = kq;
                u.dump[512 + q] = v.quad(q);
            } else {
                u.vq[q] = v.quad(q);
                score_quad(u, qs, q, kq);
            }
        }
    } else {
        // two independent decoder chains, interleaved symbol by symbol; each window is refilled as rarely as its
        // coder's worst case allows, four symbols make one packed register
        uint32_t ke[4], ve[4];
#pragma unroll
        for (int i = 0; i < 64; ++i) {
            if (i % KLane::kSymbolsPerReload == 0) k.reload();
            if (i % VLane::kSymbolsPerReload == 0) v.reload();
            ke[i & 3] = k.symbol();
            ve[i & 3] = v.symbol();
            if ((i & 3) == 3) {
                if constexpr (kMode == kFold) {
                    u.vq[0] ^= pack_low_bytes(ve[0], ve[1], ve[2], ve[3]) ^ pack_low_bytes(ke[0], ke[1], ke[2], ke[3]);
                } else if constexpr (kMode == kDump) {
                    u.dump[i >> 2] = pack_low_bytes(ke[0], ke[1], ke[2], ke[3]);
                    u.dump[512 + (i >> 2)] = pack_low_bytes(ve[0], ve[1], ve[2], ve[3]);
                } else {
                    u.vq[i >> 2] = pack_low_bytes(ve[0], ve[1], ve[2], ve[3]);
                    score_quad(u, qs, i >> 2, pack_low_bytes(ke[0], ke[1], ke[2], ke[3]));
                }
            }
        }
    }
}

// Both streams nibble-split with the same coder: 32 interleaved steps per stream, a quad from every two of them.
template <int kMode = kAttend, class Lane, int NG, class QSrc>
__device__ __forceinline__ void decode_fused_split(Lane &k, Lane &v, UnitState<NG> &u, const QSrc &qs) {
    uint32_t ke[2], ve[2], kw = 0u, vw = 0u;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        if (i % 4 == 0) {
            k.reload();
            v.reload();
        }
        ke[i & 1] = k.symbol();
        ve[i & 1] = v.symbol();
        if (i & 1) {
            const int q = i >> 1;
            if ((q & 1) == 0) {
                kw = k.lo_word(q >> 1);
                vw = v.lo_word(q >> 1);
            } else {
                kw >>= 4;
                vw >>= 4;
            }
            const uint32_t kq = merge_split_quad(ke[0], ke[1], kw), vq = merge_split_quad(ve[0], ve[1], vw);
            if constexpr (kMode == kFold) {
                u.vq[0] ^= kq ^ vq;
            } else if constexpr (kMode == kDump) {
                u.dump[q] = kq;
                u.dump[512 + q] = vq;
            } else {
                u.vq[q] = vq;
                score_quad(u, qs, q, kq);
            }
        }
    }
}

template <int kMode = kAttend, class KLane, int NG, class QSrc>
__device__ __forceinline__ void decode_k_only(KLane &k, UnitState<NG> &u, const QSrc &qs) {
#pragma unroll
    for (int q = 0; q < 16; ++q) {
        const uint32_t kq = k.quad(q);
        if constexpr (kMode == kFold) u.vq[0] ^= kq;
        else if constexpr (kMode == kDump) u.dump[q] = kq;
        else score_quad(u, qs, q, kq);
    }
}

template <int kMode = kAttend, class VLane, int NG>
__device__ __forceinline__ void decode_v_only(VLane &v, UnitState<NG> &u) {
#pragma unroll
    for (int q = 0; q < 16; ++q) {
        const uint32_t vq = v.quad(q);
        if constexpr (kMode == kFold) u.vq[0] ^= vq;
        else if constexpr (kMode == kDump) u.dump[512 + q] = vq;
        else u.vq[q] = vq;
    }
}

// ---- blocks of 128 / 256 symbols (NB = 16 / 8 blocks per stream) ------------------------------------------------
// The attention part of the kernel wants lane l to hold symbols 64 l .. 64 l + 63 of both streams. With larger blocks
// there are fewer blocks than lanes, so the decode is laid out differently and its result re-dealt through a
// per-warp tile in shared memory: lanes 0 .. NB-1 decode the K blocks while lanes 16 .. 16+NB-1 decode the V blocks
// (at NB = 16 every lane is busy and a page costs as many decoder steps per lane as with 64-symbol blocks; at NB = 8
// half the lanes idle), every four quads leave as one 16-byte store, and after a warp barrier each lane reads its
// sixteen K quads and sixteen V quads back with 16-byte loads. A tile row is one lane's 64 symbols plus 16 bytes
// of padding (row stride 80 bytes), which keeps both the stores and the loads off each other's banks; the V tile
// sits 16 bytes further for the same reason.
// The same staging serves head_dim 96, 64 and 32 (streams of 1536 / 1024 / 512 symbols): a lane's share is then
// kDim / 2 symbols of each stream (K: half of one token's channels; V: kDim / 32 channels, every token). At head_dim
// 96 with 64-symbol blocks there are 48 blocks for 32 lanes: every lane takes block `lane`, the first sixteen
// lanes also block `lane + 32`.
// one lane's kDim / 2 symbols + padding that keeps the row stride off multiples of 64 bytes
template <int kDim> constexpr uint32_t kTileRowOf = kDim / 2u + ((kDim / 2u + 16u) % 64u == 0 ? 32u : 16u);
template <int kDim> constexpr uint32_t kTileStreamOf = 32u * kTileRowOf<kDim>;
constexpr uint32_t kTileBytes = 2u * kTileStreamOf<128> + 32u;

template <int NB, int kDim, class Lane>
__device__ __forceinline__ void stage_with(Lane &d, uint32_t block, uint8_t *tile) {
    constexpr int kQuads = 4 * kDim / NB;   // per block
    constexpr uint32_t kRowQuads = kDim / 8;
#pragma unroll 2
    for (int q = 0; q < kQuads; q += 4) {
        const uint32_t a = d.quad(q), b = d.quad(q + 1), c = d.quad(q + 2), e = d.quad(q + 3);
        const uint32_t at = block * kQuads + q;   // quad index in the stream: row = at / kRowQuads, column = at % kRowQuads
        *reinterpret_cast<uint4 *>(tile + (at / kRowQuads) * kTileRowOf<kDim> + (at % kRowQuads) * 4u) = make_uint4(a, b, c, e);
    }
}

// One lane's share: block `block` of the part, whatever its coder.
template <int NB, int kDim>
__device__ __forceinline__ void stage_blocks(const uint8_t *part, uint32_t part_bytes, uint32_t coder, uint32_t block,
                                             const uint32_t *slot_table, const uint16_t *lut, uint8_t *tile) {
    constexpr int kSyms = 16 * kDim;
    if (coder == CF_B200_CODER_RANS_SPLIT4) {
        RansSplitLaneT<NB, kSyms> d;
        d.open(part, part_bytes, block, slot_table);
        stage_with<NB, kDim>(d, block, tile);
    } else if (coder == CF_B200_CODER_HUFFMAN_SPLIT4) {
        HuffSplitLaneT<NB, kSyms> d;
        d.open(part, part_bytes, block, lut);
        stage_with<NB, kDim>(d, block, tile);
    } else if (coder == CF_B200_CODER_RANS) {
        RansLaneT<NB> d;
        d.open(part, part_bytes, block, slot_table);
        stage_with<NB, kDim>(d, block, tile);
    } else if (coder == CF_B200_CODER_HUFFMAN) {
        HuffLaneT<NB> d;
        d.open(part, part_bytes, block, lut);
        stage_with<NB, kDim>(d, block, tile);
    } else {
        FixedLaneT<NB, kSyms> d;
        d.open(part, part_bytes, block);
        stage_with<NB, kDim>(d, block, tile);
    }
}

// Shared memory of one warp: two record stages, the softmax scratch, two mbarriers and (NG = 2) the query rows.
//   scratch: P rows fp16 high halves [4 NG][16] | low halves [4 NG][16] | 128 zero bytes | alpha[4 NG]
template <int NG, int NB = 32>
struct WarpLayout {
    static constexpr uint32_t kPBytes = 4 * NG * 16 * 2;
    static constexpr uint32_t kStages = NB == 32 ? 2 : 1;
    static constexpr uint32_t kPLo = kStages * kStageBytes + kPBytes;
    static constexpr uint32_t kZero = kPLo + kPBytes;
    static constexpr uint32_t kAlpha = kZero + 128;
    static constexpr uint32_t kBars = kAlpha + 4 * NG * 4;
    static constexpr uint32_t kQRows = kBars + 32;
    static constexpr uint32_t kQRowWords = 36;
    static constexpr uint32_t kTile = (kQRows + (NG == 2 ? 16 * kQRowWords * 4 : 0) + 15u) / 16u * 16u;   // NB != 32 only
    static constexpr uint32_t kBytes = kTile + (NB != 32 ? kTileBytes : 0u);
    static constexpr uint32_t kSmem = kTableBytes + kWarpsOf<NG, NB> * kBytes;
};
static_assert(WarpLayout<1>::kSmem <= 232448 && WarpLayout<2>::kSmem <= 232448 && WarpLayout<1, 16>::kSmem <= 232448 &&
              WarpLayout<2, 16>::kSmem <= 232448, "a CTA has 227 KB of shared memory");

// kSplitQ (with NG = 2): the queries are fp32. A pass serves four heads; their rows are split into binary16(q) and
// binary16(q - binary16(q)), stored as the rows of group 0 and group 1, the two score fragments are added, and one
// softmax / P V follows: the scores equal fp32-query scores to 2^-22 relative, at the cost of a second score mma.
template <int NG, int kMode = kAttend, bool kSplitQ = false, int NB = 32, int kDim = 128>
__global__ void __launch_bounds__(kThreadsOf<NG, NB>, 1) lanes_attention_kernel(AttentionParams p) {
    constexpr bool kProbe = kMode != kAttend;
    static_assert(!kSplitQ || NG == 2, "split queries use the two-group query layout");
    static_assert(NB == 32 || NB == 24 || NB == 16 || NB == 12 || NB == 8 || NB == 4, "blocks per stream");
    static_assert(kDim == 128 || ((kDim == 96 || kDim == 64 || kDim == 32) && NB != 32), "other head_dims go through the staging tile");
    constexpr int kQ = kDim / 8, kVCh = kDim / 32, kSyms = 16 * kDim;   // quads per lane and stream; V channels per lane
    constexpr uint32_t kRowWords = kDim / 4;   // words of half a query row (the channels one lane's K block covers)
    using L = WarpLayout<NG, NB>;
    using QSrc = typename std::conditional<NG == 1, QRegsT<kQ>, QSmem>::type;
    constexpr uint32_t kPassHeads = kSplitQ ? 4u : 4u * NG;
    constexpr int NS = kSplitQ ? 1 : NG;   // groups that go through softmax and P V
    extern __shared__ __align__(128) uint8_t smem[];
    uint32_t *k_slot = reinterpret_cast<uint32_t *>(smem);
    uint32_t *v_slot = k_slot + 4096;
    uint16_t *k_lut = reinterpret_cast<uint16_t *>(v_slot + 4096);
    uint16_t *v_lut = k_lut + 4096;

    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint8_t *warp_mem = smem + kTableBytes + warp * L::kBytes;
    __half *p_rows = reinterpret_cast<__half *>(warp_mem + L::kStages * kStageBytes);   // [4 NG][16] fp16(p)
    __half *p_rows_lo = reinterpret_cast<__half *>(warp_mem + L::kPLo);        // [4 NG][16] fp16(p - fp16(p))
    const __half *zero_row = reinterpret_cast<const __half *>(warp_mem + L::kZero);
    float *alpha_s = reinterpret_cast<float *>(warp_mem + L::kAlpha);          // [4 NG]
    uint64_t *bars = reinterpret_cast<uint64_t *>(warp_mem + L::kBars);
    uint32_t *q_rows = reinterpret_cast<uint32_t *>(warp_mem + L::kQRows);     // NG == 2 only

    load_tables(smem, p, tid, kThreadsOf<NG, NB>);   // coding tables: once per CTA
    reinterpret_cast<uint32_t *>(warp_mem + L::kZero)[lane] = 0u;   // the zero row inactive lanes read their fragments from
    if (lane == 0) {
        mbar_init(&bars[0], 1);
        mbar_init(&bars[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    PlanHeader *hdr = plan_header(p);
    const uint32_t subgroups = (p.group + kPassHeads - 1u) / kPassHeads;   // 4 NG query heads per pass
    const uint32_t unit_count = hdr->chunk_count * p.kv_head_span * subgroups;
    const uint32_t pages_per_unit = hdr->pages_per_unit;
    const uint32_t g = lane >> 2, t = lane & 3u;
    uint32_t phase_bits = 0u;  // bit s: parity the next wait on stage s expects

    // fixed lane roles
    const uint32_t q_head_of_col = g & 3u;                 // S columns: n = parity*4 + head
    const bool q_col_mine = (t >> 1) == (g >> 2);
    const uint32_t my_token = 2u * g + (t >> 1);           // S fragment: row g, this lane's token
    const uint32_t my_head0 = 2u * (t & 1u);               // S fragment: this lane's two heads (of each group)
    const uint32_t o_head = g & 3u;                        // O fragments: all of this lane's outputs are one head per group
    const bool row_lo_mine = t == (g >> 2), row_hi_mine = t == (g >> 2) + 2u;   // P rows with lane tag t

    for (;;) {
        uint32_t unit = 0;
        if (lane == 0) unit = atomicAdd(&hdr->next_unit, 1u);
        unit = __shfl_sync(0xffffffffu, unit, 0);
        if (unit >= unit_count) break;
        const uint32_t sub = unit % subgroups;
        const uint32_t chunk = (unit / subgroups) / p.kv_head_span;
        const uint32_t head_local = (unit / subgroups) % p.kv_head_span;
        const uint32_t kv_head = p.kv_head_begin + head_local;
        const uint32_t G = min(kPassHeads, p.group - kPassHeads * sub);       // query heads served by this pass
        const uint32_t q_head_base = kv_head * p.group + kPassHeads * sub;    // first of them
        const uint32_t out_head_base = head_local * p.group + kPassHeads * sub;
        // the chunk's start-up record, written by the plan kernel (which also took the shared pages off its front)
        const uint4 *ci = reinterpret_cast<const uint4 *>(chunk_info(p) + chunk);
        const uint4 ci0 = ci[0];
        const uint4 ci1 = ci[1];
        const uint32_t slot = ci0.y, sealed = ci0.z, qpos = ci0.w, page_begin = ci1.x, q_row = ci1.y;   // ci0.x = batch entry
        const uint32_t first_token = window_begin(qpos, p.causal_window);
        const uint32_t pages = min((sealed + 15u) / 16u, qpos / 16u + 1u);
        const uint32_t page_end = min(page_begin + pages_per_unit, pages);
        const uint32_t n_pages = page_end > page_begin ? page_end - page_begin : 0u;
        const uint32_t *table_row = p.page_table + static_cast<uint64_t>(slot) * p.page_table_stride;

        QSrc qs;
        if constexpr (NG == 1) {
            const bool live = q_col_mine && q_head_of_col < G;
            const __half *qrow = reinterpret_cast<const __half *>(p.queries) +
                                 (static_cast<uint64_t>(q_row) * p.query_head_count + q_head_base + q_head_of_col) * kDim +
                                 (kDim / 2) * (t & 1u);
#pragma unroll
            for (int s = 0; s < kQ; ++s) {
                uint2 v = make_uint2(0u, 0u);
                if (live) v = *reinterpret_cast<const uint2 *>(qrow + 4 * s);
                qs.bq[s][0] = v.x;
                qs.bq[s][1] = v.y;
            }
        } else if constexpr (kSplitQ) {
            const float2 *qsrc = reinterpret_cast<const float2 *>(
                reinterpret_cast<const float *>(p.queries) + (static_cast<uint64_t>(q_row) * p.query_head_count + q_head_base) * kDim);
            __syncwarp();  // the previous unit's readers are done
#pragma unroll
            for (int j = 0; j < kDim / 16; ++j) {    // 4 heads x kDim / 2 channel pairs; row = head*2 + half, residues 8 rows further
                const uint32_t i = lane + 32u * j, head = i / (2u * kRowWords);
                const float2 x = head < G ? qsrc[i] : make_float2(0.0f, 0.0f);
                const __half2 hi = __floats2half2_rn(x.x, x.y);
                const float2 back = __half22float2(hi);
                const __half2 lo = __floats2half2_rn(x.x - back.x, x.y - back.y);
                q_rows[(i / kRowWords) * L::kQRowWords + i % kRowWords] = *reinterpret_cast<const uint32_t *>(&hi);
                q_rows[(i / kRowWords + 8u) * L::kQRowWords + i % kRowWords] = *reinterpret_cast<const uint32_t *>(&lo);
            }
            __syncwarp();
            qs.addr = q_col_mine ? smem_addr(q_rows + (q_head_of_col * 2u + (t & 1u)) * L::kQRowWords) : smem_addr(zero_row);
            qs.group_stride = q_col_mine ? 8u * L::kQRowWords * 4u : 0u;
        } else {
            const uint32_t *qsrc = reinterpret_cast<const uint32_t *>(
                reinterpret_cast<const __half *>(p.queries) + (static_cast<uint64_t>(q_row) * p.query_head_count + q_head_base) * kDim);
            __syncwarp();  // the previous unit's readers are done
#pragma unroll
            for (int j = 0; j < kDim / 8; ++j) {   // 8 heads x kDim / 2 words; row = head*2 + half
                const uint32_t i = lane + 32u * j, head = i / (2u * kRowWords);
                q_rows[(i / kRowWords) * L::kQRowWords + i % kRowWords] = head < G ? qsrc[i] : 0u;
            }
            __syncwarp();
            qs.addr = q_col_mine ? smem_addr(q_rows + (q_head_of_col * 2u + (t & 1u)) * L::kQRowWords) : smem_addr(zero_row);
            qs.group_stride = q_col_mine ? 8u * L::kQRowWords * 4u : 0u;
        }

        UnitState<NG, kDim> u;
        if constexpr (kProbe) u.vq[0] = 0u;
        u.dump = nullptr;
#pragma unroll
        for (int n = 0; n < NG; ++n) {
#pragma unroll
            for (int a = 0; a < kVCh; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) u.acc[n][a][b] = 0.0f;
            u.m0[n] = u.m1[n] = -CUDART_INF_F;
            u.l0[n] = u.l1[n] = 0.0f;
        }
        float v_scale_prev = 1.0f;

        // bit 63 of an entry (reserved, 0 in the directory) marks the page of the wait-expiry test: armed, never fetched
        auto load_entry = [&](uint32_t page) -> uint64_t {
            const uint32_t page_id = table_row[page];
            const uint64_t entry = p.page_dir[static_cast<uint64_t>(page_id) * p.kv_head_count + kv_head];
            return page_id == p.skip_copy_page ? entry | (1ull << 63) : entry;
        };
        auto issue = [&](uint32_t st, uint64_t entry) {
            const uint32_t units16 = static_cast<uint32_t>(CF_B200_DIR_LENGTH_UNITS(entry));
            if (lane == 0 && units16 != 0 && units16 * 16u <= kStageBytes - 32u) {
                mbar_expect_tx(&bars[st], units16 * 16u);
                if (!(entry >> 63))
                    bulk_load(warp_mem + st * kStageBytes, p.arena + 16ull * CF_B200_DIR_OFFSET_UNITS(entry), units16 * 16u, &bars[st]);
            }
        };
        auto entry_ok = [&](uint64_t entry) {
            const uint32_t units16 = static_cast<uint32_t>(CF_B200_DIR_LENGTH_UNITS(entry));
            return units16 != 0 && units16 * 16u <= kStageBytes - 32u;
        };

        uint64_t entry_cur = n_pages ? load_entry(page_begin) : 0ull;
        uint64_t entry_next = n_pages > 1 ? load_entry(page_begin + 1) : 0ull;
        __syncwarp();
        issue(0, entry_cur);
        bool alive = true;

        for (uint32_t i = 0; i < n_pages; ++i) {
            const uint32_t st = NB == 32 ? (i & 1u) : 0u;
            uint64_t entry_after = 0ull;
            bool next_issued = NB == 32;
            if (i + 1 < n_pages) {
                if constexpr (NB == 32) {
                    __syncwarp();  // every lane is done with the other stage (page i-1)
                    issue(st ^ 1u, entry_next);
                }
                if (i + 2 < n_pages) entry_after = load_entry(page_begin + i + 2);
            }
            if (!entry_ok(entry_cur)) {
                if (lane == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
            } else {
                if (!mbar_wait(&bars[st], (phase_bits >> st) & 1u, p.wait_polls)) {
                    if (lane == 0) raise_status(p, CF_B200_DEVSTAT_WAIT_EXPIRED);
                    alive = false;
                    break;
                }
                phase_bits ^= 1u << st;
                const uint8_t *rec = warp_mem + st * kStageBytes;
                const uint4 hv = *reinterpret_cast<const uint4 *>(rec);
                const uint32_t k_bytes = 16u * (hv.x & 0xffffu), v_bytes = 16u * (hv.x >> 16);
                const uint32_t k_coder = hv.y & 0xffu, v_coder = (hv.y >> 8) & 0xffu, token_count = hv.y >> 16;
                const uint8_t *k_part = rec + 16;
                const uint8_t *v_part = k_part + k_bytes;
                bool offsets_ok;
                if constexpr (NB == 32) {
                    offsets_ok = part_offsets_ok(k_part, k_coder, k_bytes, lane) && part_offsets_ok(v_part, v_coder, v_bytes, lane);
                } else if constexpr (NB <= 16) {   // lanes 0..NB-1 hold the K blocks, lanes 16..16+NB-1 the V blocks
                    const bool mine = (lane & 15u) < static_cast<uint32_t>(NB);
                    offsets_ok = !mine || (lane < 16u ? part_offsets_ok<NB, kSyms>(k_part, k_coder, k_bytes, lane)
                                                      : part_offsets_ok<NB, kSyms>(v_part, v_coder, v_bytes, lane - 16u));
                } else {   // more blocks than lanes: block lane and block lane + 32 of the 2 NB (K blocks first)
                    offsets_ok = true;
#pragma unroll
                    for (uint32_t gb = lane; gb < 2u * NB; gb += 32u)
                        offsets_ok = offsets_ok && (gb < static_cast<uint32_t>(NB) ? part_offsets_ok<NB, kSyms>(k_part, k_coder, k_bytes, gb)
                                                                                 : part_offsets_ok<NB, kSyms>(v_part, v_coder, v_bytes, gb - NB));
                }
                const bool good = record_header_ok(hv, entry_cur, p.codebook_id) && __all_sync(0xffffffffu, offsets_ok);
                uint32_t dump_page = 0u;
                if constexpr (kMode == kDump) dump_page = table_row[page_begin + i];
                if (!good || dump_page >= p.dump_pages) {   // dump_pages is 1 outside the dump mode
                    if (lane == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
                } else {
                    if constexpr (kMode == kDump)   // [page id][kv head][K stream | V stream], one byte per symbol
                        u.dump = reinterpret_cast<uint32_t *>(p.output) +
                                 (static_cast<uint64_t>(dump_page) * p.kv_head_count + kv_head) * (kSyms / 2) + kQ * lane;
                    const float k_scale = __half2float(__ushort_as_half(static_cast<unsigned short>(hv.z & 0xffffu))) *
                                          (p.softmax_scale * kLog2e);
                    const float v_scale = __half2float(__ushort_as_half(static_cast<unsigned short>(hv.z >> 16)));
#pragma unroll
                    for (int n = 0; n < NG; ++n) u.score[n][0] = u.score[n][1] = u.score[n][2] = u.score[n][3] = 0.0f;

                    if constexpr (NB != 32) {
                        uint8_t *tile = warp_mem + L::kTile;
                        // One call site for both streams: the lanes that decode V blocks differ from those that decode K
                        // blocks only in the pointers they pass, so the warp runs the decoder once, not once per stream.
                        auto stage_one = [&](bool is_v, uint32_t block) {
                            stage_blocks<NB, kDim>(is_v ? v_part : k_part, is_v ? v_bytes : k_bytes, is_v ? v_coder : k_coder, block,
                                                   is_v ? v_slot : k_slot, is_v ? v_lut : k_lut,
                                                   tile + (is_v ? kTileStreamOf<kDim> + 16u : 0u));
                        };
                        if constexpr (NB <= 16) {
                            if ((lane & 15u) < static_cast<uint32_t>(NB)) stage_one(lane >= 16u, lane & 15u);
                        } else {   // two rounds: 2 NB blocks dealt over the 32 lanes, K blocks first
                            for (uint32_t gb = lane; gb < 2u * NB; gb += 32u)
                                stage_one(gb >= static_cast<uint32_t>(NB), gb >= static_cast<uint32_t>(NB) ? gb - NB : gb);
                        }
                        __syncwarp();
                        if (i + 1 < n_pages) issue(0u, entry_next);   // the record is decoded: its stage takes the next one
                        next_issued = true;
#pragma unroll
                        for (int c = 0; c < kQ / 4; ++c) {
                            const uint4 kk = *reinterpret_cast<const uint4 *>(tile + lane * kTileRowOf<kDim> + 16u * c);
                            const uint4 vv = *reinterpret_cast<const uint4 *>(tile + kTileStreamOf<kDim> + 16u + lane * kTileRowOf<kDim> + 16u * c);
                            const uint32_t kq[4] = {kk.x, kk.y, kk.z, kk.w}, vq[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                const int q = 4 * c + j;
                                if constexpr (kMode == kFold) {
                                    u.vq[0] ^= kq[j] ^ vq[j];
                                } else if constexpr (kMode == kDump) {
                                    u.dump[q] = kq[j];
                                    u.dump[kSyms / 4 + q] = vq[j];
                                } else {
                                    u.vq[q] = vq[j];
                                    score_quad(u, qs, q, kq[j]);
                                }
                            }
                        }
                        if constexpr (kProbe) __syncwarp();   // the tile is rewritten for the next page
                    } else if (k_coder == CF_B200_CODER_RANS_SPLIT4 && v_coder == CF_B200_CODER_RANS_SPLIT4) {
                        RansSplitLane k, v;
                        k.open(k_part, k_bytes, lane, k_slot);
                        v.open(v_part, v_bytes, lane, v_slot);
                        decode_fused_split<kMode>(k, v, u, qs);
                    } else if (k_coder == CF_B200_CODER_HUFFMAN_SPLIT4 && v_coder == CF_B200_CODER_HUFFMAN_SPLIT4) {
                        HuffSplitLane k, v;
                        k.open(k_part, k_bytes, lane, k_lut);
                        v.open(v_part, v_bytes, lane, v_lut);
                        decode_fused_split<kMode>(k, v, u, qs);
                    } else if (k_coder == CF_B200_CODER_RANS && v_coder == CF_B200_CODER_RANS) {
                        RansLane k, v;
                        k.open(k_part, k_bytes, lane, k_slot);
                        v.open(v_part, v_bytes, lane, v_slot);
                        decode_fused<kMode>(k, v, u, qs);
                    } else if (k_coder == CF_B200_CODER_HUFFMAN && v_coder == CF_B200_CODER_HUFFMAN) {
                        HuffLane k, v;
                        k.open(k_part, k_bytes, lane, k_lut);
                        v.open(v_part, v_bytes, lane, v_lut);
                        decode_fused<kMode>(k, v, u, qs);
                    } else if (k_coder == CF_B200_CODER_FIXED8 && v_coder == CF_B200_CODER_FIXED8) {
                        FixedLane k, v;
                        k.open(k_part, k_bytes, lane);
                        v.open(v_part, v_bytes, lane);
                        decode_fused<kMode>(k, v, u, qs);
                    } else {  // mixed coders (one stream fell back to fixed width): one stream after the other
                        if (k_coder == CF_B200_CODER_RANS) { RansLane k; k.open(k_part, k_bytes, lane, k_slot); decode_k_only<kMode>(k, u, qs); }
                        else if (k_coder == CF_B200_CODER_HUFFMAN) { HuffLane k; k.open(k_part, k_bytes, lane, k_lut); decode_k_only<kMode>(k, u, qs); }
                        else if (k_coder == CF_B200_CODER_RANS_SPLIT4) { RansSplitLane k; k.open(k_part, k_bytes, lane, k_slot); decode_k_only<kMode>(k, u, qs); }
                        else if (k_coder == CF_B200_CODER_HUFFMAN_SPLIT4) { HuffSplitLane k; k.open(k_part, k_bytes, lane, k_lut); decode_k_only<kMode>(k, u, qs); }
                        else { FixedLane k; k.open(k_part, k_bytes, lane); decode_k_only<kMode>(k, u, qs); }
                        if (v_coder == CF_B200_CODER_RANS) { RansLane v; v.open(v_part, v_bytes, lane, v_slot); decode_v_only<kMode>(v, u); }
                        else if (v_coder == CF_B200_CODER_HUFFMAN) { HuffLane v; v.open(v_part, v_bytes, lane, v_lut); decode_v_only<kMode>(v, u); }
                        else if (v_coder == CF_B200_CODER_RANS_SPLIT4) { RansSplitLane v; v.open(v_part, v_bytes, lane, v_slot); decode_v_only<kMode>(v, u); }
                        else if (v_coder == CF_B200_CODER_HUFFMAN_SPLIT4) { HuffSplitLane v; v.open(v_part, v_bytes, lane, v_lut); decode_v_only<kMode>(v, u); }
                        else { FixedLane v; v.open(v_part, v_bytes, lane); decode_v_only<kMode>(v, u); }
                    }

                    if constexpr (kSplitQ) {   // K q = K binary16(q) + K residue
#pragma unroll
                        for (int c = 0; c < 4; ++c) u.score[0][c] += u.score[1][c];
                    }
                    if constexpr (!kProbe) {
                    // ---- online softmax for this page (fp32), per group of four heads ----
                    const uint32_t token = (page_begin + i) * 16u + my_token;
                    const bool visible = my_token < token_count && token >= first_token && token < sealed && token <= qpos;
                    __syncwarp();  // the previous page's readers of the scratch are done
#pragma unroll
                    for (int n = 0; n < NS; ++n) {
                        const float s0 = visible ? u.score[n][0] * k_scale : -CUDART_INF_F;
                        const float s1 = visible ? u.score[n][1] * k_scale : -CUDART_INF_F;
                        float r0 = s0, r1 = s1;
#pragma unroll
                        for (int o = 2; o <= 16; o <<= 1) {  // lanes that hold the same two heads
                            r0 = fmaxf(r0, __shfl_xor_sync(0xffffffffu, r0, o));
                            r1 = fmaxf(r1, __shfl_xor_sync(0xffffffffu, r1, o));
                        }
                        const float n0 = fmaxf(u.m0[n], r0), n1 = fmaxf(u.m1[n], r1);
                        const float z0 = n0 == -CUDART_INF_F ? 0.0f : n0, z1 = n1 == -CUDART_INF_F ? 0.0f : n1;
                        const float p0 = exp2f(s0 - z0), p1 = exp2f(s1 - z1);
                        const float a0 = exp2f(u.m0[n] - z0), a1 = exp2f(u.m1[n] - z1);
                        u.l0[n] = u.l0[n] * a0 + p0;
                        u.l1[n] = u.l1[n] * a1 + p1;
                        u.m0[n] = n0;
                        u.m1[n] = n1;
                        // P goes to the tensor cores as fp16; the rounding residue is fed as a second operand so that
                        // P V is accurate to fp32 level whatever the magnitude of V
                        // The weights (at most 1) are scaled by 2^15 on the way, O by 2^-15 at the unit's end, both exact:
                        // binary16 then resolves weights down to 2^-40 of the row maximum instead of 2^-25.
                        const uint32_t h0 = 4u * n + my_head0;
                        const float w0 = p0 * kWeightScale, w1 = p1 * kWeightScale;
                        const __half p0h = __float2half_rn(w0), p1h = __float2half_rn(w1);
                        p_rows[h0 * 16u + my_token] = p0h;
                        p_rows[(h0 + 1u) * 16u + my_token] = p1h;
                        p_rows_lo[h0 * 16u + my_token] = __float2half_rn(w0 - __half2float(p0h));
                        p_rows_lo[(h0 + 1u) * 16u + my_token] = __float2half_rn(w1 - __half2float(p1h));
                        if (g == 0 && t < 2) {
                            alpha_s[h0] = a0;
                            alpha_s[h0 + 1u] = a1;
                        }
                    }
                    __syncwarp();
                    const float v_ratio = v_scale_prev / v_scale;   // O is kept in units of the current page's V scale
                    v_scale_prev = v_scale;
#pragma unroll
                    for (int n = 0; n < NS; ++n) {
                        const float beta = alpha_s[4u * n + o_head] * v_ratio;
#pragma unroll
                        for (int dd = 0; dd < kVCh; ++dd)
#pragma unroll
                            for (int c = 0; c < 4; ++c) u.acc[n][dd][c] *= beta;
                    }
                    // P rows as A fragments. Rows g / g+8 of the fragment belong to lane tags g>>2 / (g>>2)+2; a lane
                    // feeds the row whose tag is its own t and zeros (read from the zero row) otherwise.
                    uint32_t ra[2][NS][8], rb[2][NS][8];   // [fp16(p) | its rounding residue][group][fragment words]
#pragma unroll
                    for (int part = 0; part < 2; ++part) {
#pragma unroll
                        for (int n = 0; n < NS; ++n) {
                            const __half *rows = (part ? p_rows_lo : p_rows) + (4u * n + o_head) * 16u;
                            const __half *row_a = row_lo_mine ? rows : zero_row;
                            const __half *row_b = row_hi_mine ? rows : zero_row;
                            const uint4 a_lo = *reinterpret_cast<const uint4 *>(row_a);
                            const uint4 a_hi = *reinterpret_cast<const uint4 *>(row_a + 8);
                            const uint4 b_lo = *reinterpret_cast<const uint4 *>(row_b);
                            const uint4 b_hi = *reinterpret_cast<const uint4 *>(row_b + 8);
                            ra[part][n][0] = a_lo.x; ra[part][n][1] = a_lo.y; ra[part][n][2] = a_lo.z; ra[part][n][3] = a_lo.w;
                            ra[part][n][4] = a_hi.x; ra[part][n][5] = a_hi.y; ra[part][n][6] = a_hi.z; ra[part][n][7] = a_hi.w;
                            rb[part][n][0] = b_lo.x; rb[part][n][1] = b_lo.y; rb[part][n][2] = b_lo.z; rb[part][n][3] = b_lo.w;
                            rb[part][n][4] = b_hi.x; rb[part][n][5] = b_hi.y; rb[part][n][6] = b_hi.z; rb[part][n][7] = b_hi.w;
                        }
                    }
#pragma unroll
                    for (int tq = 0; tq < 4; ++tq) {   // token quads outside: consecutive mma feed different accumulators
#pragma unroll
                        for (int dd = 0; dd < kVCh; ++dd) {
                            uint32_t lo, hi;
                            quad_to_half2(u.vq[dd * 4 + tq], lo, hi);   // converted once, used by both parts
#pragma unroll
                            for (int part = 0; part < 2; ++part)
#pragma unroll
                                for (int n = 0; n < NS; ++n)
                                    mma_16816(u.acc[n][dd], ra[part][n][2 * tq], rb[part][n][2 * tq], ra[part][n][2 * tq + 1],
                                              rb[part][n][2 * tq + 1], lo, hi);
                        }
                    }
                    }   // !kProbe
                }
            }
            if (!next_issued && i + 1 < n_pages) {   // single stage, page skipped: nobody reads the stage any more
                __syncwarp();
                issue(0u, entry_next);
            }
            entry_cur = entry_next;
            entry_next = entry_after;
        }
        if (!alive) {
            // give the copies still in flight a bounded chance to land before this warp's buffers go away
            mbar_wait(&bars[0], phase_bits & 1u, p.wait_polls);
            if constexpr (L::kStages == 2) mbar_wait(&bars[1], (phase_bits >> 1) & 1u, p.wait_polls);
            return;
        }

        if constexpr (kMode == kDump) {
        } else if constexpr (kMode == kFold) {   // the checksum of everything the unit decoded, so that the work cannot be dropped
            uint32_t x = u.vq[0];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) x ^= __shfl_xor_sync(0xffffffffu, x, o);
            if (lane == 0) partial_ptr(p, chunk, out_head_base)[0] = __uint_as_float(x);
        } else {
        // ---- unit partials ----
#pragma unroll
        for (int n = 0; n < NS; ++n) {
            float l0 = u.l0[n], l1 = u.l1[n];
#pragma unroll
            for (int o = 2; o <= 16; o <<= 1) {
                l0 += __shfl_xor_sync(0xffffffffu, l0, o);
                l1 += __shfl_xor_sync(0xffffffffu, l1, o);
            }
            const uint32_t h0 = 4u * n + my_head0;
            if (g == 0 && t < 2) {
                if (h0 < G) {
                    float *dst = partial_ptr(p, chunk, out_head_base + h0);
                    dst[0] = u.m0[n];
                    dst[1] = l0;
                }
                if (h0 + 1u < G) {
                    float *dst = partial_ptr(p, chunk, out_head_base + h0 + 1u);
                    dst[0] = u.m1[n];
                    dst[1] = l1;
                }
            }
            if (4u * n + o_head < G) {
                float *dst = partial_ptr(p, chunk, out_head_base + 4u * n + o_head) + 2;
#pragma unroll
                for (int dd = 0; dd < kVCh; ++dd) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const uint32_t owner = 4u * (2u * t + (c & 1)) + (g >> 2) + 2u * (c >> 1);  // lane whose V block it is
                        dst[kVCh * owner + dd] = u.acc[n][dd][c] * (v_scale_prev * (1.0f / kWeightScale));
                    }
                }
            }
        }
        }   // !kProbe
        __syncwarp();
    }
}

}  // namespace

bool lanes_kernel_supports(const AttentionParams &p) {
    const bool geometry = p.page_tokens == 16 &&
                          ((p.head_dim == 128 && (p.block_size == 64 || p.block_size == 128 || p.block_size == 256)) ||
                           ((p.head_dim == 96 || p.head_dim == 64) && (p.block_size == 64 || p.block_size == 128)) ||
                           (p.head_dim == 32 && p.block_size == 64));
    return geometry && p.group >= 1 && p.group <= 16 &&
           (p.query_type == CF_B200_F16 || p.query_type == CF_B200_F32);
}

// Query groups of up to four heads per kv head run the four-head kernel; larger groups run the eight-head one, which
// decodes a page once for eight query heads (its query operands live in shared memory instead of registers). fp32
// queries (the reference's own ABIs pass nothing else) run the split-query kernel, four heads per pass.
namespace {

template <int NG, int kMode, bool kSplitQ, int NB, int kDim>
cudaError_t launch_one(const AttentionParams &p, int sm_count, cudaStream_t stream) {
    static std::atomic<uint64_t> configured{0};   // bit = device ordinal
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return e;
    const uint64_t bit = 1ull << (device & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        e = cudaFuncSetAttribute(lanes_attention_kernel<NG, kMode, kSplitQ, NB, kDim>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 static_cast<int>(WarpLayout<NG, NB>::kSmem));
        if (e != cudaSuccess) return e;
        configured.fetch_or(bit, std::memory_order_release);
    }
    lanes_attention_kernel<NG, kMode, kSplitQ, NB, kDim><<<sm_count, kThreadsOf<NG, NB>, WarpLayout<NG, NB>::kSmem, stream>>>(p);
    return cudaPeekAtLastError();
}

template <int NB, int kDim = 128>
cudaError_t launch_for_blocks(const AttentionParams &p, int sm_count, cudaStream_t stream) {
    if (p.decode_probe == 2u) return launch_one<1, kDump, false, NB, kDim>(p, sm_count, stream);
    if (p.decode_probe) return launch_one<1, kFold, false, NB, kDim>(p, sm_count, stream);
    if (p.query_type == CF_B200_F32) return launch_one<2, kAttend, true, NB, kDim>(p, sm_count, stream);
    if (p.group <= 4) return launch_one<1, kAttend, false, NB, kDim>(p, sm_count, stream);
    return launch_one<2, kAttend, false, NB, kDim>(p, sm_count, stream);
}

}  // namespace

cudaError_t launch_lanes_attention(const AttentionParams &p, cudaStream_t stream) {
    static LauncherState table[64];
    cudaError_t e;
    LauncherState *state = launcher_state(table, &e);
    if (!state) return e;
    if (p.head_dim == 64) {   // 16 x 64 pages: 16 (or 8) blocks per stream, always staged
        return p.block_size == 64 ? launch_for_blocks<16, 64>(p, state->sm_count, stream)
                                  : launch_for_blocks<8, 64>(p, state->sm_count, stream);
    }
    if (p.head_dim == 96) {
        return p.block_size == 64 ? launch_for_blocks<24, 96>(p, state->sm_count, stream)
                                  : launch_for_blocks<12, 96>(p, state->sm_count, stream);
    }
    if (p.head_dim == 32) return launch_for_blocks<8, 32>(p, state->sm_count, stream);
    if (p.block_size == 128) return launch_for_blocks<16>(p, state->sm_count, stream);
    if (p.block_size == 256) return launch_for_blocks<8>(p, state->sm_count, stream);
    return launch_for_blocks<32>(p, state->sm_count, stream);
}

}  // namespace cfb
