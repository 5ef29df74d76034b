// sealed_attention_prefix.cu — attention over a SHARED sealed prefix: pages that every sequence of the batch
// references (one copy in the arena, the same page ids at the head of every page-table row; the reference's
// shared-page semantics, src/multisequence_cache.cpp:235-292), on the 5th-generation tensor cores (tcgen05.mma with
// accumulators and the A operands in tensor memory). Geometry: head_dim 128, page_tokens 16, block 64.
//
// The per-sequence kernel would decode such a page once per sequence. Here a page is decoded once per tile of 128
// query rows (rows = sequence x query head of the kv head's group) and contracted with all those rows at once.
//
// One CTA of 20 warps per SM. The work is cut evenly (SharedSplit): the rounds (8 pages = 128 tokens) of every
// (kv head, row tile) pair form one line and each CTA takes an equal stretch of it; the part of a stretch inside one
// pair is a unit, which ends in one partial per row. The warps are specialised:
//   decoder warps 0..11  the page slots of the CTA's units form one sequence; warp w takes slots w, w + 12, ... It
//                        receives the record by one bulk async copy (mbarrier, bounded wait), decodes it with the
//                        lane-per-block decoders INTO REGISTERS (32 packed quads per lane), starts the copy of its next
//                        record, and only then waits for the tile pair of the slot's round to be free; the symbols
//                        are written as exact binary16 codes into one of TWO tile pairs in shared memory: K tile
//                        [token][channel] (B of S = Q K^T), V tile [channel][token] (B of O = P V); then the warp
//                        arrives on the pair's "full" barrier (8 arrivals = one round). A pair is free when the tensor
//                        core's commit for the round that read it has arrived on its "free" barrier. Twelve warps keep
//                        decoding while the other group works on the previous round.
//   softmax warps 12..19 a thread owns one row (= tensor-memory lane, in its warp's quarter) and half of the round's
//                        128 score columns. Thread 0 of the group issues the tensor-core work:
//                          S     8 tcgen05.mma (M 128, N 128, K 16): Q from tensor memory x K tile -> columns 0..127
//                          O    16 tcgen05.mma: P (binary16, then its rounding residue) from tensor memory x V tile
//                                -> columns 128..255, then commits to the "O" barrier and the pair's "free" barrier
//                        All threads: one tcgen05.ld of their 64 scores (kept in registers), page K scales and masks,
//                        the row's two threads share their maxima through shared memory, running max / sum updated,
//                        O rescaled in tensor memory (tcgen05.ld / .st) only when some row of the warp moved its max,
//                        P and its residue written to tensor memory (tcgen05.st) as the next A operands.
//                        Unit start: the Q rows go from global memory straight to tensor memory. Unit end: O read back,
//                        scaled, written with (max, sum) to the shared-prefix partials; the combine kernel merges
//                        them with the per-sequence partials of the private pages and the tail.
// Registers: the kernel starts at 96 per thread; the decoders drop to 80 and the softmax warps rise to 120 (setmaxnreg).
// Tensor memory (512 columns): S 0..127, O 128..255, Q 256..319, P 320..383, P residue 384..447, Q residue 448..511 (fp32
// queries only: the row is split into binary16(q) and its rounding residue, S = Q K^T + Q residue K^T) (binary16 pairs per
// column, row = lane). B tiles use the no-swizzle K-major canonical layout: 8 rows x 16 bytes core matrices, element
// (row r, 16-byte chunk c) at (r % 8) * 16 + (r / 8) * 2048 + c * 128 bytes.
// The page's V scale relative to the largest one met so far in the unit rides on P (never above 1, so the binary16
// weights cannot overflow); O is kept in units of that scale and rescaled when a larger one arrives.
// Every mbarrier wait is bounded. A warp whose wait ran out raises CF_B200_DEVSTAT_WAIT_EXPIRED and skips all later
// waits and work; a decoder warp still arrives for each of its slots, a softmax warp still takes part in its group's
// barriers, which OR-reduce the failure so that the whole group leaves its loop at the same point; the CTA then frees
// its tensor memory.

#include "lanes_decoders.cuh"

namespace cfb {
namespace {

using namespace lanes;

constexpr int kDecodeWarps = 12;     // warps 0..11 (three warpgroups)
constexpr int kSoftmaxWarps = 8;     // warps 12..19 (two warpgroups)
constexpr int kRoundPages = 8;
constexpr int kGroupThreads = kSoftmaxWarps * 32;
constexpr int kTcThreads = (kDecodeWarps + kSoftmaxWarps) * 32;
constexpr uint32_t kTileBytes = 128 * 128 * 2;   // one operand tile: 128 rows x 128 binary16
constexpr uint32_t kOffStages = kTableBytes;
constexpr uint32_t kOffTiles = (kOffStages + kDecodeWarps * kStageBytes + 127u) / 128u * 128u;   // K[0] V[0] K[1] V[1]
constexpr uint32_t kOffMeta = kOffTiles + 4 * kTileBytes;      // [pair][page of the round]: k scale, v scale, token count, -
constexpr uint32_t kOffRound = kOffMeta + 2 * kRoundPages * 16;    // [pair]: unit, flags, -, -
constexpr uint32_t kOffBars = kOffRound + 2 * 16;              // 12 copy barriers, full[2], free[2], S, O
constexpr uint32_t kBarFull = kDecodeWarps, kBarFree = kBarFull + 2, kBarS = kBarFree + 2, kBarO = kBarS + 1, kBarCount = kBarO + 1;
constexpr uint32_t kOffMisc = kOffBars + kBarCount * 8;        // [0] tmem base
constexpr uint32_t kOffRowMax = kOffMisc + 32;                 // [2 column halves][128 rows]
constexpr uint32_t kTcSmem = kOffRowMax + 2 * 128 * 4;
static_assert(kTcSmem <= 232448, "the shared-prefix kernel must fit the 227 KB of one CTA");
constexpr uint32_t kTmemColumns = 512;
constexpr uint32_t kColS = 0, kColO = 128, kColQ = 256, kColP = 320, kColPResidue = 384, kColQResidue = 448;
constexpr uint32_t kStopUnit = 0xffffffffu;
constexpr float kWeightScale = 32768.0f;   // power of two the binary16 weights are scaled by (O sheds it at a unit's end)
constexpr uint32_t kFirstRound = 1u, kLastRound = 2u;   // round flags
constexpr uint32_t kSoftmaxBarrier = 1;   // named barrier (0 is __syncthreads)
// Register split (setmaxnreg). A CTA can only redistribute the registers it was launched with: kLaunchRegs per thread,
// the most that 640 threads can have. What the softmax warps ask for must not exceed what the decoders give back, or
// the request would wait forever; the launch function checks kLaunchRegs against the compiled kernel.
constexpr int kLaunchRegs = 96, kDecoderRegs = 80, kSoftmaxRegs = 120;
static_assert(kLaunchRegs * kTcThreads <= 65536 && kDecoderRegs % 8 == 0 && kSoftmaxRegs % 8 == 0 &&
                  kDecodeWarps * 32 * kDecoderRegs + kSoftmaxWarps * 32 * kSoftmaxRegs <= kLaunchRegs * kTcThreads,
              "the register split must fit the CTA's own registers");
// instruction descriptor: f32 accumulate, f16 x f16, both operands K-major, N = 128, M = 128
constexpr uint32_t kIdesc = (1u << 4) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ uint32_t tile_offset(uint32_t row, uint32_t chunk) {
    return (row & 7u) * 16u + (row >> 3) * 2048u + chunk * 128u;
}
// Row of the V tile (= column of O) that holds channel 4 * lane + c, the c-th channel of the block lane decodes: the 32
// lanes of one store spread over all 8 rows of a core matrix, so a 16-byte store per lane meets no bank conflict.
// Inverse: column n of O is channel 4 * ((n & 7) + 8 * (n >> 5)) + ((n >> 3) & 3).
__device__ __forceinline__ uint32_t v_tile_row(uint32_t lane, uint32_t c) {
    return (lane & 7u) + 8u * c + 32u * (lane >> 3);
}
// shared-memory matrix descriptor: start address, leading (K) offset 128 B, stride (row group) offset 2048 B, version 1
__device__ __forceinline__ uint64_t tile_desc(uint32_t smem_address) {
    return static_cast<uint64_t>((smem_address >> 4) & 0x3fffu) | (static_cast<uint64_t>(128u >> 4) << 16) |
           (static_cast<uint64_t>(2048u >> 4) << 32) | (1ull << 46);
}
// D[tmem_d] (+)= A[tmem_a: 128 lanes x 8 columns of binary16 pairs] x B[shared-memory tile]^T, one K step of 16
__device__ __forceinline__ void umma(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(tmem_d),
        "r"(tmem_a), "l"(desc_b), "r"(kIdesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
// Barrier over one group (whole warps) that also ORs a predicate: every thread of the group gets the same answer.
__device__ __forceinline__ bool group_any(uint32_t barrier_id, bool pred) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.b32 p, %1, 0;\n\t"
        "bar.red.or.pred q, %2, %3, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(static_cast<uint32_t>(pred)), "r"(barrier_id), "r"(static_cast<uint32_t>(kGroupThreads))
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_store32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]), "r"(v[10]),
        "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]),
        "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]),
        "r"(v[31])
        : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Two quads of symbols (8 codes) -> one 16-byte chunk of binary16 codes, exact.
__device__ __forceinline__ uint4 codes8(uint32_t qa, uint32_t qb) {
    uint4 r;
    quad_to_half2(qa, r.x, r.y);
    quad_to_half2(qb, r.z, r.w);
    return r;
}

// Decode one record into registers: quad q of a stream = symbols 4q..4q+3 of the block this lane decodes.
template <class KLane, class VLane>
__device__ __forceinline__ void decode_page(KLane &k, VLane &v, uint32_t (&kq)[16], uint32_t (&vq)[16]) {
    // Four passes of four quads per stream. The pass is a real loop (its body is a quarter of the unrolled code, which
    // the instruction cache shares with the softmax warps' code); the results shift down the register arrays, so that
    // after the fourth pass quad q sits in element q.
#pragma unroll 1
    for (int pass = 0; pass < 4; ++pass) {
#pragma unroll
        for (int i = 0; i < 12; ++i) {
            kq[i] = kq[i + 4];
            vq[i] = vq[i + 4];
        }
#pragma unroll
        for (int q = 12; q < 16; ++q) {
            if constexpr (KLane::kWholeQuads || VLane::kWholeQuads) {   // fixed width or nibble-split: a quad per call
                kq[q] = k.quad(4 * pass + (q - 12));
                vq[q] = v.quad(4 * pass + (q - 12));
            } else {   // both entropy coded: the two chains interleave symbol by symbol
                k.reload();
                v.reload();
                uint32_t ke[4], ve[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    ke[i] = k.symbol();
                    ve[i] = v.symbol();
                }
                kq[q] = pack_low_bytes(ke[0], ke[1], ke[2], ke[3]);
                vq[q] = pack_low_bytes(ve[0], ve[1], ve[2], ve[3]);
            }
        }
    }
}
template <class Lane>
__device__ __forceinline__ void decode_stream(Lane &s, uint32_t (&quads)[16]) {
#pragma unroll
    for (int q = 0; q < 16; ++q) quads[q] = s.quad(q);
}
// The decoded page goes into slot `slot` of the round's tiles as exact binary16 codes. K quad q of lane l = token l/2,
// channels 64(l&1)+4q..+3 -> K tile row 16*slot + l/2; V quad q of lane l = channel 4l + q/4, tokens 4(q%4)..+3 -> V tile
// row v_tile_row(l, q/4), token chunks 2*slot and 2*slot+1.
__device__ __forceinline__ void store_tiles(const uint32_t (&kq)[16], const uint32_t (&vq)[16], uint8_t *k_tile, uint8_t *v_tile,
                                            uint32_t slot, uint32_t lane) {
    const uint32_t k_row = 16u * slot + (lane >> 1);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const uint32_t k_chunk = 8u * (lane & 1u) + 2u * c;
        *reinterpret_cast<uint4 *>(k_tile + tile_offset(k_row, k_chunk)) = codes8(kq[4 * c], kq[4 * c + 1]);
        *reinterpret_cast<uint4 *>(k_tile + tile_offset(k_row, k_chunk + 1u)) = codes8(kq[4 * c + 2], kq[4 * c + 3]);
        const uint32_t v_row = v_tile_row(lane, c);
        *reinterpret_cast<uint4 *>(v_tile + tile_offset(v_row, 2u * slot)) = codes8(vq[4 * c], vq[4 * c + 1]);
        *reinterpret_cast<uint4 *>(v_tile + tile_offset(v_row, 2u * slot + 1u)) = codes8(vq[4 * c + 2], vq[4 * c + 3]);
    }
}
// A page that is absent (past the chunk's end, or refused) leaves zeros in its slot of both tiles.
__device__ __forceinline__ void zero_slot(uint8_t *k_tile, uint8_t *v_tile, uint32_t slot, uint32_t lane) {
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    const uint32_t k_row = 16u * slot + (lane >> 1);
#pragma unroll
    for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4 *>(k_tile + tile_offset(k_row, 8u * (lane & 1u) + c)) = z;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        *reinterpret_cast<uint4 *>(v_tile + tile_offset(v_tile_row(lane, c), 2u * slot)) = z;
        *reinterpret_cast<uint4 *>(v_tile + tile_offset(v_tile_row(lane, c), 2u * slot + 1u)) = z;
    }
}

__device__ __forceinline__ void tmem_store8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(v[0]),
                 "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
// 2^x by the special-function unit (inputs below -126 give 0, -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void tmem_store_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// What both groups derive from a unit number: unit j of CTA b is the CTA's stretch of rounds inside the j-th head-tile it
// meets (SharedSplit). `valid` is false past the CTA's last unit.
struct UnitShape {
    uint32_t tile_index, head_local, chunk, kv_head, page_begin, page_end, valid;
};
__device__ __forceinline__ UnitShape unit_shape(const AttentionParams &p, const SharedSplit &split, uint32_t cta, uint32_t unit,
                                                uint32_t row_tiles, uint32_t shared_pages) {
    UnitShape u = {};
    const uint64_t lo = split.first_round(cta), hi = split.first_round(cta + 1u);
    const uint64_t head_tile = lo / split.rounds + unit, base = head_tile * split.rounds;
    u.valid = lo < hi && base < hi;
    if (!u.valid) return u;
    const uint32_t r0 = static_cast<uint32_t>((lo > base ? lo : base) - base);
    const uint32_t r1 = static_cast<uint32_t>((hi < base + split.rounds ? hi : base + split.rounds) - base);
    u.tile_index = static_cast<uint32_t>(head_tile % row_tiles);
    u.head_local = static_cast<uint32_t>(head_tile / row_tiles);
    u.chunk = cta - split.cta_of(base);
    u.kv_head = p.kv_head_begin + u.head_local;
    u.page_begin = 8u * r0;
    u.page_end = min(8u * r1, shared_pages);
    return u;
}

// ---- decoder group: warps 0..11 -----------------------------------------------------------------------------------
// The page slots of the CTA's units (pages of a unit padded to whole rounds of eight) form one sequence; decoder warp w takes slots w, w + 12, w + 24, ... A slot is decoded into registers first;
// only then does the warp wait for the tile pair of the slot's round, so that decoding never waits for the tensor core.
struct SlotCursor {
    uint32_t unit, valid, first_slot, first_round, slots;   // of the unit that holds the slot
    UnitShape u;
};

__device__ __forceinline__ void decoder_role(const AttentionParams &p, uint8_t *smem, PlanHeader *hdr, uint32_t warp, uint32_t lane,
                                             uint32_t row_tiles, const SharedSplit &split) {
    const uint32_t *k_slot = reinterpret_cast<const uint32_t *>(smem);
    const uint32_t *v_slot = k_slot + 4096;
    const uint16_t *k_lut = reinterpret_cast<const uint16_t *>(v_slot + 4096);
    const uint16_t *v_lut = k_lut + 4096;
    uint8_t *stage = smem + kOffStages + warp * kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBars);
    uint64_t *bar = bars + warp, *bar_full = bars + kBarFull, *bar_free = bars + kBarFree;
    uint32_t *round_desc = reinterpret_cast<uint32_t *>(smem + kOffRound);
    const uint32_t shared_pages = hdr->shared_pages;
    const uint32_t *table_row = p.page_table + static_cast<uint64_t>(slot_of(p, 0)) * p.page_table_stride;

    auto load_unit = [&](SlotCursor &c) {
        c.u = unit_shape(p, split, blockIdx.x, c.unit, row_tiles, shared_pages);
        c.valid = c.u.valid;
        if (c.valid) c.slots = (c.u.page_end - c.u.page_begin + 7u) / 8u * 8u;
    };
    auto seek = [&](SlotCursor &c, uint32_t n) {   // the unit that holds slot n (n only grows)
        while (c.valid && n >= c.first_slot + c.slots) {
            c.first_slot += c.slots;
            c.first_round += c.slots / 8u;
            c.unit += 1u;
            load_unit(c);
        }
    };
    // directory entry of slot n, 0 if the slot is padding or past the CTA's last unit
    auto slot_entry = [&](const SlotCursor &c, uint32_t n) -> uint64_t {
        if (!c.valid) return 0ull;
        const uint32_t page = c.u.page_begin + (n - c.first_slot);
        if (page >= c.u.page_end) return 0ull;
        const uint32_t page_id = table_row[page];   // bit 63 marks the page of the wait-expiry test: armed, never fetched
        const uint64_t e = p.page_dir[static_cast<uint64_t>(page_id) * p.kv_head_count + c.u.kv_head];
        return page_id == p.skip_copy_page ? e | (1ull << 63) : e;
    };
    auto entry_ok = [&](uint64_t entry) {
        const uint32_t units16 = static_cast<uint32_t>(CF_B200_DIR_LENGTH_UNITS(entry));
        return units16 != 0 && units16 * 16u <= kStageBytes - 32u;
    };
    auto issue = [&](uint64_t entry) {
        if (lane == 0 && entry_ok(entry)) {
            const uint32_t bytes = static_cast<uint32_t>(CF_B200_DIR_LENGTH_UNITS(entry)) * 16u;
            mbar_expect_tx(bar, bytes);
            if (!(entry >> 63)) bulk_load(stage, p.arena + 16ull * CF_B200_DIR_OFFSET_UNITS(entry), bytes, bar);
        }
    };
    uint32_t copy_phase = 0;
    bool failed = false;   // warp-uniform; once set, the warp waits for nothing and decodes nothing, but keeps arriving
    // The pair of round `it` is free once the tensor core has finished round it - 2. The parity wait is sound because a
    // warp's slots are 12 apart, less than two rounds: it has always seen the completion before the one it waits for.
    auto wait_pair_free = [&](uint32_t it) {
        if (it >= 2u && !failed && !__all_sync(0xffffffffu, mbar_wait(&bar_free[it & 1u], ((it >> 1) - 1u) & 1u, p.wait_polls))) {
            failed = true;
            if (lane == 0) raise_status(p, CF_B200_DEVSTAT_WAIT_EXPIRED);
        }
    };

    SlotCursor cur;
    cur.unit = 0;
    cur.first_slot = 0;
    cur.first_round = 0;
    cur.slots = 0;
    load_unit(cur);
    uint32_t n = warp;
    seek(cur, n);
    uint64_t entry = slot_entry(cur, n);
    issue(entry);

    for (;; n += kDecodeWarps) {
        if (!cur.valid) {   // past the last unit: the eight slots after it make the round that tells the softmax group to stop
            if (n < cur.first_slot + 8u) {
                wait_pair_free(cur.first_round);
                if (lane == 0) {
                    if (n == cur.first_slot) round_desc[4 * (cur.first_round & 1u)] = kStopUnit;
                    mbar_arrive(&bar_full[cur.first_round & 1u]);
                }
            }
            break;
        }
        const uint32_t in_unit = n - cur.first_slot, slot = in_unit & 7u, it = cur.first_round + (in_unit >> 3), pair = it & 1u;
        // the warp's next slot: its directory entry is fetched now (dependent loads), needed only after this decode
        SlotCursor next = cur;
        seek(next, n + kDecodeWarps);
        const uint64_t next_entry = slot_entry(next, n + kDecodeWarps);

        float k_scale = 0.0f, v_scale = 0.0f;
        uint32_t token_count = 0;
        uint32_t kq[16] = {}, vq[16] = {};
        if (cur.u.page_begin + in_unit < cur.u.page_end && !failed) {
            if (!entry_ok(entry)) {
                if (lane == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
            } else if (!__all_sync(0xffffffffu, mbar_wait(bar, copy_phase & 1u, p.wait_polls))) {
                failed = true;
                if (lane == 0) raise_status(p, CF_B200_DEVSTAT_WAIT_EXPIRED);
            } else {
                copy_phase ^= 1u;
                const uint4 hv = *reinterpret_cast<const uint4 *>(stage);
                const uint32_t k_bytes = 16u * (hv.x & 0xffffu), v_bytes = 16u * (hv.x >> 16);
                const uint32_t k_coder = hv.y & 0xffu, v_coder = (hv.y >> 8) & 0xffu;
                const uint8_t *k_part = stage + 16, *v_part = k_part + k_bytes;
                if (!record_header_ok(hv, entry, p.codebook_id) ||
                    !__all_sync(0xffffffffu, part_offsets_ok(k_part, k_coder, k_bytes, lane) &&
                                                 part_offsets_ok(v_part, v_coder, v_bytes, lane))) {
                    if (lane == 0) raise_status(p, CF_B200_DEVSTAT_BAD_RECORD);
                } else {
                    token_count = hv.y >> 16;
                    k_scale = __half2float(__ushort_as_half(static_cast<unsigned short>(hv.z & 0xffffu))) * (p.softmax_scale * kLog2e);
                    v_scale = __half2float(__ushort_as_half(static_cast<unsigned short>(hv.z >> 16)));
                    if (k_coder == CF_B200_CODER_RANS && v_coder == CF_B200_CODER_RANS) {
                        RansLane k, v;
                        k.open(k_part, k_bytes, lane, k_slot);
                        v.open(v_part, v_bytes, lane, v_slot);
                        decode_page(k, v, kq, vq);
                    } else if (k_coder == CF_B200_CODER_HUFFMAN && v_coder == CF_B200_CODER_HUFFMAN) {
                        HuffLane k, v;
                        k.open(k_part, k_bytes, lane, k_lut);
                        v.open(v_part, v_bytes, lane, v_lut);
                        decode_page(k, v, kq, vq);
                    } else if (k_coder == CF_B200_CODER_FIXED8 && v_coder == CF_B200_CODER_FIXED8) {
                        FixedLane k, v;
                        k.open(k_part, k_bytes, lane);
                        v.open(v_part, v_bytes, lane);
                        decode_page(k, v, kq, vq);
                    } else if (k_coder == CF_B200_CODER_RANS_SPLIT4 && v_coder == CF_B200_CODER_RANS_SPLIT4) {
                        RansSplitLane k, v;
                        k.open(k_part, k_bytes, lane, k_slot);
                        v.open(v_part, v_bytes, lane, v_slot);
                        decode_page(k, v, kq, vq);
                    } else if (k_coder == CF_B200_CODER_HUFFMAN_SPLIT4 && v_coder == CF_B200_CODER_HUFFMAN_SPLIT4) {
                        HuffSplitLane k, v;
                        k.open(k_part, k_bytes, lane, k_lut);
                        v.open(v_part, v_bytes, lane, v_lut);
                        decode_page(k, v, kq, vq);
                    } else {
                        if (k_coder == CF_B200_CODER_RANS) { RansLane k; k.open(k_part, k_bytes, lane, k_slot); decode_stream(k, kq); }
                        else if (k_coder == CF_B200_CODER_HUFFMAN) { HuffLane k; k.open(k_part, k_bytes, lane, k_lut); decode_stream(k, kq); }
                        else if (k_coder == CF_B200_CODER_RANS_SPLIT4) { RansSplitLane k; k.open(k_part, k_bytes, lane, k_slot); decode_stream(k, kq); }
                        else if (k_coder == CF_B200_CODER_HUFFMAN_SPLIT4) { HuffSplitLane k; k.open(k_part, k_bytes, lane, k_lut); decode_stream(k, kq); }
                        else { FixedLane k; k.open(k_part, k_bytes, lane); decode_stream(k, kq); }
                        if (v_coder == CF_B200_CODER_RANS) { RansLane v; v.open(v_part, v_bytes, lane, v_slot); decode_stream(v, vq); }
                        else if (v_coder == CF_B200_CODER_HUFFMAN) { HuffLane v; v.open(v_part, v_bytes, lane, v_lut); decode_stream(v, vq); }
                        else if (v_coder == CF_B200_CODER_RANS_SPLIT4) { RansSplitLane v; v.open(v_part, v_bytes, lane, v_slot); decode_stream(v, vq); }
                        else if (v_coder == CF_B200_CODER_HUFFMAN_SPLIT4) { HuffSplitLane v; v.open(v_part, v_bytes, lane, v_lut); decode_stream(v, vq); }
                        else { FixedLane v; v.open(v_part, v_bytes, lane); decode_stream(v, vq); }
                    }
                    if (p.decode_probe == 2u) {   // test mode: the quads as decoded, [page id][kv head][K stream | V stream]
                        const uint32_t page_id = table_row[cur.u.page_begin + in_unit];
                        if (page_id < p.dump_pages) {
                            uint32_t *dump = reinterpret_cast<uint32_t *>(p.output) +
                                             (static_cast<uint64_t>(page_id) * p.kv_head_count + cur.u.kv_head) * 1024u + 16u * lane;
#pragma unroll
                            for (int q = 0; q < 16; ++q) {
                                dump[q] = kq[q];
                                dump[512 + q] = vq[q];
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();   // every lane is done with the stage: the next record may land in it
        if (!failed) issue(next_entry);

        wait_pair_free(it);
        uint8_t *k_tile = smem + kOffTiles + pair * 2u * kTileBytes, *v_tile = k_tile + kTileBytes;
        if (token_count != 0u) store_tiles(kq, vq, k_tile, v_tile, slot, lane);
        else zero_slot(k_tile, v_tile, slot, lane);
        if (lane == 0) {
            float *meta = reinterpret_cast<float *>(smem + kOffMeta) + pair * 32u + 4u * slot;
            meta[0] = k_scale;
            meta[1] = v_scale;
            meta[2] = __uint_as_float(token_count);   // 0: the page contributes nothing
            if (slot == 0) {
                round_desc[4 * pair] = cur.unit;
                round_desc[4 * pair + 1] = (in_unit < 8u ? kFirstRound : 0u) | (in_unit + 8u >= cur.slots ? kLastRound : 0u);
            }
        }
        fence_async_smem();   // the tiles were written through the generic proxy; the tensor core reads through the async one
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_full[pair]);
        cur = next;
        entry = next_entry;
    }
    // a copy whose wait ran out gets one more bounded chance to land before the CTA's shared memory is given back
    if (failed) mbar_wait(bar, copy_phase & 1u, p.wait_polls);
}

// ---- softmax group: warps 12..19; its thread 0 also issues the tensor-core work ---------------------------------------
// kSplitQ: the queries are fp32; a row goes to tensor memory as binary16(q) and as binary16(q - binary16(q)), and S is the
// sum of two products, which equals the fp32-query product to 2^-22 relative.
template <bool kSplitQ>
__device__ __forceinline__ void softmax_role(const AttentionParams &p, uint8_t *smem, PlanHeader *hdr, uint32_t tmem, uint32_t warp,
                                             uint32_t lane, uint32_t row_tiles, const SharedSplit &split) {
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBars);
    uint64_t *bar_full = bars + kBarFull, *bar_free = bars + kBarFree, *bar_s = bars + kBarS, *bar_o = bars + kBarO;
    const uint32_t *round_desc = reinterpret_cast<const uint32_t *>(smem + kOffRound);
    float *row_max = reinterpret_cast<float *>(smem + kOffRowMax);
    const uint32_t shared_pages = hdr->shared_pages;
    const uint32_t G = p.group, rows_total = p.seq_count * G;
    // Thread (warp w, lane) owns row 32 (w & 3) + lane — its warp's quarter of the tensor-memory lanes — and the 64 score
    // columns (4 pages) of half (w - 12) >> 2; the two threads of a row meet through row_max[].
    const uint32_t half = (warp - kDecodeWarps) >> 2, row_in_tile = (warp & 3u) * 32u + lane;
    const uint32_t tmem_row = tmem + (((warp & 3u) * 32u) << 16);
    const bool issuer = warp == kDecodeWarps && lane == 0;

    uint32_t s_phase = 0, o_phase = 0;
    bool failed = false;      // warp-uniform
    bool o_pending = false;   // a P V commit whose arrival on the O barrier has not been waited for yet
    auto wait_o = [&]() {     // O and P in tensor memory may be touched again once the last P V has completed
        if (!o_pending) return;
        o_pending = false;
        if (!failed && !__all_sync(0xffffffffu, mbar_wait(bar_o, o_phase & 1u, p.wait_polls))) {
            failed = true;
            if (lane == 0) raise_status(p, CF_B200_DEVSTAT_WAIT_EXPIRED);
        }
        o_phase ^= 1u;
        tc_fence_after();
    };
    UnitShape u = {};
    float m_run = -CUDART_INF_F, l_run = 0.0f;   // the row's running maximum; this thread's half of its running sum
    float v_unit = 0.0f;                          // largest V scale met so far in the unit: the unit of O
    bool o_started = false;

    for (uint32_t it = 0;; ++it) {
        const uint32_t pair = it & 1u;
        uint8_t *k_tile = smem + kOffTiles + pair * 2u * kTileBytes, *v_tile = k_tile + kTileBytes;
        const float *meta = reinterpret_cast<const float *>(smem + kOffMeta) + pair * 4u * kRoundPages;
        // ---- the round's tiles are decoded (one thread waits, the barrier passes the news on) ----
        if (issuer && !failed && !mbar_wait(&bar_full[pair], (it >> 1) & 1u, p.wait_polls)) {
            failed = true;
            raise_status(p, CF_B200_DEVSTAT_WAIT_EXPIRED);
        }
        failed = __any_sync(0xffffffffu, failed);
        if (group_any(kSoftmaxBarrier, failed)) break;
        const uint32_t unit = round_desc[4 * pair], flags = round_desc[4 * pair + 1];
        if (unit == kStopUnit) break;

        if (flags & kFirstRound) {   // Q rows of the unit: global memory -> tensor memory (binary16 pairs, 64 columns)
            u = unit_shape(p, split, blockIdx.x, unit, row_tiles, shared_pages);
            m_run = -CUDART_INF_F;
            l_run = 0.0f;
            v_unit = 0.0f;
            o_started = false;
            const uint32_t row = u.tile_index * 128u + row_in_tile;
            if constexpr (kSplitQ) {
                const float4 *src = reinterpret_cast<const float4 *>(
                    reinterpret_cast<const float *>(p.queries) +
                    (static_cast<uint64_t>(min(row, rows_total - 1u) / G) * p.query_head_count + u.kv_head * G + min(row, rows_total - 1u) % G) * 128u +
                    64u * half);
#pragma unroll
                for (int c = 0; c < 4; ++c) {   // 16 channels = 8 columns of pairs at a time
                    uint32_t hi[8], lo[8];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        float4 x = src[4 * c + j];
                        if (row >= rows_total) x = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        const __half2 h0 = __floats2half2_rn(x.x, x.y), h1 = __floats2half2_rn(x.z, x.w);
                        const float2 b0 = __half22float2(h0), b1 = __half22float2(h1);
                        const __half2 l0 = __floats2half2_rn(x.x - b0.x, x.y - b0.y), l1 = __floats2half2_rn(x.z - b1.x, x.w - b1.y);
                        hi[2 * j] = *reinterpret_cast<const uint32_t *>(&h0);
                        hi[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&h1);
                        lo[2 * j] = *reinterpret_cast<const uint32_t *>(&l0);
                        lo[2 * j + 1] = *reinterpret_cast<const uint32_t *>(&l1);
                    }
                    tmem_store8(tmem_row + kColQ + 32u * half + 8u * c, hi);
                    tmem_store8(tmem_row + kColQResidue + 32u * half + 8u * c, lo);
                }
            } else {
            uint32_t q_raw[32];
            if (row < rows_total) {
                const uint4 *src = reinterpret_cast<const uint4 *>(
                    reinterpret_cast<const __half *>(p.queries) +
                    (static_cast<uint64_t>(row / G) * p.query_head_count + u.kv_head * G + row % G) * 128u + 64u * half);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 x = src[c];
                    q_raw[4 * c] = x.x;
                    q_raw[4 * c + 1] = x.y;
                    q_raw[4 * c + 2] = x.z;
                    q_raw[4 * c + 3] = x.w;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) q_raw[j] = 0u;
            }
            tmem_store32(tmem_row + kColQ + 32u * half, q_raw);
            }
            tmem_store_wait();
            tc_fence_before();
            if (group_any(kSoftmaxBarrier, false)) break;
        }

        // ---- S = Q K^T ----
        if (issuer) {
            tc_fence_after();
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s) umma(tmem + kColS, tmem + kColQ + 8u * s, tile_desc(smem_addr(k_tile) + 256u * s), s);
            if constexpr (kSplitQ) {
#pragma unroll
                for (uint32_t s = 0; s < 8; ++s) umma(tmem + kColS, tmem + kColQResidue + 8u * s, tile_desc(smem_addr(k_tile) + 256u * s), 1u);
            }
            umma_commit(bar_s);
        }
        float round_scale = 0.0f;   // largest V scale among the round's present pages
#pragma unroll
        for (uint32_t pg = 0; pg < kRoundPages; ++pg)
            if (__float_as_uint(meta[4 * pg + 2]) != 0u) round_scale = fmaxf(round_scale, meta[4 * pg + 1]);
        if (!failed && !__all_sync(0xffffffffu, mbar_wait(bar_s, s_phase & 1u, p.wait_polls))) {
            failed = true;
            if (lane == 0) raise_status(p, CF_B200_DEVSTAT_WAIT_EXPIRED);
        }
        s_phase ^= 1u;
        tc_fence_after();
        uint32_t s_raw[2][32];
        if (!failed) {
            tmem_load32(tmem_row + kColS + 64u * half, s_raw[0]);
            tmem_load32(tmem_row + kColS + 64u * half + 32u, s_raw[1]);
            tmem_load_wait();
        }
        // maximum of the scaled, masked scores of this thread's 4 pages; the raw scores stay in the registers
        float part_max = -CUDART_INF_F;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t pg = 4u * half + q;
            const uint32_t count = __float_as_uint(meta[4 * pg + 2]);
            const float ks = meta[4 * pg];
            if (count == 16u) {   // a full page (the usual case): the scale is applied to the extreme, not to every score
                float hi = __uint_as_float(s_raw[q >> 1][16 * (q & 1)]), lo = hi;
#pragma unroll
                for (int j = 1; j < 16; ++j) {
                    hi = fmaxf(hi, __uint_as_float(s_raw[q >> 1][16 * (q & 1) + j]));
                    lo = fminf(lo, __uint_as_float(s_raw[q >> 1][16 * (q & 1) + j]));
                }
                part_max = fmaxf(part_max, fmaxf(hi * ks, lo * ks));
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (static_cast<uint32_t>(j) < count)
                        part_max = fmaxf(part_max, __uint_as_float(s_raw[q >> 1][16 * (q & 1) + j]) * ks);
            }
        }
        row_max[half * 128u + row_in_tile] = part_max;
        tc_fence_before();   // this thread's reads of S are complete: the next round's S may overwrite it
        if (group_any(kSoftmaxBarrier, failed)) break;

        wait_o();   // the previous round's P V is done with O and P
        if (!failed) {
            const float m_new = fmaxf(m_run, fmaxf(row_max[row_in_tile], row_max[128u + row_in_tile]));
            const float z = m_new == -CUDART_INF_F ? 0.0f : m_new;
            const float alpha = fast_exp2(m_run - z);   // m_run = -inf gives 0
            m_run = m_new;
            // The unit of O is the largest V scale met so far in the unit, so that a page's scale relative to it (which
            // rides on the binary16 weights) never exceeds 1; when a round brings a larger one, O changes unit with it.
            float o_scale = alpha;
            if (round_scale > v_unit) {
                o_scale *= v_unit / round_scale;   // v_unit = 0: nothing accumulated yet
                v_unit = round_scale;
            }
            // O in tensor memory follows the new maximum and unit (this thread's 64 channels); skipped when no row of the
            // warp moved
            if (o_started && !__all_sync(0xffffffffu, o_scale == 1.0f)) {
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < 64u; c0 += 32u) {
                    uint32_t o_raw[32];
                    tmem_load32(tmem_row + kColO + 64u * half + c0, o_raw);
                    tmem_load_wait();
#pragma unroll
                    for (int j = 0; j < 32; ++j) o_raw[j] = __float_as_uint(__uint_as_float(o_raw[j]) * o_scale);
                    tmem_store32(tmem_row + kColO + 64u * half + c0, o_raw);
                }
            }
            // weights as binary16 plus their rounding residue (two A operands), so that P V is accurate to fp32 level
            // whatever the spread of the V scales
            float sum = 0.0f;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t pg = 4u * half + q;
                const uint32_t count = __float_as_uint(meta[4 * pg + 2]);
                const float ks = meta[4 * pg];
                // the weights (at most 1) also carry 2^15, exactly, which O sheds at the unit's end: binary16 then resolves
                // weights down to 2^-40 of the row maximum instead of 2^-25
                const float ratio = count ? __fdividef(meta[4 * pg + 1], v_unit) * kWeightScale : 0.0f;
                uint32_t hi[8], lo[8];
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    float w0 = fast_exp2(fmaf(__uint_as_float(s_raw[q >> 1][16 * (q & 1) + j]), ks, -z));
                    float w1 = fast_exp2(fmaf(__uint_as_float(s_raw[q >> 1][16 * (q & 1) + j + 1]), ks, -z));
                    if (count != 16u) {   // tokens past the page's count weigh nothing
                        w0 = static_cast<uint32_t>(j) < count ? w0 : 0.0f;
                        w1 = static_cast<uint32_t>(j + 1) < count ? w1 : 0.0f;
                    }
                    sum += w0 + w1;
                    const float a0 = w0 * ratio, a1 = w1 * ratio;
                    const __half2 h = __floats2half2_rn(a0, a1);
                    const float2 back = __half22float2(h);
                    const __half2 l = __floats2half2_rn(a0 - back.x, a1 - back.y);
                    hi[j >> 1] = *reinterpret_cast<const uint32_t *>(&h);
                    lo[j >> 1] = *reinterpret_cast<const uint32_t *>(&l);
                }
                tmem_store8(tmem_row + kColP + 8u * pg, hi);          // 16 tokens = 8 columns of pairs
                tmem_store8(tmem_row + kColPResidue + 8u * pg, lo);
            }
            tmem_store_wait();
            l_run = l_run * alpha + sum;   // this thread's half of the row's sum; the halves are added at the unit's end
        }
        tc_fence_before();
        if (group_any(kSoftmaxBarrier, failed)) break;

        // ---- O += P V ----
        if (issuer) {
            tc_fence_after();
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s)
                umma(tmem + kColO, tmem + kColP + 8u * s, tile_desc(smem_addr(v_tile) + 256u * s), (o_started || s) ? 1u : 0u);
#pragma unroll
            for (uint32_t s = 0; s < 8; ++s) umma(tmem + kColO, tmem + kColPResidue + 8u * s, tile_desc(smem_addr(v_tile) + 256u * s), 1u);
            umma_commit(bar_o);
            umma_commit(&bar_free[pair]);   // the decoders may refill this pair of tiles
        }
        o_started = true;
        o_pending = true;

        // ---- last round of the unit: one (max, sum, weighted[128]) per row; each thread writes its 64 channels ----
        if (flags & kLastRound) {
            wait_o();
            row_max[half * 128u + row_in_tile] = l_run;   // reused: the two halves of the row's sum
            if (group_any(kSoftmaxBarrier, failed)) break;
            const uint32_t row = u.tile_index * 128u + row_in_tile;
            const bool live = row < rows_total;   // whole warps go on: the tensor-memory loads are warp-wide
            float *dst = live ? shared_partial_ptr(p, u.chunk, row / G, u.head_local * G + row % G) : nullptr;
            const float o_unit = v_unit * (1.0f / kWeightScale);
            if (live && half == 0) {
                dst[0] = m_run;
                dst[1] = row_max[row_in_tile] + row_max[128u + row_in_tile];
            }
#pragma unroll 1
            for (uint32_t c0 = 0; c0 < 64u; c0 += 32u) {
                uint32_t o_raw[32];
                tmem_load32(tmem_row + kColO + 64u * half + c0, o_raw);
                tmem_load_wait();
                if (live) {
#pragma unroll
                    for (int t = 0; t < 8; ++t) {   // columns t, t + 8, t + 16, t + 24 of the 32 are 4 consecutive channels
                        float *out = dst + 2 + 64u * half + c0 + 4 * t;
                        *reinterpret_cast<float2 *>(out) =
                            make_float2(__uint_as_float(o_raw[t]) * o_unit, __uint_as_float(o_raw[t + 8]) * o_unit);
                        *reinterpret_cast<float2 *>(out + 2) =
                            make_float2(__uint_as_float(o_raw[t + 16]) * o_unit, __uint_as_float(o_raw[t + 24]) * o_unit);
                    }
                }
            }
            tc_fence_before();
        }
    }
    // leaving early: give the tensor core's last commit a bounded chance to arrive before tensor memory is freed
    if (o_pending && !failed) mbar_wait(bar_o, o_phase & 1u, p.wait_polls);
}

template <bool kSplitQ>
__global__ void __launch_bounds__(kTcThreads, 1) prefix_attention_kernel(AttentionParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kOffBars);
    uint32_t *misc = reinterpret_cast<uint32_t *>(smem + kOffMisc);

    PlanHeader *hdr = plan_header(p);
    // uniform: nothing shared, the plan refused the hint, or the split leaves this CTA without a share
    if (hdr->shared_pages == 0 || blockIdx.x >= hdr->shared_ctas) return;

    load_tables(smem, p, tid, kTcThreads);
    if (tid == 0) {
        for (uint32_t w = 0; w < kDecodeWarps; ++w) mbar_init(bars + w, 1);   // copies
        mbar_init(bars + kBarFull, kRoundPages);                    // full[0], full[1]: one arrival per page slot of the round
        mbar_init(bars + kBarFull + 1, kRoundPages);
        for (uint32_t i = kBarFree; i < kBarCount; ++i) mbar_init(bars + i, 1);   // free[0], free[1], S, O: tensor-core commits
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    if (warp == 0) {   // one whole warp allocates the CTA's tensor memory and frees it at the end
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&misc[0])), "r"(kTmemColumns));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc[0];

    const uint32_t rows_total = p.seq_count * p.group;
    const uint32_t row_tiles = (rows_total + 127u) / 128u;
    const SharedSplit split = {hdr->shared_rounds, p.kv_head_span * row_tiles, hdr->shared_ctas};

    if (warp < kDecodeWarps) {   // whole warpgroups on either side: the register split is per warpgroup
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kDecoderRegs));
        decoder_role(p, smem, hdr, warp, lane, row_tiles, split);
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
        softmax_role<kSplitQ>(p, smem, hdr, tmem, warp, lane, row_tiles, split);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemColumns));
}

}  // namespace

cudaError_t launch_prefix_attention(const AttentionParams &p, cudaStream_t stream) {
    static LauncherState table[64];
    cudaError_t e;
    LauncherState *state = launcher_state(table, &e);
    if (!state) return e;
    const int sm_count = state->sm_count;
    if (!state->configured) {
        for (int split = 0; split < 2; ++split) {
            const void *kernel = split ? reinterpret_cast<const void *>(prefix_attention_kernel<true>)
                                       : reinterpret_cast<const void *>(prefix_attention_kernel<false>);
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kTcSmem));
            if (e != cudaSuccess) return e;
            cudaFuncAttributes attr;
            e = cudaFuncGetAttributes(&attr, kernel);
            if (e != cudaSuccess) return e;
            if (attr.numRegs != kLaunchRegs) return cudaErrorLaunchOutOfResources;   // the register split assumes this count
        }
        state->configured = true;
    }
    if (p.query_type == CF_B200_F32) prefix_attention_kernel<true><<<sm_count, kTcThreads, kTcSmem, stream>>>(p);
    else prefix_attention_kernel<false><<<sm_count, kTcThreads, kTcSmem, stream>>>(p);
    return cudaPeekAtLastError();
}

}  // namespace cfb
