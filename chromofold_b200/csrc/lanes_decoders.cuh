// lanes_decoders.cuh — pieces shared by the lane-per-block kernels (sealed_attention_lanes.cu,
// sealed_attention_prefix.cu): PTX wrappers (bulk async copy + mbarrier with bounded waits, mma.sync), the exact
// symbol -> binary16 conversion, and the per-lane block decoders for streams of 2048 symbols (head_dim 128, page_tokens
// 16) cut into NB blocks: NB = 32 (block_size 64, lane l decodes block l: the layout every kernel is built around),
// 16 or 8 (block_size 128 / 256, decoded into a shared-memory tile first, see sealed_attention_lanes.cu).
#ifndef CHROMOFOLD_B200_LANES_DECODERS_CUH
#define CHROMOFOLD_B200_LANES_DECODERS_CUH

#include <math_constants.h>

#include "attention_params.cuh"

namespace cfb {
namespace lanes {

constexpr uint32_t kStageBytes = 4160;   // 16 header + 2 * 2048 payload max + 48 slack (decoders read ahead)
constexpr uint32_t kTableBytes = 2 * 4096 * 4 + 2 * 4096 * 2;
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kMagic = 0x64646464u;       // fp16 1024.0 high byte, for the byte-permute conversion
constexpr uint32_t kBias2 = 0x64806480u;       // half2(1152, 1152) = 1024 + zero point

// ---- PTX wrappers ------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_addr(const void *p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
// One poll; the warp may be suspended for up to about a microsecond inside it (the hint bounds a single poll, so that
// a number of polls is a bound on time).
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity), "r"(1000u)
        : "memory");
    return ok != 0;
}
// Bounded wait: false if the barrier did not complete within `polls` polls (AttentionParams::wait_polls).
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t polls) {
    for (uint32_t i = 0; i < polls; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// One bulk async copy global -> this CTA's shared memory (16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load(void *dst, const void *src, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
// Four packed symbols (byte i = symbol i) -> two half2 of codes (symbol - 128), exact.
__device__ __forceinline__ void quad_to_half2(uint32_t quad, uint32_t &lo, uint32_t &hi) {
    lo = hsub2_u32(__byte_perm(quad, kMagic, 0x4140), kBias2);  // (s0, s1)
    hi = hsub2_u32(__byte_perm(quad, kMagic, 0x4342), kBias2);  // (s2, s3)
}

// a * b + c on the multiply-add pipe. Plain adds and constant shifts written this way leave the integer ALU pipe,
// which is the busiest one in the decoders, to the operations that have no other home (logic, funnel shifts).
__device__ __forceinline__ uint32_t imad(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}

// The low bytes of four table entries as one register, first symbol in byte 0: three byte permutes.
__device__ __forceinline__ uint32_t pack_low_bytes(uint32_t e0, uint32_t e1, uint32_t e2, uint32_t e3) {
    return __byte_perm(__byte_perm(e0, e1, 0x0040), __byte_perm(e2, e3, 0x0040), 0x5410);
}

// ---- per-lane block decoders: each yields four symbols packed in one register -----------------------------------
// Both entropy decoders are written without branches so that the K chain and the V chain of a lane interleave in
// one straight instruction stream. A 64-bit window holds the upcoming stream bits, top aligned; it is reloaded from
// shared memory once per quad (four symbols), which is as often as it can run dry.
template <int NB>
struct RansLaneT {
    static constexpr bool kWholeQuads = false;
    static constexpr uint32_t kHead = (6u * NB + 3u) / 4u * 4u;   // u32 state0[NB] | u16 byte_off[NB]
    static constexpr int kSymbolsPerReload = 4;   // a symbol takes at most two bytes; the window holds eight
    uint32_t x, whi, wlo, used;   // state; window (next byte = top byte of whi); bits taken since the reload
    uint32_t pos;                 // shared-memory byte address of the first byte not yet taken at the last reload
    uint32_t table;               // shared-memory byte address of the slot table
    // The block's start offset is clamped to the part (part_bytes from the record header): whatever the block table
    // says, the decoder starts inside its own part, and from there a block takes at most 64 * 2 bytes plus one
    // 12-byte window, which stays inside the warp's own shared memory (part_offsets_ok reports the bad table).
    __device__ __forceinline__ void open(const uint8_t *part, uint32_t part_bytes, uint32_t lane, const uint32_t *slot_table) {
        x = reinterpret_cast<const uint32_t *>(part)[lane];
        const uint32_t payload = part_bytes > kHead ? part_bytes - kHead : 0u;
        pos = smem_addr(part) + kHead + min(static_cast<uint32_t>(reinterpret_cast<const uint16_t *>(part + 4 * NB)[lane]), payload);
        table = smem_addr(slot_table);
        used = 0;
    }
    // Eight bytes starting at `pos`, in stream order, most significant first (the order rans.cu:23 shifts them in).
    __device__ __forceinline__ void reload() {
        pos += used >> 3;
        used = 0;
        const uint32_t base = pos & ~3u, align = imad(pos & 3u, 0x1111u, 0x0123u);
        uint32_t w0, w1, w2;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w0) : "r"(base));
        asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(w1) : "r"(base));
        asm volatile("ld.shared.u32 %0, [%1+8];" : "=r"(w2) : "r"(base));
        whi = __byte_perm(w0, w1, align);
        wlo = __byte_perm(w1, w2, align);
    }
    // src/cuda/rans.cu:20-23: x = freq * (x >> 12) + (x & 4095) - cum, then bytes are shifted in while x < 2^23.
    // The shared-memory table holds e = sym | (slot - cum) << 8 | freq << 20, so e >> 8 = (slot - cum) + freq * 4096
    // and the update is freq * ((x >> 12) - 4096) + (e >> 8): no field of the entry needs masking.
    // After the update the state is >= 2^11, so the reference's loop runs 0, 1 or 2 times: (clz(state) - 1) / 8.
    __device__ __forceinline__ uint32_t symbol() {
        uint32_t e;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(e) : "r"(imad(x & (CF_B200_RANS_M - 1u), 4u, table)));
        x = imad(e >> 20, imad(x >> CF_B200_RANS_PROB_BITS, 1u, 0u - CF_B200_RANS_M), e >> 8);
        const uint32_t shift = imad(static_cast<uint32_t>(__clz(x)), 1u, 0xffffffffu) & 24u;
        x = __funnelshift_l(whi, x, shift);
        whi = __funnelshift_l(wlo, whi, shift);
        wlo <<= shift;
        used = imad(shift, 1u, used);
        return e;
    }
    __device__ __forceinline__ uint32_t quad(int) {   // quad index: the decoders that need it get it from an unrolled loop
        reload();
        const uint32_t e0 = symbol(), e1 = symbol(), e2 = symbol(), e3 = symbol();
        return pack_low_bytes(e0, e1, e2, e3);
    }
};
using RansLane = RansLaneT<32>;

// Low nibbles of the four symbols of a quad (in the low nibble of each byte of w; its high nibbles are ignored) under
// the two pair symbols that hold their high nibbles (table entries, pair A:B in the low byte): four symbols, first in byte 0.
__device__ __forceinline__ uint32_t merge_split_quad(uint32_t e0, uint32_t e1, uint32_t w) {
    const uint32_t t = __byte_perm(e0, e1, 0x4400);             // (s1, s1, s0, s0), s = A:B
    const uint32_t t4 = imad(t, 16u, 0u);                       // bytes 1 and 3 now start with B
    const uint32_t h = __byte_perm(t, t4, 0x7250);              // (B1:*, A1:*, B0:*, A0:*)
    return (h & 0xf0f0f0f0u) | (w & 0x0f0f0f0fu);
}

// Nibble-split rANS (CF_B200_CODER_RANS_SPLIT4): the low nibble of every symbol is stored raw in a lane-interleaved
// plane, and the rANS stream codes PAIRS of high nibbles (pair symbol = hi(2k) << 4 | hi(2k + 1)), so a block of 64
// symbols is 32 steps of the same recurrence. Part layout: u32 state0[NB] | u16 byte_off[NB] | u32 lo[symbols/NB/8][NB] |
// bytes; lo[j][l] holds the low nibbles of symbols 8j..8j+7 of block l: symbol 8j + i at bits 8i..8i+3 for i < 4,
// symbol 8j + 4 + i at bits 8i+4..8i+7. The plane is 1024 bytes whatever the block size.
template <int NB, int kSyms = 2048>
struct RansSplitLaneT : RansLaneT<NB> {
    using Base = RansLaneT<NB>;
    using Base::x; using Base::pos; using Base::table; using Base::used; using Base::kHead;
    static constexpr bool kWholeQuads = true;   // callers ask for a quad at a time (the window is refilled inside)
    static constexpr uint32_t kPlaneBytes = kSyms / 2u;   // a nibble per symbol
    uint32_t lo;   // shared-memory byte address of lo[0][lane]
    __device__ __forceinline__ void open(const uint8_t *part, uint32_t part_bytes, uint32_t lane, const uint32_t *slot_table) {
        x = reinterpret_cast<const uint32_t *>(part)[lane];
        const uint32_t payload = part_bytes > kHead + kPlaneBytes ? part_bytes - kHead - kPlaneBytes : 0u;
        lo = smem_addr(part) + kHead + 4u * lane;
        pos = smem_addr(part) + kHead + kPlaneBytes + min(static_cast<uint32_t>(reinterpret_cast<const uint16_t *>(part + 4 * NB)[lane]), payload);
        table = smem_addr(slot_table);
        used = 0;
    }
    __device__ __forceinline__ uint32_t lo_word(int j) const {
        uint32_t w;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(lo + 4u * NB * j));
        return w;
    }
    __device__ __forceinline__ uint32_t quad(int q) {   // one stream on its own (mixed-coder records)
        if ((q & 1) == 0) Base::reload();
        const uint32_t e0 = Base::symbol(), e1 = Base::symbol();
        return merge_split_quad(e0, e1, lo_word(q >> 1) >> (4 * (q & 1)));
    }
};
using RansSplitLane = RansSplitLaneT<32>;

template <int NB>
struct HuffLaneT {
    static constexpr bool kWholeQuads = false;
    static constexpr uint32_t kHead = (2u * NB + 3u) / 4u * 4u;   // u16 bit_off[NB]
    static constexpr int kSymbolsPerReload = 5;   // a code takes at most 12 bits; the window holds 64
    uint32_t whi, wlo, used;   // window of upcoming bits, MSB first; bits taken since the reload
    uint32_t words, bit;       // shared-memory address of the payload words; bit position at the last reload
    uint32_t table;
    // Start offset clamped to the part as in RansLane::open; a block takes at most 64 * 12 bits plus one window.
    __device__ __forceinline__ void open(const uint8_t *part, uint32_t part_bytes, uint32_t lane, const uint16_t *lut) {
        const uint32_t payload_bits = part_bytes > kHead ? (part_bytes - kHead) * 8u : 0u;
        bit = min(static_cast<uint32_t>(reinterpret_cast<const uint16_t *>(part)[lane]), payload_bits);
        words = smem_addr(part) + kHead;
        table = smem_addr(lut);
        used = 0;
    }
    __device__ __forceinline__ void reload() {
        bit += used;
        used = 0;
        const uint32_t base = words + ((bit >> 5) << 2), off = bit & 31u;
        uint32_t w0, w1, w2;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w0) : "r"(base));
        asm volatile("ld.shared.u32 %0, [%1+4];" : "=r"(w1) : "r"(base));
        asm volatile("ld.shared.u32 %0, [%1+8];" : "=r"(w2) : "r"(base));
        whi = __funnelshift_l(w1, w0, off);
        wlo = __funnelshift_l(w2, w1, off);
    }
    // include/chromofold/detail/block_huffman_device.cuh:12-19: the next 12 bits, MSB-first, index the LUT.
    __device__ __forceinline__ uint32_t symbol() {
        uint32_t e;
        asm volatile("ld.shared.u16 %0, [%1];" : "=r"(e) : "r"(imad(whi >> (32u - CF_B200_HUFF_MAXLEN), 2u, table)));
        const uint32_t len = e >> 8;
        whi = __funnelshift_l(wlo, whi, len);
        wlo <<= len;
        used = imad(len, 1u, used);
        return e;
    }
    __device__ __forceinline__ uint32_t quad(int) {
        reload();
        const uint32_t e0 = symbol(), e1 = symbol(), e2 = symbol(), e3 = symbol();
        return pack_low_bytes(e0, e1, e2, e3);
    }
};
using HuffLane = HuffLaneT<32>;

// Nibble-split Huffman (CF_B200_CODER_HUFFMAN_SPLIT4): u16 bit_off[NB] | u32 lo[symbols/NB/8][NB] | words; one LUT hit = a pair.
template <int NB, int kSyms = 2048>
struct HuffSplitLaneT : HuffLaneT<NB> {
    using Base = HuffLaneT<NB>;
    using Base::bit; using Base::words; using Base::table; using Base::used; using Base::kHead;
    static constexpr bool kWholeQuads = true;
    static constexpr uint32_t kPlaneBytes = kSyms / 2u;   // a nibble per symbol
    uint32_t lo;
    __device__ __forceinline__ void open(const uint8_t *part, uint32_t part_bytes, uint32_t lane, const uint16_t *lut) {
        const uint32_t payload_bits = part_bytes > kHead + kPlaneBytes ? (part_bytes - kHead - kPlaneBytes) * 8u : 0u;
        bit = min(static_cast<uint32_t>(reinterpret_cast<const uint16_t *>(part)[lane]), payload_bits);
        lo = smem_addr(part) + kHead + 4u * lane;
        words = smem_addr(part) + kHead + kPlaneBytes;
        table = smem_addr(lut);
        used = 0;
    }
    __device__ __forceinline__ uint32_t lo_word(int j) const {
        uint32_t w;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w) : "r"(lo + 4u * NB * j));
        return w;
    }
    __device__ __forceinline__ uint32_t quad(int q) {
        if ((q & 1) == 0) Base::reload();   // four pair symbols take at most 48 bits
        const uint32_t e0 = Base::symbol(), e1 = Base::symbol();
        return merge_split_quad(e0, e1, lo_word(q >> 1) >> (4 * (q & 1)));
    }
};
using HuffSplitLane = HuffSplitLaneT<32>;

template <int NB, int kSyms = 2048>
struct FixedLaneT {
    static constexpr bool kWholeQuads = true;  // a quad is one word: nothing to interleave
    static constexpr int kSymbolsPerReload = 4;
    const uint32_t *words;
    // A fixed-width part is kSyms bytes at a 16-byte aligned offset of at most 16 + 2048 into the stage: always inside it.
    __device__ __forceinline__ void open(const uint8_t *part, uint32_t, uint32_t lane) {
        words = reinterpret_cast<const uint32_t *>(part) + (kSyms / 4u / NB) * lane;
    }
    // src/runtime/kv_gpu_fixture.cpp:110-116: symbol i sits in the i-th byte from the top of the word.
    __device__ __forceinline__ uint32_t quad(int) { return __byte_perm(*words++, 0u, 0x0123); }
};
using FixedLane = FixedLaneT<32>;

// Coding tables into shared memory, once per CTA: [k rANS slots | v rANS slots | k Huffman LUT | v Huffman LUT].
// Slot entries are re-packed for RansLane::symbol(): sym | (slot - cum) << 8 | freq << 20.
__device__ __forceinline__ void load_tables(uint8_t *smem, const AttentionParams &p, uint32_t tid, uint32_t threads) {
    uint32_t *k_slot = reinterpret_cast<uint32_t *>(smem);
    uint32_t *v_slot = k_slot + 4096;
    auto repack = [](uint32_t e) { return (e & 0xffu) | ((e >> 20) << 8) | (((e >> 8) & 0xfffu) << 20); };
    for (uint32_t i = tid; i < 4096; i += threads) {
        k_slot[i] = repack(p.k_tables->rans_slot[i]);
        v_slot[i] = repack(p.v_tables->rans_slot[i]);
    }
    const uint4 *src = reinterpret_cast<const uint4 *>(p.k_tables->huff_lut);
    uint4 *dst = reinterpret_cast<uint4 *>(v_slot + 4096);
    for (uint32_t i = tid; i < 512; i += threads) dst[i] = src[i];
    src = reinterpret_cast<const uint4 *>(p.v_tables->huff_lut);
    dst += 512;
    for (uint32_t i = tid; i < 512; i += threads) dst[i] = src[i];
}

// Header checks of a staged record against its directory entry; false = the page is to be skipped.
__device__ __forceinline__ bool record_header_ok(const uint4 &hv, uint64_t dir_entry, uint32_t codebook_id) {
    const uint32_t k_units = hv.x & 0xffffu, v_units = hv.x >> 16;
    const uint32_t k_coder = hv.y & 0xffu, v_coder = (hv.y >> 8) & 0xffu, token_count = hv.y >> 16;
    const uint32_t codebook = hv.w & 0xffffu, version = hv.w >> 24;
    return version == CF_B200_FORMAT_VERSION && codebook == codebook_id &&
           1u + k_units + v_units == CF_B200_DIR_LENGTH_UNITS(dir_entry) && k_units <= 128u && v_units <= 128u &&
           k_coder <= CF_B200_CODER_MAX && v_coder <= CF_B200_CODER_MAX && token_count >= 1u && token_count <= 16u;
}

// The block table of a staged part against the part's length: lane l checks the start of block l. The reference
// validates its descriptors on the host before the launch (src/cuda/paged_kv_attention.cu:280-299); records here are
// written by the sealer, by import or by unpack, so the check runs where the table is read.
template <int NB = 32, int kSyms = 2048>
__device__ __forceinline__ bool part_offsets_ok(const uint8_t *part, uint32_t coder, uint32_t part_bytes, uint32_t lane) {
    constexpr uint32_t kRansHead = RansLaneT<NB>::kHead, kHuffHead = HuffLaneT<NB>::kHead, kPlane = kSyms / 2u;
    // A rANS block's start state must lie in [2^23, 2^31), as every state the sealer leaves does: the lane decoders
    // rely on it (a state in range stays in range, and then a step takes at most two bytes).
    if (coder == CF_B200_CODER_RANS || coder == CF_B200_CODER_RANS_SPLIT4) {
        const uint32_t state0 = reinterpret_cast<const uint32_t *>(part)[lane];
        if (part_bytes < kRansHead || state0 < CF_B200_RANS_L || state0 >= (CF_B200_RANS_L << 8)) return false;
    }
    if (coder == CF_B200_CODER_RANS)
        return part_bytes >= kRansHead && reinterpret_cast<const uint16_t *>(part + 4 * NB)[lane] <= part_bytes - kRansHead;
    if (coder == CF_B200_CODER_HUFFMAN)
        return part_bytes >= kHuffHead && reinterpret_cast<const uint16_t *>(part)[lane] <= (part_bytes - kHuffHead) * 8u;
    if (coder == CF_B200_CODER_RANS_SPLIT4)
        return part_bytes >= kRansHead + kPlane && reinterpret_cast<const uint16_t *>(part + 4 * NB)[lane] <= part_bytes - kRansHead - kPlane;
    if (coder == CF_B200_CODER_HUFFMAN_SPLIT4)
        return part_bytes >= kHuffHead + kPlane && reinterpret_cast<const uint16_t *>(part)[lane] <= (part_bytes - kHuffHead - kPlane) * 8u;
    return part_bytes == static_cast<uint32_t>(kSyms);
}

}  // namespace lanes
}  // namespace cfb

#endif
