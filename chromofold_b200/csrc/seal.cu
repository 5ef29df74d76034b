// seal.cu — GPU page sealer: quantise, entropy-code and publish full pages in one launch.
//
// The reference seals on the device in six launches with a host synchronisation in the middle and one allocation
// per array (src/cuda/device_kv_seal_attention.cu:244-334: finite_scan, quantize_int4, pack_nibbles, then a host
// side table upload) and only produces fixed-width nibbles. Here one CTA owns one (page, kv head): it scans for
// non-finite values, derives the two stream scales, quantises (round-half-even, clamp, +zero point —
// src/runtime/kv_gpu_fixture.cpp:12-16), codes both streams block by block with the exact inverse of the decoders in
// cf_device_common.cuh, takes room in the arena with one atomic add, writes the record and only then the directory
// entry, so a reader never sees a half-written page and the host is not involved.

#include <cuda_bf16.h>

#include <type_traits>

#include "cf_device_common.cuh"

namespace cfb {
namespace {

constexpr int kSealThreads = 128;

struct SealSmem {
    uint32_t off_ksym, off_vsym, off_kpair, off_vpair, off_scratch, off_part, off_blk, off_enc, part_capacity, slot_bytes, total;
};

__host__ __device__ inline bool split_coder(uint32_t coder) {
    return coder == CF_B200_CODER_RANS_SPLIT4 || coder == CF_B200_CODER_HUFFMAN_SPLIT4;
}
__host__ __device__ inline bool rans_family(uint32_t coder) { return coder == CF_B200_CODER_RANS || coder == CF_B200_CODER_RANS_SPLIT4; }

__host__ __device__ inline SealSmem seal_smem(uint32_t symbols, uint32_t nblocks, uint32_t block_size) {
    SealSmem s;
    s.slot_bytes = align_up_u32(block_size * 3u / 2u + 4u, 4u);  // a symbol costs at most 12 bits
    s.part_capacity = align_up_u32(symbols, 16u) + 16u;
    s.off_ksym = 0;
    s.off_vsym = s.off_ksym + align_up_u32(symbols, 16u);
    s.off_kpair = s.off_vsym + align_up_u32(symbols, 16u);          // pair symbols of the nibble-split coders
    s.off_vpair = s.off_kpair + align_up_u32(symbols / 2u, 16u);
    s.off_scratch = s.off_vpair + align_up_u32(symbols / 2u, 16u);
    s.off_part = s.off_scratch + 2u * nblocks * s.slot_bytes;   // one scratch area per stream
    s.off_blk = s.off_part + 2u * s.part_capacity;
    s.off_enc = align_up_u32(s.off_blk + 6u * nblocks * 4u, 8u);
    s.total = s.off_enc + 2u * 256u * 8u + 64u;
    return s;
}

struct SealParams {
    uint32_t kv_head_count, head_dim, page_tokens, block_size, coder, codebook_id, symbols, nblocks;
    const cf_b200_codebook_tables *k_tables, *v_tables;
    const void *tail_k, *tail_v;
    uint32_t tail_type, tail_capacity;
    const uint32_t *job_slots, *job_pages, *job_tokens, *job_heads, *job_rows;
    uint8_t *arena;
    uint64_t arena_units;
    unsigned long long *cursor;
    uint64_t *page_dir;
    uint32_t *status;
};

__device__ __forceinline__ uint16_t scale_bits_from_absmax(float maximum) {
    if (maximum == 0.0f) return 0x3c00u;  // all-zero stream: scale 1 (kv_gpu_fixture.cpp:70)
    uint16_t bits = __half_as_ushort(__float2half_rn(__fdiv_rn(maximum, 127.0f)));
    if (bits == 0) bits = 1;
    if ((bits & 0x7c00u) == 0x7c00u) bits = 0x7bffu;
    return bits;
}

__device__ __forceinline__ uint32_t quantise_symbol(float x, float scale) {
    int q = __float2int_rn(__fdiv_rn(x, scale));
    q = max(-128, min(127, q));
    return static_cast<uint32_t>(q + kZero);
}

// The same symbol without the IEEE division on the common path. With r = RN(1 / scale), y = RN(x * r) differs from
// q = RN(x / scale) by at most 1.5 * 2^-23 * |q|, which is below 2^-15 wherever the clamp does not decide anyway; so when
// y is further than 2^-14 from every half-integer, rint(y) = rint(q), and only the few values closer than that take
// the division. (Beyond +-129 both round far outside the clamp; an overflowing product is +-inf on both paths.)
__device__ __forceinline__ uint32_t quantise_symbol_rcp(float x, float scale, float rcp) {
    const float y = x * rcp, n = rintf(y);
    if (fabsf(fabsf(y - n) - 0.5f) < 6.103515625e-05f) return quantise_symbol(x, scale);
    const int q = max(-128, min(127, __float2int_rn(n)));
    return static_cast<uint32_t>(q + kZero);
}

// Block-wide absmax and non-finite flag over `count` binary16 values.
__device__ __forceinline__ float tile_value(const void *base, uint32_t type, uint64_t i) {
    return type == CF_B200_F32 ? static_cast<const float *>(base)[i] : __half2float(static_cast<const __half *>(base)[i]);
}

__device__ float tile_absmax(const void *base, uint32_t type, uint64_t tile, uint32_t count, int *nonfinite, float *red) {
    float m = 0.0f;
    int bad = 0;
    for (uint32_t i = threadIdx.x; i < count; i += kSealThreads) {
        const float x = tile_value(base, type, tile + i);
        if (!isfinite(x)) bad = 1;
        else m = fmaxf(m, fabsf(x));
    }
    m = warp_max(m);
    bad = __any_sync(0xffffffffu, bad);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
        red[threadIdx.x >> 5] = m;
        red[4 + (threadIdx.x >> 5)] = static_cast<float>(bad);
    }
    __syncthreads();
    float r = 0.0f, b = 0.0f;
    for (int w = 0; w < kSealThreads / 32; ++w) {
        r = fmaxf(r, red[w]);
        b = fmaxf(b, red[4 + w]);
    }
    *nonfinite = b != 0.0f;
    return r;
}

// Inverse of rans_decode_block: symbols pushed last to first from state L; bytes leave the low end of the state
// and are written backwards so that they read forwards. Returns the byte count; *state0 gets the final state.
__device__ uint32_t rans_encode_block(const uint8_t *sym, int count, const uint2 *enc, uint8_t *slot_end, uint32_t *state0) {
    uint32_t x = kRansL;
    uint8_t *p = slot_end;
    for (int j = count - 1; j >= 0; --j) {
        const uint2 e = enc[sym[j]];   // rans_enc of the codebook: {rcp, cum | (4096 - f) << 13 | (shift - 1) << 25}
        const uint32_t cmpl = (e.y >> 13) & 0xfffu, x_max = (4096u - cmpl) << 19;  // ((L >> 12) << 8) * f
        while (x >= x_max) {
            *--p = static_cast<uint8_t>(x & 0xffu);
            x >>= 8;
        }
        x = x + (e.y & 0x1fffu) + (__umulhi(x, e.x) >> (e.y >> 25)) * cmpl;
    }
    *state0 = x;
    return static_cast<uint32_t>(slot_end - p);
}

// Append `len` bits (MSB-first) at bit position `bit` of a zeroed word array shared with other writers.
__device__ __forceinline__ void put_bits(uint32_t *words, uint32_t bit, uint32_t code, uint32_t len) {
    const uint32_t w = bit >> 5, room = 32u - (bit & 31u);
    if (len <= room) {
        atomicOr(&words[w], code << (room - len));
    } else {
        atomicOr(&words[w], code >> (len - room));
        atomicOr(&words[w + 1], code << (32u - (len - room)));
    }
}

// Encode the K stream (which = 0) and the V stream (which = 1) into their parts (shared memory, zeroed by the caller),
// both at once: block b of stream w is the job of thread w * nblocks + b. Whole-CTA call. bytes_out[w] gets the part
// size (a multiple of 16), coder_out[w] the coder actually stored.
struct StreamJob {
    const uint8_t *sym;
    uint8_t *pairs;      // room for symbols / 2 pair symbols (nibble-split coders)
    const cf_b200_codebook_tables *tables;
    const uint2 *enc;
    uint8_t *part;
};

__device__ void encode_streams(const SealParams &p, const SealSmem &lay, const StreamJob (&job)[2], uint8_t *scratch,
                               uint32_t *blk_len, uint32_t *blk_off, uint32_t *blk_state, volatile uint32_t *s_flag,
                               uint32_t (&coder_out)[2], uint32_t (&bytes_out)[2]) {
    const uint32_t tid = threadIdx.x, nb = p.nblocks, n = p.symbols;
    const uint32_t fixed_bytes = align_up_u32(n, 16u);
    uint32_t coder[2] = {p.coder, p.coder};
    bytes_out[0] = bytes_out[1] = fixed_bytes;
    // What the entropy coder sees: the symbols, or (nibble-split) the pairs of high nibbles, half as many per block; the
    // raw low-nibble plane of a split part sits between the block table and the payload.
    const bool split = split_coder(p.coder), rans = rans_family(p.coder);
    const uint32_t per = split ? 2u : 1u, head = align_up_u32(rans ? 6u * nb : 2u * nb, 4u);
    const uint32_t plane_bytes = split ? (p.block_size / 8u) * nb * 4u : 0u;
    if (split) {
        for (uint32_t i = tid; i < n; i += kSealThreads) {   // pair symbols, and every symbol's low nibble into its plane word
            const uint32_t w = i / (n / 2u), k = i % (n / 2u);
            const uint8_t *sym = job[w].sym;
            job[w].pairs[k] = static_cast<uint8_t>((sym[2u * k] & 0xf0u) | (sym[2u * k + 1u] >> 4));
        }
        for (uint32_t i = tid; i < 2u * plane_bytes / 4u; i += kSealThreads) {
            const uint32_t w = i / (plane_bytes / 4u), r = i % (plane_bytes / 4u), j = r / nb, b = r % nb;
            const uint32_t first = b * p.block_size + 8u * j;   // lo[j][b]: symbols first .. first + 7
            uint32_t word = 0u;
            for (uint32_t a = 0; a < 8u; ++a)
                if (first + a < n) word |= static_cast<uint32_t>(job[w].sym[first + a] & 0x0fu) << (a < 4u ? 8u * a : 8u * (a - 4u) + 4u);
            reinterpret_cast<uint32_t *>(job[w].part + head)[r] = word;
        }
        __syncthreads();
    }
    if (p.coder != CF_B200_CODER_FIXED8) {
        for (uint32_t j = tid; j < 2u * nb; j += kSealThreads) {  // pass 1: coded length of every block
            const uint32_t w = j / nb, b = j % nb, base = b * p.block_size;
            const int count = static_cast<int>(min(p.block_size, n - base) / per);
            const uint8_t *src = split ? job[w].pairs + base / 2u : job[w].sym + base;
            if (rans) {
                uint32_t st;
                blk_len[j] = rans_encode_block(src, count, job[w].enc, scratch + (j + 1) * lay.slot_bytes, &st);
                blk_state[j] = st;
            } else {
                uint32_t bits = 0;
                for (int i = 0; i < count; ++i) bits += job[w].tables->huff_code[src[i]] >> 16;
                blk_len[j] = bits;
            }
        }
        __syncthreads();
        if (tid < 2) {
            uint32_t run = 0;
            for (uint32_t b = 0; b < nb; ++b) {
                blk_off[tid * nb + b] = run;
                run += blk_len[tid * nb + b];
            }
            const uint32_t bytes = rans ? align_up_u32(head + plane_bytes + run, 16u)
                                        : align_up_u32(head + plane_bytes + 4u * ((run + 31u) / 32u), 16u);
            s_flag[2 * tid] = bytes > fixed_bytes ? 1u : 0u;  // would not shrink: store fixed-width instead
            s_flag[2 * tid + 1] = bytes;
        }
        __syncthreads();
        for (int w = 0; w < 2; ++w) {
            if (s_flag[2 * w]) coder[w] = CF_B200_CODER_FIXED8;
            else bytes_out[w] = s_flag[2 * w + 1];
        }
    }
    for (uint32_t j = tid; j < 2u * nb; j += kSealThreads) {   // pass 2: tables and payload of the coded streams
        const uint32_t w = j / nb, b = j % nb;
        uint8_t *part = job[w].part;
        if (coder[w] == CF_B200_CODER_FIXED8) continue;
        if (rans) {
            reinterpret_cast<uint32_t *>(part)[b] = blk_state[j];
            reinterpret_cast<uint16_t *>(part + 4u * nb)[b] = static_cast<uint16_t>(blk_off[j]);
            const uint8_t *src = scratch + (j + 1) * lay.slot_bytes - blk_len[j];
            uint8_t *dst = part + head + plane_bytes + blk_off[j];
            for (uint32_t i = 0; i < blk_len[j]; ++i) dst[i] = src[i];
        } else {
            uint32_t *words = reinterpret_cast<uint32_t *>(part + head + plane_bytes);
            const uint32_t base = b * p.block_size;
            const int count = static_cast<int>(min(p.block_size, n - base) / per);
            const uint8_t *src = split ? job[w].pairs + base / 2u : job[w].sym + base;
            uint32_t bit = blk_off[j];
            reinterpret_cast<uint16_t *>(part)[b] = static_cast<uint16_t>(bit);
            for (int i = 0; i < count; ++i) {
                const uint32_t cl = job[w].tables->huff_code[src[i]];
                put_bits(words, bit, cl & 0xffffu, cl >> 16);
                bit += cl >> 16;
            }
        }
    }
    // (a split stream that fell back to fixed width: the fixed words below overwrite the plane its part already holds)
    for (int w = 0; w < 2; ++w) {
        if (coder[w] != CF_B200_CODER_FIXED8) continue;
        uint32_t *words = reinterpret_cast<uint32_t *>(job[w].part);
        for (uint32_t i = tid; i < (n + 3u) / 4u; i += kSealThreads) {
            uint32_t v = 0;
            for (uint32_t k = 0; k < 4; ++k) {
                const uint32_t at = 4u * i + k;
                if (at < n) v |= static_cast<uint32_t>(job[w].sym[at]) << (24u - 8u * k);
            }
            words[i] = v;
        }
    }
    __syncthreads();
    coder_out[0] = coder[0];
    coder_out[1] = coder[1];
}

__device__ __forceinline__ void quantise_tiles(const SealParams &p, uint64_t tile, uint32_t rows, float k_scale,
                                               float v_scale, uint8_t *ksym, uint8_t *vsym) {
    const uint32_t D = p.head_dim, T = p.page_tokens;
    for (uint32_t i = threadIdx.x; i < p.symbols; i += kSealThreads) {
        const uint32_t t = i / D, d = i % D;
        uint32_t ks = kZero, vs = kZero;
        if (t < rows) {
            ks = quantise_symbol(tile_value(p.tail_k, p.tail_type, tile + i), k_scale);
            vs = quantise_symbol(tile_value(p.tail_v, p.tail_type, tile + i), v_scale);
        }
        ksym[i] = static_cast<uint8_t>(ks);          // K order: token-major
        vsym[d * T + t] = static_cast<uint8_t>(vs);  // V order: token-minor
    }
}

__global__ void __launch_bounds__(kSealThreads) seal_pages_kernel(SealParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ float red[8];
    __shared__ uint32_t s_flag[4];
    __shared__ unsigned long long s_offset;
    const SealSmem lay = seal_smem(p.symbols, p.nblocks, p.block_size);
    uint8_t *ksym = smem + lay.off_ksym;
    uint8_t *vsym = smem + lay.off_vsym;
    uint8_t *scratch = smem + lay.off_scratch;
    uint8_t *k_part = smem + lay.off_part;
    uint8_t *v_part = k_part + lay.part_capacity;
    uint32_t *blk_len = reinterpret_cast<uint32_t *>(smem + lay.off_blk);   // [2 streams][nblocks] each
    uint32_t *blk_off = blk_len + 2u * p.nblocks;
    uint32_t *blk_state = blk_off + 2u * p.nblocks;
    uint2 *enc = reinterpret_cast<uint2 *>(smem + lay.off_enc);               // [2 streams][256 symbols]

    const uint32_t job = blockIdx.x, tid = threadIdx.x;
    const uint32_t kv_head = p.job_heads ? p.job_heads[job] : blockIdx.y;
    const uint32_t slot = p.job_slots[job];
    const uint32_t rows = p.job_tokens ? min(p.job_tokens[job], p.page_tokens) : p.page_tokens;
    const uint64_t tile = ((static_cast<uint64_t>(slot) * p.kv_head_count + kv_head) * p.tail_capacity +
                           (p.job_rows ? p.job_rows[job] : 0u)) * p.head_dim;

    int k_bad, v_bad;
    const float k_max = tile_absmax(p.tail_k, p.tail_type, tile, rows * p.head_dim, &k_bad, red);
    const float v_max = tile_absmax(p.tail_v, p.tail_type, tile, rows * p.head_dim, &v_bad, red);
    if (rows == 0 || k_bad || v_bad) {  // finite validation failed: nothing is published
        if (tid == 0 && p.status) atomicOr(p.status, CF_B200_DEVSTAT_NONFINITE);
        return;
    }
    const uint16_t k_bits = scale_bits_from_absmax(k_max), v_bits = scale_bits_from_absmax(v_max);
    quantise_tiles(p, tile, rows, __half2float(__ushort_as_half(k_bits)), __half2float(__ushort_as_half(v_bits)), ksym,
                   vsym);
    for (uint32_t i = tid; i < 2u * lay.part_capacity / 4u; i += kSealThreads) reinterpret_cast<uint32_t *>(k_part)[i] = 0u;
    if (rans_family(p.coder))
        for (uint32_t i = tid; i < 512u; i += kSealThreads) {
            const cf_b200_codebook_tables *t = i < 256u ? p.k_tables : p.v_tables;
            enc[i] = make_uint2(t->rans_enc[i & 255u][0], t->rans_enc[i & 255u][1]);
        }
    __syncthreads();

    const StreamJob jobs[2] = {{ksym, smem + lay.off_kpair, p.k_tables, enc, k_part},
                               {vsym, smem + lay.off_vpair, p.v_tables, enc + 256, v_part}};
    uint32_t coders[2], bytes[2];
    encode_streams(p, lay, jobs, scratch, blk_len, blk_off, blk_state, s_flag, coders, bytes);
    const uint32_t k_coder = coders[0], v_coder = coders[1], k_bytes = bytes[0], v_bytes = bytes[1];

    const uint32_t units = 1u + k_bytes / 16u + v_bytes / 16u;
    if (tid == 0) s_offset = atomicAdd(p.cursor, static_cast<unsigned long long>(units));
    __syncthreads();
    const unsigned long long offset = s_offset;
    if (offset + units > p.arena_units) {
        if (tid == 0 && p.status) atomicOr(p.status, CF_B200_DEVSTAT_ARENA_FULL);
        return;
    }
    uint4 *dst = reinterpret_cast<uint4 *>(p.arena + 16ull * offset);
    if (tid == 0) {
        cf_b200_record_header h;
        h.k_part_units = static_cast<uint16_t>(k_bytes / 16u);
        h.v_part_units = static_cast<uint16_t>(v_bytes / 16u);
        h.k_coder = static_cast<uint8_t>(k_coder);
        h.v_coder = static_cast<uint8_t>(v_coder);
        h.token_count = static_cast<uint16_t>(rows);
        h.k_scale_f16 = k_bits;
        h.v_scale_f16 = v_bits;
        h.codebook_id = static_cast<uint16_t>(p.codebook_id);
        h.flags = 0;
        h.version = CF_B200_FORMAT_VERSION;
        dst[0] = *reinterpret_cast<const uint4 *>(&h);
    }
    for (uint32_t i = tid; i < k_bytes / 16u; i += kSealThreads) dst[1 + i] = reinterpret_cast<const uint4 *>(k_part)[i];
    for (uint32_t i = tid; i < v_bytes / 16u; i += kSealThreads)
        dst[1 + k_bytes / 16u + i] = reinterpret_cast<const uint4 *>(v_part)[i];
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        p.page_dir[static_cast<uint64_t>(p.job_pages[job]) * p.kv_head_count + kv_head] = CF_B200_DIR_ENTRY(offset, units);
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The sealer for the geometry the lane-per-block attention kernel reads: head_dim 128, 16-token pages, 64-symbol
// blocks (32 blocks per stream). It writes the same records as seal_pages_kernel, byte for byte; what differs is
// that the geometry is known at compile time, so nothing is divided at run time and a value is loaded once:
//   * thread t owns the K symbols 16 t .. 16 t + 15 (token t / 8, sixteen channels: two 16-byte loads) and channel t
//     of V with all its tokens, which are sixteen consecutive symbols of the token-minor V stream: both streams
//     leave the quantiser as four packed words per thread, and the pair symbols and low-nibble plane words of the
//     nibble-split coders are made from those registers;
//   * warp w (0, 1) codes stream w, lane = block: block symbols read as words and indexed statically, block
//     lengths turned into offsets with a warp scan, bytes moved into the part — no barrier inside the coder;
//   * the encoder's division is a multiplication by the reciprocal the codebook carries (rans_enc of
//     cf_b200_codebook_tables): the update of src/cuda/rans.cu:20-22 run backwards is
//     x + cum + floor(x / f) * (4096 - f).
#ifndef CFB_SEAL_CTAS
#define CFB_SEAL_CTAS 8   // resident CTAs per SM the register budget is set for (64 registers per thread)
#endif
constexpr uint32_t kFastDim = 128, kFastTokens = 16, kFastBlock = 64, kFastSymbols = 2048, kFastBlocks = 32;
constexpr uint32_t kFastPart = 2064;   // a part never exceeds the fixed-width 2048 bytes; one unit of slack for the coders
constexpr uint32_t kFastSlot = 100;    // a block codes into at most 64 * 12 bits + the bytes the start state sheds

// Symbols w[0..kCount/4) (first symbol in byte 0 of w[0]) pushed last to first; bytes written backwards from slot_end.
template <int kCount>
__device__ __forceinline__ uint32_t fast_rans_encode(const uint32_t *w, const uint2 *enc, uint8_t *slot_end, uint32_t *state0) {
    uint32_t x = kRansL;
    uint8_t *p = slot_end;
#pragma unroll
    for (int j = kCount - 1; j >= 0; --j) {
        const uint2 e = enc[(w[j >> 2] >> (8 * (j & 3))) & 0xffu];
        const uint32_t cmpl = (e.y >> 13) & 0xfffu, x_max = (4096u - cmpl) << 19;
        if (x >= x_max) {   // the state is below 2^31 and x_max at least 2^19: two bytes at most
            *--p = static_cast<uint8_t>(x);
            x >>= 8;
            if (x >= x_max) {
                *--p = static_cast<uint8_t>(x);
                x >>= 8;
            }
        }
        x = x + (e.y & 0x1fffu) + (__umulhi(x, e.x) >> (e.y >> 25)) * cmpl;
    }
    *state0 = x;
    return static_cast<uint32_t>(slot_end - p);
}

template <int kCount>
__device__ __forceinline__ uint32_t fast_huffman_bits(const uint32_t *w, const uint2 *enc) {
    uint32_t bits = 0;
#pragma unroll
    for (int j = 0; j < kCount; ++j) bits += enc[(w[j >> 2] >> (8 * (j & 3))) & 0xffu].x >> 16;
    return bits;
}

// MSB-first codes of the block appended at bit `bit` of the zeroed word array. Only the first and the last word of a
// block can be shared with a neighbour; those are OR-ed in atomically, the words between are plain stores.
template <int kCount>
__device__ __forceinline__ void fast_huffman_emit(const uint32_t *w, const uint2 *enc, uint32_t *words, uint32_t bit) {
    uint32_t at = bit >> 5, filled = bit & 31u;
    unsigned long long acc = 0;
    bool first = true;
#pragma unroll
    for (int j = 0; j < kCount; ++j) {
        const uint32_t cl = enc[(w[j >> 2] >> (8 * (j & 3))) & 0xffu].x, len = cl >> 16;
        acc |= static_cast<unsigned long long>(cl & 0xffffu) << (64u - filled - len);
        filled += len;
        if (filled >= 32u) {
            const uint32_t word = static_cast<uint32_t>(acc >> 32);
            if (first) atomicOr(&words[at], word);
            else words[at] = word;
            first = false;
            ++at;
            acc <<= 32;
            filled -= 32u;
        }
    }
    if (filled) atomicOr(&words[at], static_cast<uint32_t>(acc >> 32));
}

// The coder of one stream, run by one warp (lane = block). Returns the part's size; *coder_out = the coder stored.
template <int kCount>
__device__ __forceinline__ uint32_t fast_code_stream(uint32_t coder, const uint8_t *src, const uint8_t *sym, const uint2 *enc,
                                                     uint8_t *part, uint8_t *slot_end, uint32_t lane, uint32_t *coder_out) {
    constexpr bool kSplit = kCount == 32;
    const bool rans = rans_family(coder);
    const uint32_t head = rans ? 6u * kFastBlocks : 2u * kFastBlocks, plane = kSplit ? 4u * 8u * kFastBlocks : 0u;
    uint32_t w[kCount / 4];
#pragma unroll
    for (int i = 0; i < kCount / 16; ++i) {
        const uint4 q = reinterpret_cast<const uint4 *>(src + kCount * lane)[i];
        w[4 * i] = q.x, w[4 * i + 1] = q.y, w[4 * i + 2] = q.z, w[4 * i + 3] = q.w;
    }
    uint32_t state = 0;
    const uint32_t len = rans ? fast_rans_encode<kCount>(w, enc, slot_end, &state) : fast_huffman_bits<kCount>(w, enc);
    uint32_t incl = len;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= static_cast<uint32_t>(d)) incl += t;
    }
    const uint32_t off = incl - len, run = __shfl_sync(0xffffffffu, incl, 31);
    const uint32_t bytes = align_up_u32(head + plane + (rans ? run : 4u * ((run + 31u) / 32u)), 16u);
    if (bytes > kFastSymbols) {   // would not shrink: fixed-width words, most significant byte first, over the whole part
        for (uint32_t i = lane; i < kFastSymbols / 4u; i += 32u)
            reinterpret_cast<uint32_t *>(part)[i] = __byte_perm(reinterpret_cast<const uint32_t *>(sym)[i], 0u, 0x0123);
        *coder_out = CF_B200_CODER_FIXED8;
        return kFastSymbols;
    }
    if (rans) {
        reinterpret_cast<uint32_t *>(part)[lane] = state;
        reinterpret_cast<uint16_t *>(part + 4u * kFastBlocks)[lane] = static_cast<uint16_t>(off);
        const uint8_t *from = slot_end - len;
        uint8_t *to = part + head + plane + off;
        for (uint32_t i = 0; i < len; ++i) to[i] = from[i];
    } else {
        reinterpret_cast<uint16_t *>(part)[lane] = static_cast<uint16_t>(off);
        fast_huffman_emit<kCount>(w, enc, reinterpret_cast<uint32_t *>(part + head + plane), off);
    }
    *coder_out = coder;
    return bytes;
}

template <bool kF32>
__global__ void __launch_bounds__(kSealThreads, CFB_SEAL_CTAS) seal_pages_fast_kernel(SealParams p) {
    __shared__ __align__(16) uint8_t s_sym[2][kFastSymbols];
    __shared__ __align__(16) uint8_t s_pair[2][kFastSymbols / 2];
    __shared__ __align__(16) uint8_t s_part[2][kFastPart];
    __shared__ __align__(8) uint2 s_enc[2][256];
    __shared__ __align__(4) uint8_t s_scratch[2 * kFastBlocks][kFastSlot];
    __shared__ uint32_t s_red[8], s_coder[2], s_bytes[2];
    __shared__ unsigned long long s_offset;
    using Scalar = typename std::conditional<kF32, float, __half>::type;

    const uint32_t job = blockIdx.x, tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t kv_head = p.job_heads ? p.job_heads[job] : blockIdx.y;
    const uint32_t slot = p.job_slots[job];
    const uint32_t rows = p.job_tokens ? min(p.job_tokens[job], kFastTokens) : kFastTokens;
    const uint64_t tile = ((static_cast<uint64_t>(slot) * p.kv_head_count + kv_head) * p.tail_capacity +
                           (p.job_rows ? p.job_rows[job] : 0u)) * kFastDim;
    const Scalar *tk = static_cast<const Scalar *>(p.tail_k) + tile, *tv = static_cast<const Scalar *>(p.tail_v) + tile;
    const bool split = split_coder(p.coder), rans = rans_family(p.coder);

    // values: K row-wise (sixteen channels of token tid / 8), V column-wise (channel tid, every token)
    float kf[16], vf[16];
    const bool k_live = (tid >> 3) < rows;
    if constexpr (kF32) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 q = k_live ? reinterpret_cast<const float4 *>(tk + 16u * tid)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            kf[4 * i] = q.x, kf[4 * i + 1] = q.y, kf[4 * i + 2] = q.z, kf[4 * i + 3] = q.w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint4 q = k_live ? reinterpret_cast<const uint4 *>(tk + 16u * tid)[i] : make_uint4(0u, 0u, 0u, 0u);
            const uint32_t h[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&h[j]));
                kf[8 * i + 2 * j] = f.x, kf[8 * i + 2 * j + 1] = f.y;
            }
        }
    }
#pragma unroll
    for (uint32_t t = 0; t < kFastTokens; ++t) {
        if constexpr (kF32) vf[t] = t < rows ? tv[t * kFastDim + tid] : 0.f;
        else vf[t] = t < rows ? __half2float(tv[t * kFastDim + tid]) : 0.f;
    }
    // absmax and the finite check at once: the magnitude bits of inf and NaN are above those of every finite value
    uint32_t km = 0u, vm = 0u;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        km = max(km, __float_as_uint(kf[i]) & 0x7fffffffu);
        vm = max(vm, __float_as_uint(vf[i]) & 0x7fffffffu);
    }
    km = __reduce_max_sync(0xffffffffu, km);
    vm = __reduce_max_sync(0xffffffffu, vm);
    if (lane == 0) {
        s_red[warp] = km;
        s_red[4 + warp] = vm;
    }
    for (uint32_t i = tid; i < 2u * kFastPart / 16u; i += kSealThreads) reinterpret_cast<uint4 *>(&s_part[0][0])[i] = make_uint4(0u, 0u, 0u, 0u);
    for (uint32_t i = tid; i < 512u; i += kSealThreads) {
        const cf_b200_codebook_tables *t = i < 256u ? p.k_tables : p.v_tables;
        (&s_enc[0][0])[i] = rans ? make_uint2(t->rans_enc[i & 255u][0], t->rans_enc[i & 255u][1]) : make_uint2(t->huff_code[i & 255u], 0u);
    }
    __syncthreads();
    km = max(max(s_red[0], s_red[1]), max(s_red[2], s_red[3]));
    vm = max(max(s_red[4], s_red[5]), max(s_red[6], s_red[7]));
    if (rows == 0 || km >= 0x7f800000u || vm >= 0x7f800000u) {  // finite validation failed: nothing is published
        if (tid == 0 && p.status) atomicOr(p.status, CF_B200_DEVSTAT_NONFINITE);
        return;
    }
    const uint16_t k_bits = scale_bits_from_absmax(__uint_as_float(km)), v_bits = scale_bits_from_absmax(__uint_as_float(vm));
    const float k_scale = __half2float(__ushort_as_half(k_bits)), v_scale = __half2float(__ushort_as_half(v_bits));
    const float k_rcp = __frcp_rn(k_scale), v_rcp = __frcp_rn(v_scale);
    uint32_t kw[4], vw[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t a = 0u, b = 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            a |= (k_live ? quantise_symbol_rcp(kf[4 * i + j], k_scale, k_rcp) : static_cast<uint32_t>(kZero)) << (8 * j);
            b |= (static_cast<uint32_t>(4 * i + j) < rows ? quantise_symbol_rcp(vf[4 * i + j], v_scale, v_rcp) : static_cast<uint32_t>(kZero)) << (8 * j);
        }
        kw[i] = a, vw[i] = b;
    }
    reinterpret_cast<uint4 *>(&s_sym[0][0])[tid] = make_uint4(kw[0], kw[1], kw[2], kw[3]);
    reinterpret_cast<uint4 *>(&s_sym[1][0])[tid] = make_uint4(vw[0], vw[1], vw[2], vw[3]);
    if (split) {
        // pair symbol = hi(s[2k]) << 4 | hi(s[2k+1]): with h = w & 0xf0f0f0f0, bytes 0 and 2 of h | h >> 12
        // plane word = low nibbles of eight symbols: first four in the low nibbles of the bytes, next four in the high ones
        const uint32_t head = rans ? 6u * kFastBlocks : 2u * kFastBlocks, b = tid >> 2, j0 = 2u * (tid & 3u);
#pragma unroll
        for (int s2 = 0; s2 < 2; ++s2) {
            const uint32_t *w = s2 ? vw : kw;
            uint32_t t[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t h = w[i] & 0xf0f0f0f0u;
                t[i] = h | (h >> 12);
            }
            reinterpret_cast<uint2 *>(&s_pair[s2][0])[tid] = make_uint2(__byte_perm(t[0], t[1], 0x6420), __byte_perm(t[2], t[3], 0x6420));
            uint32_t *plane = reinterpret_cast<uint32_t *>(&s_part[s2][head]);
            plane[j0 * kFastBlocks + b] = (w[0] & 0x0f0f0f0fu) | ((w[1] & 0x0f0f0f0fu) << 4);
            plane[(j0 + 1u) * kFastBlocks + b] = (w[2] & 0x0f0f0f0fu) | ((w[3] & 0x0f0f0f0fu) << 4);
        }
    }
    __syncthreads();

    if (warp < 2u) {
        uint32_t coder = p.coder, bytes = kFastSymbols;
        uint8_t *slot_end = &s_scratch[warp * kFastBlocks + lane][kFastSlot];
        if (p.coder == CF_B200_CODER_FIXED8) {
            for (uint32_t i = lane; i < kFastSymbols / 4u; i += 32u)
                reinterpret_cast<uint32_t *>(&s_part[warp][0])[i] = __byte_perm(reinterpret_cast<const uint32_t *>(&s_sym[warp][0])[i], 0u, 0x0123);
        } else if (split) {
            bytes = fast_code_stream<32>(p.coder, &s_pair[warp][0], &s_sym[warp][0], &s_enc[warp][0], &s_part[warp][0], slot_end, lane, &coder);
        } else {
            bytes = fast_code_stream<64>(p.coder, &s_sym[warp][0], &s_sym[warp][0], &s_enc[warp][0], &s_part[warp][0], slot_end, lane, &coder);
        }
        if (lane == 0) {
            s_coder[warp] = coder;
            s_bytes[warp] = bytes;
        }
    }
    __syncthreads();
    const uint32_t k_bytes = s_bytes[0], v_bytes = s_bytes[1];
    const uint32_t units = 1u + k_bytes / 16u + v_bytes / 16u;
    if (tid == 0) s_offset = atomicAdd(p.cursor, static_cast<unsigned long long>(units));
    __syncthreads();
    const unsigned long long offset = s_offset;
    if (offset + units > p.arena_units) {
        if (tid == 0 && p.status) atomicOr(p.status, CF_B200_DEVSTAT_ARENA_FULL);
        return;
    }
    uint4 *dst = reinterpret_cast<uint4 *>(p.arena + 16ull * offset);
    if (tid == 0) {
        cf_b200_record_header h;
        h.k_part_units = static_cast<uint16_t>(k_bytes / 16u);
        h.v_part_units = static_cast<uint16_t>(v_bytes / 16u);
        h.k_coder = static_cast<uint8_t>(s_coder[0]);
        h.v_coder = static_cast<uint8_t>(s_coder[1]);
        h.token_count = static_cast<uint16_t>(rows);
        h.k_scale_f16 = k_bits;
        h.v_scale_f16 = v_bits;
        h.codebook_id = static_cast<uint16_t>(p.codebook_id);
        h.flags = 0;
        h.version = CF_B200_FORMAT_VERSION;
        dst[0] = *reinterpret_cast<const uint4 *>(&h);
    }
    for (uint32_t i = tid; i < k_bytes / 16u; i += kSealThreads) dst[1 + i] = reinterpret_cast<const uint4 *>(&s_part[0][0])[i];
    for (uint32_t i = tid; i < v_bytes / 16u; i += kSealThreads)
        dst[1 + k_bytes / 16u + i] = reinterpret_cast<const uint4 *>(&s_part[1][0])[i];
    __threadfence();
    __syncthreads();
    if (tid == 0) p.page_dir[static_cast<uint64_t>(p.job_pages[job]) * p.kv_head_count + kv_head] = CF_B200_DIR_ENTRY(offset, units);
}

__global__ void __launch_bounds__(kSealThreads) histogram_kernel(SealParams p, unsigned long long *hist_k,
                                                                 unsigned long long *hist_v) {
    __shared__ float red[8];
    __shared__ uint32_t hk[256], hv[256];
    const uint32_t job = blockIdx.x, tid = threadIdx.x;
    const uint32_t kv_head = p.job_heads ? p.job_heads[job] : blockIdx.y;
    const uint32_t slot = p.job_slots[job];
    const uint32_t rows = p.job_tokens ? min(p.job_tokens[job], p.page_tokens) : p.page_tokens;
    const uint64_t tile = ((static_cast<uint64_t>(slot) * p.kv_head_count + kv_head) * p.tail_capacity +
                           (p.job_rows ? p.job_rows[job] : 0u)) * p.head_dim;
    for (uint32_t i = tid; i < 256; i += kSealThreads) hk[i] = hv[i] = 0;
    int k_bad, v_bad;
    const float k_max = tile_absmax(p.tail_k, p.tail_type, tile, rows * p.head_dim, &k_bad, red);
    const float v_max = tile_absmax(p.tail_v, p.tail_type, tile, rows * p.head_dim, &v_bad, red);
    if (rows == 0 || k_bad || v_bad) return;
    const float ks = __half2float(__ushort_as_half(scale_bits_from_absmax(k_max)));
    const float vs = __half2float(__ushort_as_half(scale_bits_from_absmax(v_max)));
    if (split_coder(p.coder)) {   // the symbols these coders code: hi(s[2k]) << 4 | hi(s[2k+1]) in stream order
        const uint32_t D = p.head_dim, T = p.page_tokens;
        auto k_sym = [&](uint32_t t, uint32_t d) {
            return t < rows ? quantise_symbol(tile_value(p.tail_k, p.tail_type, tile + t * D + d), ks) : static_cast<uint32_t>(kZero);
        };
        auto v_sym = [&](uint32_t t, uint32_t d) {
            return t < rows ? quantise_symbol(tile_value(p.tail_v, p.tail_type, tile + t * D + d), vs) : static_cast<uint32_t>(kZero);
        };
        for (uint32_t i = tid; i < p.symbols / 2u; i += kSealThreads) {
            const uint32_t kt = (2u * i) / D, kd = (2u * i) % D;        // K stream: token-major
            atomicAdd(&hk[(k_sym(kt, kd) & 0xf0u) | (k_sym((2u * i + 1u) / D, (2u * i + 1u) % D) >> 4)], 1u);
            const uint32_t vd = (2u * i) / T, vt = (2u * i) % T;        // V stream: token-minor
            atomicAdd(&hv[(v_sym(vt, vd) & 0xf0u) | (v_sym((2u * i + 1u) % T, (2u * i + 1u) / T) >> 4)], 1u);
        }
    } else {
        for (uint32_t i = tid; i < rows * p.head_dim; i += kSealThreads) {
            atomicAdd(&hk[quantise_symbol(tile_value(p.tail_k, p.tail_type, tile + i), ks)], 1u);
            atomicAdd(&hv[quantise_symbol(tile_value(p.tail_v, p.tail_type, tile + i), vs)], 1u);
        }
    }
    __syncthreads();
    for (uint32_t i = tid; i < 256; i += kSealThreads) {
        if (hk[i]) atomicAdd(&hist_k[i], static_cast<unsigned long long>(hk[i]));
        if (hv[i]) atomicAdd(&hist_v[i], static_cast<unsigned long long>(hv[i]));
    }
}

void fill(const cf_b200_seal_desc *d, SealParams *p) {
    p->kv_head_count = d->kv_head_count;
    p->head_dim = d->head_dim;
    p->page_tokens = d->page_tokens;
    p->block_size = d->block_size;
    p->coder = d->coder;
    p->codebook_id = d->codebook_id;
    p->symbols = d->head_dim * d->page_tokens;
    p->nblocks = (p->symbols + d->block_size - 1) / d->block_size;
    p->k_tables = d->k_tables;
    p->v_tables = d->v_tables;
    p->tail_k = d->tail_k;
    p->tail_v = d->tail_v;
    p->tail_type = d->tail_type == CF_B200_F32 ? CF_B200_F32 : CF_B200_F16;
    p->job_slots = d->job_slots;
    p->job_pages = d->job_pages;
    p->job_tokens = d->job_tokens;
    p->job_heads = d->job_heads;
    p->job_rows = d->job_rows;
    p->tail_capacity = d->tail_capacity ? d->tail_capacity : d->page_tokens;
    p->arena = d->arena;
    p->arena_units = d->arena_units;
    p->cursor = d->arena_cursor_units;
    p->page_dir = d->page_dir;
    p->status = d->status;
}

cf_status validate_common(const cf_b200_seal_desc *d) {
    if (d == nullptr || d->struct_size != sizeof(cf_b200_seal_desc) || d->abi_version != CF_B200_ABI_VERSION)
        return CF_ERR_INVALID_ARGUMENT;
    if (d->kv_head_count == 0 || d->head_dim == 0 || d->page_tokens == 0 || d->block_size == 0 ||
        d->tail_k == nullptr || d->tail_v == nullptr || (d->job_count != 0 && d->job_slots == nullptr))
        return CF_ERR_INVALID_ARGUMENT;
    if (d->head_dim > CF_KV_MAX_HEAD_DIM || d->head_dim * d->page_tokens > CF_B200_MAX_STREAM_SYMBOLS ||
        d->block_size < 16 || d->block_size > 1024 || d->kv_head_count > 65535u)
        return CF_ERR_UNSUPPORTED;
    return CF_OK;
}

}  // namespace
}  // namespace cfb

extern "C" cf_status cf_b200_seal_validate(const cf_b200_seal_desc *d) {
    const cf_status s = cfb::validate_common(d);
    if (s != CF_OK) return s;
    if (d->coder > CF_B200_CODER_MAX || d->codebook_id > 65535u || d->k_tables == nullptr || d->v_tables == nullptr ||
        d->arena == nullptr || d->arena_cursor_units == nullptr || d->page_dir == nullptr ||
        (d->job_count != 0 && d->job_pages == nullptr) || (reinterpret_cast<uintptr_t>(d->arena) & 15u) != 0 ||
        d->arena_units >= (1ull << 40))
        return CF_ERR_INVALID_ARGUMENT;
    if (cfb::split_coder(d->coder) && (d->block_size % 8u != 0 || (d->head_dim * d->page_tokens) % 8u != 0))
        return CF_ERR_UNSUPPORTED;   // the raw low-nibble plane is cut into words of eight symbols
    return CF_OK;
}

extern "C" cf_status cf_b200_seal_pages_async(const cf_b200_seal_desc *d, void *stream) {
    const cf_status s = cf_b200_seal_validate(d);
    if (s != CF_OK) return s;
    if (d->job_count == 0) return CF_OK;
    if (!cfb::on_current_device(d->arena) || !cfb::on_current_device(d->tail_k) || !cfb::on_current_device(d->page_dir))
        return CF_ERR_INVALID_ARGUMENT;   // memory of another GPU: the call must be made with that GPU current
    cfb::SealParams p;
    cfb::fill(d, &p);
    if (d->head_dim == cfb::kFastDim && d->page_tokens == cfb::kFastTokens && d->block_size == cfb::kFastBlock &&
        ((reinterpret_cast<uintptr_t>(d->tail_k) | reinterpret_cast<uintptr_t>(d->tail_v)) & 15u) == 0) {
        const dim3 grid(d->job_count, d->job_heads ? 1u : d->kv_head_count);
        if (p.tail_type == CF_B200_F32) cfb::seal_pages_fast_kernel<true><<<grid, cfb::kSealThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
        else cfb::seal_pages_fast_kernel<false><<<grid, cfb::kSealThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
        return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
    }
    const cfb::SealSmem lay = cfb::seal_smem(p.symbols, p.nblocks, p.block_size);
    if (cudaFuncSetAttribute(cfb::seal_pages_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(lay.total)) != cudaSuccess)
        return CF_ERR_CUDA;
    cfb::seal_pages_kernel<<<dim3(d->job_count, d->job_heads ? 1u : d->kv_head_count), cfb::kSealThreads, lay.total,
                             static_cast<cudaStream_t>(stream)>>>(p);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}

namespace cfb {
namespace {

// One block per row: the K and V rows of a token go to position tail_tokens[slot] of the slot's tails.
__global__ void __launch_bounds__(128) append_rows_kernel(cf_b200_append_desc d) {
    const uint32_t row = blockIdx.x, slot = d.slots[row];
    const uint32_t at = d.tail_tokens[slot];
    if (at >= d.tail_capacity) {
        if (threadIdx.x == 0 && d.status) atomicOr(d.status, CF_B200_DEVSTAT_TAIL_FULL);
        return;
    }
    const uint32_t values = d.kv_head_count * d.head_dim;
    for (uint32_t i = threadIdx.x; i < values; i += blockDim.x) {
        const uint32_t head = i / d.head_dim, dim = i % d.head_dim;
        const uint64_t src = static_cast<uint64_t>(row) * values + i;
        const uint64_t dst = ((static_cast<uint64_t>(slot) * d.kv_head_count + head) * d.tail_capacity + at) * d.head_dim + dim;
        float k, v;
        if (d.row_type == CF_B200_BF16) {
            k = __bfloat162float(static_cast<const __nv_bfloat16 *>(d.k_rows)[src]);
            v = __bfloat162float(static_cast<const __nv_bfloat16 *>(d.v_rows)[src]);
        } else {
            k = tile_value(d.k_rows, d.row_type, src);
            v = tile_value(d.v_rows, d.row_type, src);
        }
        if (d.tail_type == CF_B200_F32) {
            static_cast<float *>(d.tail_k)[dst] = k;
            static_cast<float *>(d.tail_v)[dst] = v;
        } else {
            static_cast<__half *>(d.tail_k)[dst] = __float2half_rn(k);
            static_cast<__half *>(d.tail_v)[dst] = __float2half_rn(v);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) d.tail_tokens[slot] = at + 1u;
}

}  // namespace
}  // namespace cfb

extern "C" cf_status cf_b200_append_rows_async(const cf_b200_append_desc *d, void *stream) {
    if (d == nullptr || d->struct_size != sizeof(cf_b200_append_desc) || d->abi_version != CF_B200_ABI_VERSION ||
        d->kv_head_count == 0 || d->head_dim == 0 || d->tail_capacity == 0 || d->tail_k == nullptr || d->tail_v == nullptr ||
        d->tail_tokens == nullptr || (d->row_count != 0 && (d->slots == nullptr || d->k_rows == nullptr || d->v_rows == nullptr)) ||
        (d->row_type != CF_B200_F16 && d->row_type != CF_B200_F32 && d->row_type != CF_B200_BF16))
        return CF_ERR_INVALID_ARGUMENT;
    if (d->row_count == 0) return CF_OK;
    if (!cfb::on_current_device(d->tail_k) || !cfb::on_current_device(d->k_rows) || !cfb::on_current_device(d->tail_tokens))
        return CF_ERR_INVALID_ARGUMENT;   // memory of another GPU: the call must be made with that GPU current
    cf_b200_append_desc local = *d;
    local.tail_type = d->tail_type == CF_B200_F32 ? CF_B200_F32 : CF_B200_F16;
    cfb::append_rows_kernel<<<d->row_count, 128, 0, static_cast<cudaStream_t>(stream)>>>(local);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}

extern "C" cf_status cf_b200_histogram_async(const cf_b200_seal_desc *d, unsigned long long *hist_k,
                                             unsigned long long *hist_v, void *stream) {
    const cf_status s = cfb::validate_common(d);
    if (s != CF_OK) return s;
    if (hist_k == nullptr || hist_v == nullptr) return CF_ERR_INVALID_ARGUMENT;
    if (d->job_count == 0) return CF_OK;
    if (!cfb::on_current_device(d->tail_k) || !cfb::on_current_device(hist_k)) return CF_ERR_INVALID_ARGUMENT;
    cfb::SealParams p;
    cfb::fill(d, &p);
    cfb::histogram_kernel<<<dim3(d->job_count, d->job_heads ? 1u : d->kv_head_count), cfb::kSealThreads, 0,
                            static_cast<cudaStream_t>(stream)>>>(p, hist_k, hist_v);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}
