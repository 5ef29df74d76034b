// seal.cu — GPU page sealer: quantise, entropy-code and publish full pages in one launch.
//
// The reference seals on the device in six launches with a host synchronisation in the middle and one allocation
// per array (src/cuda/device_kv_seal_attention.cu:244-334: finite_scan, quantize_int4, pack_nibbles, then a host
// side table upload) and only produces fixed-width nibbles. Here one CTA owns one (page, kv head): it scans for
// non-finite values, derives the two stream scales, quantises (round-half-even, clamp, +zero point —
// src/runtime/kv_gpu_fixture.cpp:12-16), codes both streams block by block with the exact inverse of the decoders in
// cf_device_common.cuh, takes room in the arena with one atomic add, writes the record and only then the directory
// entry, so a reader never sees a half-written page and the host is not involved.

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

// Per-symbol encoder entry in shared memory: x = freq | cum << 12 | shift << 24, y = ceil(2^(31 + shift) / freq) with
// shift = ceil(log2 freq). Then floor(v / freq) = (v * y) >> (31 + shift) exactly for every v < 2^31, so the encoder
// needs no division.
__device__ __forceinline__ uint2 encoder_entry(uint32_t freq, uint32_t cum) {
    const uint32_t shift = freq > 1u ? 32u - static_cast<uint32_t>(__clz(freq - 1u)) : 0u;
    const unsigned long long rcp = ((1ull << (31u + shift)) + freq - 1u) / freq;
    return make_uint2(freq | (cum << 12) | (shift << 24), static_cast<uint32_t>(rcp));
}

// Inverse of rans_decode_block: symbols pushed last to first from state L; bytes leave the low end of the state
// and are written backwards so that they read forwards. Returns the byte count; *state0 gets the final state.
__device__ uint32_t rans_encode_block(const uint8_t *sym, int count, const uint2 *enc, uint8_t *slot_end, uint32_t *state0) {
    uint32_t x = kRansL;
    uint8_t *p = slot_end;
    for (int j = count - 1; j >= 0; --j) {
        const uint2 e = enc[sym[j]];
        const uint32_t f = e.x & 0xfffu, cum = (e.x >> 12) & 0xfffu, shift = e.x >> 24;
        const uint32_t x_max = f << 19;  // ((L >> 12) << 8) * f
        while (x >= x_max) {
            *--p = static_cast<uint8_t>(x & 0xffu);
            x >>= 8;
        }
        const uint32_t q = static_cast<uint32_t>((static_cast<unsigned long long>(x) * e.y) >> (31u + shift));
        x = (q << CF_B200_RANS_PROB_BITS) + (x - q * f) + cum;
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
            enc[i] = encoder_entry(t->rans_freq[i & 255u], t->rans_cum[i & 255u]);
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
    const cfb::SealSmem lay = cfb::seal_smem(p.symbols, p.nblocks, p.block_size);
    if (cudaFuncSetAttribute(cfb::seal_pages_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(lay.total)) != cudaSuccess)
        return CF_ERR_CUDA;
    cfb::seal_pages_kernel<<<dim3(d->job_count, d->job_heads ? 1u : d->kv_head_count), cfb::kSealThreads, lay.total,
                             static_cast<cudaStream_t>(stream)>>>(p);
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
