// cf_oracle.cpp — CPU restatement of the reference's sealed-KV arithmetic. TEST INFRASTRUCTURE ONLY:
// it is the checker the CUDA path is compared with and the timed CPU baseline; nothing in the product
// links, imports or calls it.
//
// Each function names the reference lines it restates (paths inside the reference project).
//
// Pinning status:
//   * fixed-width decode, Huffman LUT decode, KIVI quantiser, double-precision online softmax, merge
//     and paged attention are checked against the reference's own compiled sources (oracle/_ref) and
//     against golden vectors generated from them (tests/golden).
//   * the rANS decoder is a restatement of src/cuda/rans.cu:16-26; that file needs a CUDA compiler, so
//     on a GPU it is additionally checked against the reference's own kernel built into oracle/_ref.
//   * the rANS and Huffman ENCODERS have no counterpart in the reference tree (they live in an
//     out-of-tree Python module with no pinned version, tools/export_rans.py:27-29). They are written
//     here as exact inverses of the decoders; the choice of start state (L) and of the frequency
//     normalisation rule is this project's. Bitstream parity with that module: PARITY UNPINNED.
//     Decode parity (decode(encode(x)) == x through the restated reference decoders) is exact.
//   * the per-stream fp16 absmax quantiser is the layout the benchmark configuration names; the
//     reference has no such quantiser, so it follows kv_gpu_fixture.cpp:12-16 (lrint, clamp, +zp) with
//     one scale per stream.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <queue>
#include <thread>
#include <vector>

#include "chromofold_b200/sealed_page_format.h"

namespace {

constexpr uint32_t kM = CF_B200_RANS_M;
constexpr uint32_t kL = CF_B200_RANS_L;

// ---- binary16 <-> float (round to nearest even), no hardware dependency --------------------------
float half_to_float(uint16_t h) {
    const uint32_t sign = (h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            bits = sign | ((127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 112) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

uint16_t float_to_half(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return static_cast<uint16_t>(sign | 0x7c00u | ((x > 0x7f800000u) ? 0x200u : 0u));
    if (x >= 0x477ff000u) return static_cast<uint16_t>(sign | 0x7c00u);  // rounds to inf
    if (x < 0x33000001u) return static_cast<uint16_t>(sign);              // rounds to zero
    if (x < 0x38800000u) {                                                // subnormal half
        const uint32_t shift = 126 - (x >> 23);
        const uint32_t man = (x & 0x7fffffu) | 0x800000u;
        uint32_t h = man >> shift;
        const uint32_t rem = man & ((1u << shift) - 1u);
        const uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (h & 1u))) ++h;
        return static_cast<uint16_t>(sign | h);
    }
    uint32_t h = ((x >> 13) - (112u << 10));
    const uint32_t rem = x & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return static_cast<uint16_t>(sign | h);
}

// ---- decoders (restatements) ----------------------------------------------------------------------

// src/cuda/rans.cu:16-26 — slot lookup, state update, 8-bit renormalisation.
void rans_decode_block(const uint8_t *data, int pos, uint32_t state, const int32_t *slot2sym,
                       const int32_t *freq, const int32_t *cum, int cnt, int32_t *out) {
    for (int j = 0; j < cnt; ++j) {
        const int slot = static_cast<int>(state & (kM - 1));
        const int s = slot2sym[slot];
        state = static_cast<uint32_t>(freq[s]) * (state >> CF_B200_RANS_PROB_BITS) +
                static_cast<uint32_t>(slot - cum[s]);
        while (state < kL) {
            state = (state << 8) | static_cast<uint32_t>(data[pos]);
            ++pos;
        }
        out[j] = s;
    }
}

// include/chromofold/detail/block_huffman_device.cuh:12-19 — maxlen bits MSB-first, one LUT hit.
int bh_decode_at(const uint32_t *words, const int32_t *lut, int maxlen, int pos) {
    int look = 0;
    for (int k = 0; k < maxlen; ++k) {
        const int wpos = pos + k;
        look = (look << 1) | static_cast<int>((words[wpos >> 5] >> (31 - (wpos & 31))) & 1u);
    }
    return lut[look];
}

// ---- codebook construction (this project's rule; see header) --------------------------------------

// Frequencies normalised to M = 4096 with freq >= 1 for all 256 symbols:
//   f_i = 1 + floor(h_i * 3840 / N); the remaining slots go to the largest remainders
//   (h_i * 3840) mod N, ties to the lower symbol. N == 0 gives the uniform table.
void build_rans_tables(const uint64_t *hist, int32_t *freq, int32_t *cum, int32_t *slot2sym) {
    uint64_t total = 0;
    for (int i = 0; i < 256; ++i) total += hist[i];
    if (total == 0) {
        for (int i = 0; i < 256; ++i) freq[i] = 16;
    } else {
        const uint64_t budget = kM - 256;
        std::vector<std::pair<uint64_t, int>> rem(256);
        uint64_t used = 0;
        for (int i = 0; i < 256; ++i) {
            const unsigned __int128 scaled = static_cast<unsigned __int128>(hist[i]) * budget;
            const uint64_t q = static_cast<uint64_t>(scaled / total);
            rem[i] = {static_cast<uint64_t>(scaled % total), i};
            freq[i] = 1 + static_cast<int32_t>(q);
            used += q;
        }
        uint64_t left = budget - used;
        std::stable_sort(rem.begin(), rem.end(), [](const auto &a, const auto &b) {
            if (a.first != b.first) return a.first > b.first;
            return a.second < b.second;
        });
        for (uint64_t k = 0; k < left; ++k) freq[rem[k % 256].second] += 1;
    }
    int32_t running = 0;
    for (int i = 0; i < 256; ++i) {
        cum[i] = running;
        for (int32_t k = 0; k < freq[i]; ++k) slot2sym[running + k] = i;
        running += freq[i];
    }
}

// Length-limited canonical Huffman code for 256 symbols, max length 12.
//   weights w_i = 2*h_i + 1 (every symbol stays codable);
//   plain Huffman lengths; lengths above 12 are cut to 12; while the Kraft sum exceeds 2^12 the
//   lightest symbol with len < 12 (ties: higher symbol) is lengthened; then, heaviest first (ties:
//   lower symbol), symbols are shortened while the sum allows it.
//   Canonical assignment in (len, symbol) order, first code all zeros, codes read MSB-first.
void build_huffman(const uint64_t *hist, uint8_t *len, uint32_t *code, int32_t *lut) {
    constexpr int kMax = CF_B200_HUFF_MAXLEN;
    struct Node { uint64_t w; int left, right; };
    std::vector<Node> nodes;
    nodes.reserve(511);
    using Item = std::pair<uint64_t, int>;  // weight, node id (ties: lower id first)
    std::priority_queue<Item, std::vector<Item>, std::greater<Item>> heap;
    for (int i = 0; i < 256; ++i) {
        nodes.push_back({2 * hist[i] + 1, -1, -1});
        heap.push({nodes.back().w, i});
    }
    while (heap.size() > 1) {
        const Item a = heap.top(); heap.pop();
        const Item b = heap.top(); heap.pop();
        nodes.push_back({a.first + b.first, a.second, b.second});
        heap.push({a.first + b.first, static_cast<int>(nodes.size()) - 1});
    }
    std::vector<int> depth(nodes.size(), 0);
    for (int n = static_cast<int>(nodes.size()) - 1; n >= 256; --n) {
        depth[nodes[n].left] = depth[n] + 1;
        depth[nodes[n].right] = depth[n] + 1;
    }
    for (int i = 0; i < 256; ++i) len[i] = static_cast<uint8_t>(std::min(depth[i], kMax));

    auto kraft = [&]() {
        uint64_t k = 0;
        for (int i = 0; i < 256; ++i) k += 1ull << (kMax - len[i]);
        return k;
    };
    uint64_t k = kraft();
    const uint64_t cap = 1ull << kMax;
    std::vector<int> light(256), heavy(256);
    for (int i = 0; i < 256; ++i) light[i] = heavy[i] = i;
    std::stable_sort(light.begin(), light.end(), [&](int a, int b) {
        if (hist[a] != hist[b]) return hist[a] < hist[b];
        return a > b;
    });
    std::stable_sort(heavy.begin(), heavy.end(), [&](int a, int b) {
        if (hist[a] != hist[b]) return hist[a] > hist[b];
        return a < b;
    });
    while (k > cap) {
        for (int idx : light) {
            if (len[idx] < kMax) {
                k -= 1ull << (kMax - len[idx] - 1);
                len[idx] += 1;
                break;
            }
        }
    }
    bool changed = true;
    while (changed) {
        changed = false;
        for (int idx : heavy) {
            if (len[idx] > 1 && k + (1ull << (kMax - len[idx])) <= cap) {
                k += 1ull << (kMax - len[idx]);
                len[idx] -= 1;
                changed = true;
            }
        }
    }
    std::vector<int> order(256);
    for (int i = 0; i < 256; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) {
        if (len[a] != len[b]) return len[a] < len[b];
        return a < b;
    });
    uint32_t next = 0;
    int prev_len = len[order[0]];
    for (int i = 0; i < (1 << kMax); ++i) lut[i] = 0;
    for (int idx : order) {
        next <<= (len[idx] - prev_len);
        prev_len = len[idx];
        code[idx] = next;
        const uint32_t first = next << (kMax - len[idx]);
        const uint32_t span = 1u << (kMax - len[idx]);
        for (uint32_t e = 0; e < span; ++e) lut[first + e] = idx | (static_cast<int32_t>(len[idx]) << 8);
        next += 1;
    }
}

// ---- encoders (exact inverses of the decoders above) ----------------------------------------------

// Inverse of rans_decode_block: symbols are pushed last to first starting from state L; bytes leave the
// low end of the state, so the emitted sequence is reversed at the end and the decoder's forward reads
// (state << 8 | byte) undo them. Returns the start state; appends the block's bytes to `out`.
uint32_t rans_encode_block(const uint8_t *sym, int cnt, const int32_t *freq, const int32_t *cum,
                           std::vector<uint8_t> *out) {
    uint32_t x = kL;
    std::vector<uint8_t> rev;
    for (int j = cnt - 1; j >= 0; --j) {
        const uint32_t f = static_cast<uint32_t>(freq[sym[j]]);
        const uint64_t x_max = (static_cast<uint64_t>(kL >> CF_B200_RANS_PROB_BITS) << 8) * f;
        while (x >= x_max) {
            rev.push_back(static_cast<uint8_t>(x & 0xffu));
            x >>= 8;
        }
        x = ((x / f) << CF_B200_RANS_PROB_BITS) + (x % f) + static_cast<uint32_t>(cum[sym[j]]);
    }
    out->insert(out->end(), rev.rbegin(), rev.rend());
    return x;
}

struct BitWriter {
    std::vector<uint32_t> words;
    uint32_t bits = 0;
    void put(uint32_t code, uint32_t len) {  // MSB-first, kv_gpu_fixture.cpp:36-40 generalised to any length
        for (int b = static_cast<int>(len) - 1; b >= 0; --b) {
            if ((bits & 31u) == 0) words.push_back(0u);
            if ((code >> b) & 1u) words.back() |= 1u << (31 - (bits & 31u));
            ++bits;
        }
    }
};

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Geometry {
    uint32_t head_dim, page_tokens, block_size;
    uint32_t symbols() const { return head_dim * page_tokens; }
    uint32_t nblocks() const { return (symbols() + block_size - 1) / block_size; }
};

bool is_split(uint32_t coder) { return coder == CF_B200_CODER_RANS_SPLIT4 || coder == CF_B200_CODER_HUFFMAN_SPLIT4; }

// Nibble-split coders (sealed_page_format.h): pair symbols and the raw low-nibble plane of a stream.
void split_symbols(const uint8_t *sym, const Geometry &g, std::vector<uint8_t> *pairs, std::vector<uint32_t> *plane) {
    const uint32_t n = g.symbols(), nb = g.nblocks(), words_per_block = g.block_size / 8;
    pairs->assign(n / 2, 0);
    plane->assign(static_cast<size_t>(words_per_block) * nb, 0u);
    for (uint32_t i = 0; i < n; i += 2) (*pairs)[i / 2] = static_cast<uint8_t>((sym[i] & 0xf0u) | (sym[i + 1] >> 4));
    for (uint32_t i = 0; i < n; ++i) {
        const uint32_t b = i / g.block_size, r = i % g.block_size, j = r / 8, at = r % 8;
        const uint32_t shift = at < 4 ? 8 * at : 8 * (at - 4) + 4;
        (*plane)[static_cast<size_t>(j) * nb + b] |= static_cast<uint32_t>(sym[i] & 0x0fu) << shift;
    }
}
uint8_t plane_nibble(const uint32_t *plane, const Geometry &g, uint32_t i) {
    const uint32_t b = i / g.block_size, r = i % g.block_size, j = r / 8, at = r % 8;
    const uint32_t shift = at < 4 ? 8 * at : 8 * (at - 4) + 4;
    return static_cast<uint8_t>((plane[static_cast<size_t>(j) * g.nblocks() + b] >> shift) & 0x0fu);
}

// The block table and the payload of one plain coded stream (RANS / HUFFMAN / FIXED8) over `n` symbols.
void encode_stream(const uint8_t *sym, uint32_t n, uint32_t block_size, uint32_t coder, const int32_t *freq, const int32_t *cum,
                   const uint8_t *hlen, const uint32_t *hcode, std::vector<uint8_t> *table, std::vector<uint8_t> *payload) {
    const uint32_t nb = (n + block_size - 1) / block_size;
    table->clear();
    payload->clear();
    if (coder == CF_B200_CODER_RANS) {
        std::vector<uint32_t> state0(nb);
        std::vector<uint16_t> off(nb);
        for (uint32_t b = 0; b < nb; ++b) {
            const uint32_t base = b * block_size;
            const int cnt = static_cast<int>(std::min(block_size, n - base));
            off[b] = static_cast<uint16_t>(payload->size());
            state0[b] = rans_encode_block(sym + base, cnt, freq, cum, payload);
        }
        table->assign(align_up(nb * 4 + nb * 2, 4), 0);
        std::memcpy(table->data(), state0.data(), nb * 4);
        std::memcpy(table->data() + nb * 4, off.data(), nb * 2);
    } else if (coder == CF_B200_CODER_HUFFMAN) {
        std::vector<uint16_t> off(nb);
        BitWriter w;
        for (uint32_t i = 0; i < n; ++i) {
            if (i % block_size == 0) off[i / block_size] = static_cast<uint16_t>(w.bits);
            w.put(hcode[sym[i]], hlen[sym[i]]);
        }
        table->assign(align_up(nb * 2, 4), 0);
        std::memcpy(table->data(), off.data(), nb * 2);
        payload->assign(w.words.size() * 4, 0);
        std::memcpy(payload->data(), w.words.data(), payload->size());
    } else {
        BitWriter w;
        for (uint32_t i = 0; i < n; ++i) w.put(sym[i], 8);
        payload->assign(w.words.size() * 4, 0);
        std::memcpy(payload->data(), w.words.data(), payload->size());
    }
}

// One stream part in the record layout of sealed_page_format.h: table | (raw low-nibble plane) | payload | pad to 16.
void encode_part(const uint8_t *sym, const Geometry &g, uint32_t coder, const int32_t *freq, const int32_t *cum,
                 const uint8_t *hlen, const uint32_t *hcode, std::vector<uint8_t> *part) {
    std::vector<uint8_t> table, payload, pairs;
    std::vector<uint32_t> plane;
    if (is_split(coder)) {   // the pair symbols go through the plain coder with half the block size
        split_symbols(sym, g, &pairs, &plane);
        encode_stream(pairs.data(), g.symbols() / 2, g.block_size / 2,
                      coder == CF_B200_CODER_RANS_SPLIT4 ? CF_B200_CODER_RANS : CF_B200_CODER_HUFFMAN, freq, cum, hlen, hcode,
                      &table, &payload);
    } else {
        encode_stream(sym, g.symbols(), g.block_size, coder, freq, cum, hlen, hcode, &table, &payload);
    }
    part->assign(align_up(table.size() + plane.size() * 4 + payload.size(), 16), 0);
    std::memcpy(part->data(), table.data(), table.size());
    if (!plane.empty()) std::memcpy(part->data() + table.size(), plane.data(), plane.size() * 4);
    if (!payload.empty()) std::memcpy(part->data() + table.size() + plane.size() * 4, payload.data(), payload.size());
}

// A plain coded stream back to its `n` symbols: `table` and `payload` as encode_stream laid them out.
void decode_stream(const uint8_t *table, const uint8_t *payload, uint32_t n, uint32_t block_size, uint32_t coder,
                   const int32_t *slot2sym, const int32_t *freq, const int32_t *cum, const int32_t *lut, uint8_t *sym) {
    const uint32_t nb = (n + block_size - 1) / block_size;
    if (coder == CF_B200_CODER_RANS) {
        const uint32_t *state0 = reinterpret_cast<const uint32_t *>(table);
        const uint16_t *off = reinterpret_cast<const uint16_t *>(table + nb * 4);
        std::vector<int32_t> tmp(block_size);
        for (uint32_t b = 0; b < nb; ++b) {  // rans.cu:28-36, one block per loop turn
            const uint32_t base = b * block_size;
            const int cnt = static_cast<int>(std::min(block_size, n - base));
            rans_decode_block(payload, off[b], state0[b], slot2sym, freq, cum, cnt, tmp.data());
            for (int j = 0; j < cnt; ++j) sym[base + j] = static_cast<uint8_t>(tmp[j]);
        }
    } else if (coder == CF_B200_CODER_HUFFMAN) {
        const uint16_t *off = reinterpret_cast<const uint16_t *>(table);
        const uint32_t *words = reinterpret_cast<const uint32_t *>(payload);
        for (uint32_t b = 0; b < nb; ++b) {
            const uint32_t base = b * block_size;
            const uint32_t cnt = std::min(block_size, n - base);
            int pos = off[b];
            for (uint32_t j = 0; j < cnt; ++j) {  // paged_kv_attention.cu:101-106 walk
                const int sl = bh_decode_at(words, lut, CF_B200_HUFF_MAXLEN, pos);
                sym[base + j] = static_cast<uint8_t>(sl & 0xff);
                pos += sl >> 8;
            }
        }
    } else {
        const uint32_t *words = reinterpret_cast<const uint32_t *>(payload);
        for (uint32_t i = 0; i < n; ++i) {  // kv_gpu_fixture.cpp:110-116 at 8 bits
            const uint32_t bit = i * 8;
            sym[i] = static_cast<uint8_t>((words[bit >> 5] >> (24 - (bit & 31u))) & 0xffu);
        }
    }
}

void decode_part(const uint8_t *part, const Geometry &g, uint32_t coder, const int32_t *slot2sym,
                 const int32_t *freq, const int32_t *cum, const int32_t *lut, uint8_t *sym) {
    const uint32_t n = g.symbols(), nb = g.nblocks();
    if (is_split(coder)) {   // the pair symbols through the restated reference decoder, then the nibbles put together
        const bool rans = coder == CF_B200_CODER_RANS_SPLIT4;
        const size_t table = align_up(rans ? nb * 6 : nb * 2, 4), plane_bytes = static_cast<size_t>(g.block_size / 8) * nb * 4;
        std::vector<uint8_t> pairs(n / 2);
        decode_stream(part, part + table + plane_bytes, n / 2, g.block_size / 2, rans ? CF_B200_CODER_RANS : CF_B200_CODER_HUFFMAN,
                      slot2sym, freq, cum, lut, pairs.data());
        const uint32_t *plane = reinterpret_cast<const uint32_t *>(part + table);
        for (uint32_t i = 0; i < n; i += 2) {
            sym[i] = static_cast<uint8_t>((pairs[i / 2] & 0xf0u) | plane_nibble(plane, g, i));
            sym[i + 1] = static_cast<uint8_t>(((pairs[i / 2] & 0x0fu) << 4) | plane_nibble(plane, g, i + 1));
        }
        return;
    }
    const size_t table = coder == CF_B200_CODER_RANS ? align_up(nb * 6, 4) : coder == CF_B200_CODER_HUFFMAN ? align_up(nb * 2, 4) : 0;
    decode_stream(part, part + table, n, g.block_size, coder, slot2sym, freq, cum, lut, sym);
}

// kv_gpu_fixture.cpp:12-16 with one scale per stream: scale = absmax/127 stored as binary16 (1.0 when
// the stream is all zero, :70), code = clamp(lrint(x / scale), -128, 127), symbol = code + 128.
// Returns false when a value is not finite (kv_gpu_fixture.cpp:13).
bool quantize_stream(const float *x, uint32_t count, uint16_t *scale_bits, int8_t *codes) {
    float maximum = 0.0f;
    for (uint32_t i = 0; i < count; ++i) {
        if (!std::isfinite(x[i])) return false;
        maximum = std::max(maximum, std::fabs(x[i]));
    }
    uint16_t bits = maximum == 0.0f ? 0x3c00u : float_to_half(maximum / 127.0f);
    if (bits == 0) bits = 1;              // absmax so small that the scale rounds to zero
    if ((bits & 0x7c00u) == 0x7c00u) bits = 0x7bffu;
    const float scale = half_to_float(bits);
    for (uint32_t i = 0; i < count; ++i) {
        const long r = std::lrint(x[i] / scale);
        codes[i] = static_cast<int8_t>(std::clamp(r, -128l, 127l));
    }
    *scale_bits = bits;
    return true;
}

}  // namespace

extern "C" {

float orc_half_to_float(uint16_t h) { return half_to_float(h); }
uint16_t orc_float_to_half(float f) { return float_to_half(f); }

void orc_rans_decode(const uint8_t *data, const int32_t *byte_off, const uint32_t *state0,
                     const int32_t *slot2sym, const int32_t *freq, const int32_t *cum, int block, int n,
                     int32_t *out) {
    const int nblocks = (n + block - 1) / block;
    for (int b = 0; b < nblocks; ++b) {
        const int base = b * block;
        rans_decode_block(data, byte_off[b], state0[b], slot2sym, freq, cum, std::min(block, n - base), out + base);
    }
}

int orc_bh_decode_at(const uint32_t *words, const int32_t *lut, int maxlen, int pos) {
    return bh_decode_at(words, lut, maxlen, pos);
}

void orc_build_rans_tables(const uint64_t *hist, int32_t *freq, int32_t *cum, int32_t *slot2sym) {
    build_rans_tables(hist, freq, cum, slot2sym);
}

void orc_build_huffman(const uint64_t *hist, uint8_t *len, uint32_t *code, int32_t *lut) {
    build_huffman(hist, len, code, lut);
}

// Flat block-rANS stream in the layout of tools/export_rans.py:13-17 (data | byte_off | state0).
// Returns the number of data bytes written (capacity must be >= 2*n + 8).
int64_t orc_rans_encode(const uint8_t *sym, int n, int block, const int32_t *freq, const int32_t *cum,
                        uint8_t *data, int32_t *byte_off, uint32_t *state0) {
    std::vector<uint8_t> payload;
    const int nblocks = (n + block - 1) / block;
    for (int b = 0; b < nblocks; ++b) {
        const int base = b * block;
        byte_off[b] = static_cast<int32_t>(payload.size());
        state0[b] = rans_encode_block(sym + base, std::min(block, n - base), freq, cum, &payload);
    }
    std::memcpy(data, payload.data(), payload.size());
    return static_cast<int64_t>(payload.size());
}

// Block-Huffman stream in the layout of kv_gpu_fixture.hpp:11-18 (words, block bit offsets).
int64_t orc_huff_encode(const uint8_t *sym, int n, int block, const uint8_t *len, const uint32_t *code,
                        uint32_t *words, int32_t *block_offsets) {
    BitWriter w;
    for (int i = 0; i < n; ++i) {
        if (i % block == 0) block_offsets[i / block] = static_cast<int32_t>(w.bits);
        w.put(code[sym[i]], len[sym[i]]);
    }
    w.words.push_back(0u);  // the 12-bit look-ahead of the last symbol may touch one more word
    std::memcpy(words, w.words.data(), w.words.size() * 4);
    return static_cast<int64_t>(w.words.size());
}

void orc_huff_decode(const uint32_t *words, const int32_t *block_offsets, const int32_t *lut, int maxlen,
                     int block, int n, uint8_t *out) {
    for (int b = 0; b * block < n; ++b) {
        int pos = block_offsets[b];
        for (int j = 0; j < block && b * block + j < n; ++j) {
            const int sl = bh_decode_at(words, lut, maxlen, pos);
            out[b * block + j] = static_cast<uint8_t>(sl & 0xff);
            pos += sl >> 8;
        }
    }
}

int orc_quantize_stream(const float *x, uint32_t count, uint16_t *scale_bits, int8_t *codes) {
    return quantize_stream(x, count, scale_bits, codes) ? 0 : 1;
}

struct orc_codebook {
    int32_t freq[256], cum[256], slot2sym[4096];
    uint8_t hlen[256];
    uint32_t hcode[256];
    int32_t lut[4096];
};

void orc_codebook_build(const uint64_t *hist, orc_codebook *cb) {
    build_rans_tables(hist, cb->freq, cb->cum, cb->slot2sym);
    build_huffman(hist, cb->hlen, cb->hcode, cb->lut);
}

// Seal one (page, kv_head) into a format-v1 record.
//   k, v: float [page_tokens][head_dim] (only the first token_count rows are read).
//   coder: requested coder for both streams; a stream whose coded part would be larger than the
//   fixed-width part is stored fixed-width instead.
// Returns the record size in bytes, 0 if a value is not finite. `record` needs 2*(n + 6*nblocks) + 64.
// Optionally returns the symbols (k_sym in K order, v_sym in V order) for bit-exactness checks.
uint32_t orc_seal_record(const float *k, const float *v, uint32_t token_count, uint32_t head_dim,
                         uint32_t page_tokens, uint32_t block_size, uint32_t coder, uint32_t codebook_id,
                         const orc_codebook *kcb, const orc_codebook *vcb, uint8_t *record, uint8_t *k_sym_out,
                         uint8_t *v_sym_out) {
    const Geometry g{head_dim, page_tokens, block_size};
    const uint32_t n = g.symbols();
    std::vector<int8_t> kc(token_count * head_dim), vc(token_count * head_dim);
    uint16_t ks = 0, vs = 0;
    if (!quantize_stream(k, token_count * head_dim, &ks, kc.data())) return 0;
    if (!quantize_stream(v, token_count * head_dim, &vs, vc.data())) return 0;
    std::vector<uint8_t> ksym(n, CF_B200_ZERO_POINT), vsym(n, CF_B200_ZERO_POINT);
    for (uint32_t t = 0; t < token_count; ++t) {
        for (uint32_t d = 0; d < head_dim; ++d) {
            ksym[t * head_dim + d] = static_cast<uint8_t>(kc[t * head_dim + d] + CF_B200_ZERO_POINT);
            vsym[d * page_tokens + t] = static_cast<uint8_t>(vc[t * head_dim + d] + CF_B200_ZERO_POINT);
        }
    }
    std::vector<uint8_t> kp, vp, fixed;
    uint32_t kcoder = coder, vcoder = coder;
    encode_part(ksym.data(), g, coder, kcb->freq, kcb->cum, kcb->hlen, kcb->hcode, &kp);
    if (coder != CF_B200_CODER_FIXED8 && kp.size() > align_up(n, 16)) {
        kcoder = CF_B200_CODER_FIXED8;
        encode_part(ksym.data(), g, kcoder, nullptr, nullptr, nullptr, nullptr, &kp);
    }
    encode_part(vsym.data(), g, coder, vcb->freq, vcb->cum, vcb->hlen, vcb->hcode, &vp);
    if (coder != CF_B200_CODER_FIXED8 && vp.size() > align_up(n, 16)) {
        vcoder = CF_B200_CODER_FIXED8;
        encode_part(vsym.data(), g, vcoder, nullptr, nullptr, nullptr, nullptr, &vp);
    }
    cf_b200_record_header h{};
    h.k_part_units = static_cast<uint16_t>(kp.size() / 16);
    h.v_part_units = static_cast<uint16_t>(vp.size() / 16);
    h.k_coder = static_cast<uint8_t>(kcoder);
    h.v_coder = static_cast<uint8_t>(vcoder);
    h.token_count = static_cast<uint16_t>(token_count);
    h.k_scale_f16 = ks;
    h.v_scale_f16 = vs;
    h.codebook_id = static_cast<uint16_t>(codebook_id);
    h.flags = 0;
    h.version = CF_B200_FORMAT_VERSION;
    std::memcpy(record, &h, sizeof h);
    std::memcpy(record + 16, kp.data(), kp.size());
    std::memcpy(record + 16 + kp.size(), vp.data(), vp.size());
    if (k_sym_out) std::memcpy(k_sym_out, ksym.data(), n);
    if (v_sym_out) std::memcpy(v_sym_out, vsym.data(), n);
    return static_cast<uint32_t>(16 + kp.size() + vp.size());
}

// Encode given symbols (already in stream order) into a record; used for synthetic code distributions.
uint32_t orc_seal_record_symbols(const uint8_t *k_sym, const uint8_t *v_sym, uint16_t k_scale_bits,
                                 uint16_t v_scale_bits, uint32_t token_count, uint32_t head_dim,
                                 uint32_t page_tokens, uint32_t block_size, uint32_t coder, uint32_t codebook_id,
                                 const orc_codebook *kcb, const orc_codebook *vcb, uint8_t *record) {
    const Geometry g{head_dim, page_tokens, block_size};
    const uint32_t n = g.symbols();
    std::vector<uint8_t> kp, vp;
    uint32_t kcoder = coder, vcoder = coder;
    encode_part(k_sym, g, coder, kcb->freq, kcb->cum, kcb->hlen, kcb->hcode, &kp);
    if (coder != CF_B200_CODER_FIXED8 && kp.size() > align_up(n, 16)) {
        kcoder = CF_B200_CODER_FIXED8;
        encode_part(k_sym, g, kcoder, nullptr, nullptr, nullptr, nullptr, &kp);
    }
    encode_part(v_sym, g, coder, vcb->freq, vcb->cum, vcb->hlen, vcb->hcode, &vp);
    if (coder != CF_B200_CODER_FIXED8 && vp.size() > align_up(n, 16)) {
        vcoder = CF_B200_CODER_FIXED8;
        encode_part(v_sym, g, vcoder, nullptr, nullptr, nullptr, nullptr, &vp);
    }
    cf_b200_record_header h{};
    h.k_part_units = static_cast<uint16_t>(kp.size() / 16);
    h.v_part_units = static_cast<uint16_t>(vp.size() / 16);
    h.k_coder = static_cast<uint8_t>(kcoder);
    h.v_coder = static_cast<uint8_t>(vcoder);
    h.token_count = static_cast<uint16_t>(token_count);
    h.k_scale_f16 = k_scale_bits;
    h.v_scale_f16 = v_scale_bits;
    h.codebook_id = static_cast<uint16_t>(codebook_id);
    h.version = CF_B200_FORMAT_VERSION;
    std::memcpy(record, &h, sizeof h);
    std::memcpy(record + 16, kp.data(), kp.size());
    std::memcpy(record + 16 + kp.size(), vp.data(), vp.size());
    return static_cast<uint32_t>(16 + kp.size() + vp.size());
}

// Decode a record back to symbols (K order / V order) through the restated reference decoders.
int orc_open_record(const uint8_t *record, uint32_t head_dim, uint32_t page_tokens, uint32_t block_size,
                    const orc_codebook *kcb, const orc_codebook *vcb, uint8_t *k_sym, uint8_t *v_sym) {
    cf_b200_record_header h;
    std::memcpy(&h, record, sizeof h);
    if (h.version != CF_B200_FORMAT_VERSION) return 1;
    const Geometry g{head_dim, page_tokens, block_size};
    decode_part(record + 16, g, h.k_coder, kcb->slot2sym, kcb->freq, kcb->cum, kcb->lut, k_sym);
    decode_part(record + 16 + 16 * static_cast<size_t>(h.k_part_units), g, h.v_coder, vcb->slot2sym, vcb->freq,
                vcb->cum, vcb->lut, v_sym);
    return 0;
}

// ---- attention ------------------------------------------------------------------------------------

// src/runtime/kv_reference.cpp:50-67 — double-precision online softmax state.
struct OnlineState {
    double maximum = -std::numeric_limits<double>::infinity();
    double denominator = 0.0;
    double weighted[CF_B200_MAX_STREAM_SYMBOLS / 16];
    uint32_t dim;
    explicit OnlineState(uint32_t d) : dim(d) { for (uint32_t i = 0; i < d; ++i) weighted[i] = 0.0; }
    void add(double score, const float *value) {
        const double next_max = std::max(maximum, score);
        const double old_scale = denominator == 0.0 ? 0.0 : std::exp(maximum - next_max);
        const double new_scale = std::exp(score - next_max);
        denominator = denominator * old_scale + new_scale;
        for (uint32_t d = 0; d < dim; ++d) weighted[d] = weighted[d] * old_scale + static_cast<double>(value[d]) * new_scale;
        maximum = next_max;
    }
};

// kv_reference.cpp:164-243 over dense (dequantised) rows: keys/values are float
// [kv_head_count][token_count][head_dim] holding tokens token_begin.., queries
// [query_count][query_head_count][head_dim]. GQA map qh*Hkv/Hq (:69-72), visible tokens
// earliest <= t <= query_token (:197-199,206). Returns 1 if a query sees no token (:235).
int orc_dense_attention(const float *keys, const float *values, uint32_t token_begin, uint32_t token_count,
                        const float *queries, uint32_t query_count, uint32_t query_head_count,
                        uint32_t kv_head_count, uint32_t head_dim, uint32_t query_token_begin,
                        uint32_t causal_window, float score_scale, float *output) {
    if (head_dim > CF_B200_MAX_STREAM_SYMBOLS / 16) return 2;
    for (uint32_t q = 0; q < query_count; ++q) {
        const uint32_t query_token = query_token_begin + q;
        const uint32_t earliest = causal_window == 0 || query_token + 1u <= causal_window ? 0u : query_token + 1u - causal_window;
        for (uint32_t qh = 0; qh < query_head_count; ++qh) {
            const uint32_t kvh = static_cast<uint32_t>((static_cast<uint64_t>(qh) * kv_head_count) / query_head_count);
            const float *query = queries + (static_cast<size_t>(q) * query_head_count + qh) * head_dim;
            OnlineState state(head_dim);
            for (uint32_t t = 0; t < token_count; ++t) {
                const uint32_t token = token_begin + t;
                if (token < earliest || token > query_token) continue;
                const float *key = keys + (static_cast<size_t>(kvh) * token_count + t) * head_dim;
                double dot = 0.0;
                for (uint32_t d = 0; d < head_dim; ++d) dot += static_cast<double>(query[d]) * key[d];
                state.add(dot * score_scale, values + (static_cast<size_t>(kvh) * token_count + t) * head_dim);
            }
            if (state.denominator == 0.0) return 1;
            float *dst = output + (static_cast<size_t>(q) * query_head_count + qh) * head_dim;
            for (uint32_t d = 0; d < head_dim; ++d) dst[d] = static_cast<float>(state.weighted[d] / state.denominator);
        }
    }
    return 0;
}

// Decode-step attention of a batch straight from sealed records — the whole CPU path the GPU kernel
// replaces: decode (restated reference decoders) -> dequantise (paged_kv_attention.cu:222) -> double
// online softmax (kv_reference.cpp:195-240). One query token per sequence, placed after its context.
//   arena            : bytes holding all records
//   dir_offset       : [page_id * kv_head_count + kv_head] byte offset of the record in arena
//   page_table       : [seq][table_stride] page ids
//   seq_tokens       : [seq] sealed context length
//   tail_k / tail_v  : optional binary16 [seq][kv_head][page_tokens][head_dim] unsealed rows,
//   tail_count       : [seq] number of valid tail rows (may be null)
//   queries          : binary16 bits [seq][query_head_count][head_dim]
// Work is split over (sequence, kv_head) units across `threads` host threads.
int orc_sealed_decode_attention(const uint8_t *arena, const uint64_t *dir_offset, const uint32_t *page_table,
                                uint32_t table_stride, const uint32_t *seq_tokens, uint32_t seq_count,
                                const uint16_t *tail_k, const uint16_t *tail_v, const uint32_t *tail_count,
                                const uint16_t *queries, uint32_t query_head_count, uint32_t kv_head_count,
                                uint32_t head_dim, uint32_t page_tokens, uint32_t block_size, uint32_t causal_window,
                                float score_scale, const orc_codebook *kcb, const orc_codebook *vcb,
                                uint32_t threads, float *output) {
    if (head_dim > CF_B200_MAX_STREAM_SYMBOLS / 16 || query_head_count % kv_head_count != 0) return 2;
    const uint32_t group = query_head_count / kv_head_count;
    const uint32_t units = seq_count * kv_head_count;
    std::atomic<uint32_t> next{0};
    std::atomic<int> status{0};
    auto worker = [&]() {
        const uint32_t n = head_dim * page_tokens;
        std::vector<uint8_t> ksym(n), vsym(n);
        std::vector<float> krow(head_dim), vrow(head_dim), q(static_cast<size_t>(group) * head_dim);
        for (;;) {
            const uint32_t u = next.fetch_add(1);
            if (u >= units) break;
            const uint32_t s = u / kv_head_count, kvh = u % kv_head_count;
            const uint32_t tail = tail_count ? tail_count[s] : 0;
            const uint32_t query_token = seq_tokens[s] + tail;
            const uint32_t earliest = causal_window == 0 || query_token + 1u <= causal_window ? 0u : query_token + 1u - causal_window;
            std::vector<OnlineState> state(group, OnlineState(head_dim));
            for (uint32_t g = 0; g < group; ++g)
                for (uint32_t d = 0; d < head_dim; ++d)
                    q[g * head_dim + d] = half_to_float(queries[(static_cast<size_t>(s) * query_head_count + kvh * group + g) * head_dim + d]);
            auto consume = [&](uint32_t token, const float *key, const float *value) {
                if (token < earliest || token > query_token) return;
                for (uint32_t g = 0; g < group; ++g) {
                    double dot = 0.0;
                    for (uint32_t d = 0; d < head_dim; ++d) dot += static_cast<double>(q[g * head_dim + d]) * key[d];
                    state[g].add(dot * score_scale, value);
                }
            };
            const uint32_t pages = (seq_tokens[s] + page_tokens - 1) / page_tokens;
            for (uint32_t p = 0; p < pages; ++p) {
                const uint32_t page_id = page_table[static_cast<size_t>(s) * table_stride + p];
                const uint8_t *record = arena + dir_offset[static_cast<size_t>(page_id) * kv_head_count + kvh];
                cf_b200_record_header h;
                std::memcpy(&h, record, sizeof h);
                if (orc_open_record(record, head_dim, page_tokens, block_size, kcb, vcb, ksym.data(), vsym.data())) {
                    status = 3;
                    return;
                }
                const float kscale = half_to_float(h.k_scale_f16), vscale = half_to_float(h.v_scale_f16);
                for (uint32_t t = 0; t < h.token_count; ++t) {
                    for (uint32_t d = 0; d < head_dim; ++d) {
                        krow[d] = static_cast<float>(static_cast<int>(ksym[t * head_dim + d]) - CF_B200_ZERO_POINT) * kscale;
                        vrow[d] = static_cast<float>(static_cast<int>(vsym[d * page_tokens + t]) - CF_B200_ZERO_POINT) * vscale;
                    }
                    consume(p * page_tokens + t, krow.data(), vrow.data());
                }
            }
            for (uint32_t t = 0; t < tail; ++t) {
                const size_t base = ((static_cast<size_t>(s) * kv_head_count + kvh) * page_tokens + t) * head_dim;
                for (uint32_t d = 0; d < head_dim; ++d) {
                    krow[d] = half_to_float(tail_k[base + d]);
                    vrow[d] = half_to_float(tail_v[base + d]);
                }
                consume(seq_tokens[s] + t, krow.data(), vrow.data());
            }
            for (uint32_t g = 0; g < group; ++g) {
                float *dst = output + (static_cast<size_t>(s) * query_head_count + kvh * group + g) * head_dim;
                if (state[g].denominator == 0.0) {
                    for (uint32_t d = 0; d < head_dim; ++d) dst[d] = 0.0f;  // paged_kv_attention.cu:170-173
                } else {
                    for (uint32_t d = 0; d < head_dim; ++d) dst[d] = static_cast<float>(state[g].weighted[d] / state[g].denominator);
                }
            }
        }
    };
    const uint32_t nthreads = std::max(1u, std::min(threads, units));
    std::vector<std::thread> pool;
    for (uint32_t i = 1; i < nthreads; ++i) pool.emplace_back(worker);
    worker();
    for (auto &t : pool) t.join();
    return status.load();
}

// src/runtime/kv_runtime.cpp:179-253 — accumulate / merge / finalize restated on plain arrays.
void orc_online_merge(double *dst_max, double *dst_sum, double *dst_weighted, int *dst_init, double src_max,
                      double src_sum, const double *src_weighted, int src_init, uint32_t dim) {
    if (!src_init) return;
    if (!*dst_init) {
        *dst_max = src_max;
        *dst_sum = src_sum;
        *dst_init = 1;
        std::memcpy(dst_weighted, src_weighted, sizeof(double) * dim);
        return;
    }
    const double next_max = std::max(src_max, *dst_max);
    const double dst_scale = std::exp(*dst_max - next_max);
    const double src_scale = std::exp(src_max - next_max);
    *dst_sum = *dst_sum * dst_scale + src_sum * src_scale;
    for (uint32_t d = 0; d < dim; ++d) dst_weighted[d] = dst_weighted[d] * dst_scale + src_weighted[d] * src_scale;
    *dst_max = next_max;
}

unsigned orc_hardware_threads() { return std::max(1u, std::thread::hardware_concurrency()); }

}  // extern "C"
