// codebook.cpp — host-side construction of the shared coding tables (set-up work, outside the query path).
//
// The reference keeps a LUT per page and has no table builder in-tree (its exporters import one from an
// out-of-tree module, tools/export_rans.py:27-29); the decode side fixes what a table must look like:
//   rANS   : frequencies sum to M = 4096, slot -> symbol, state' = freq*(state>>12) + slot - cum
//            (src/cuda/rans.cu:11-13,20-22)
//   Huffman: canonical codes, at most maxlen bits, LUT entry sym | len<<8 for every maxlen-bit prefix
//            (include/chromofold/detail/block_huffman_device.cuh:10-19)
// The normalisation and length-limiting rules below are this library's own and are stated in sealed_kv.h.

#include <algorithm>
#include <array>
#include <cstring>
#include <numeric>
#include <vector>

#include "chromofold_b200/sealed_kv.h"

namespace {

constexpr int kSymbols = 256;
constexpr uint32_t kSlots = CF_B200_RANS_M;
constexpr int kMaxLen = CF_B200_HUFF_MAXLEN;

void normalise_frequencies(const uint64_t *hist, std::array<uint32_t, kSymbols> &freq) {
    const uint64_t total = std::accumulate(hist, hist + kSymbols, uint64_t{0});
    if (total == 0) {
        freq.fill(kSlots / kSymbols);
        return;
    }
    const uint64_t spare = kSlots - kSymbols;  // slots left after every symbol got one
    std::array<uint64_t, kSymbols> remainder{};
    uint64_t handed = 0;
    for (int s = 0; s < kSymbols; ++s) {
        const unsigned __int128 share = static_cast<unsigned __int128>(hist[s]) * spare;
        freq[s] = 1u + static_cast<uint32_t>(share / total);
        remainder[s] = static_cast<uint64_t>(share % total);
        handed += freq[s] - 1u;
    }
    std::array<int, kSymbols> by_remainder;
    std::iota(by_remainder.begin(), by_remainder.end(), 0);
    std::stable_sort(by_remainder.begin(), by_remainder.end(),
                     [&](int a, int b) { return remainder[a] > remainder[b]; });  // stable: ties keep the lower symbol first
    for (uint64_t extra = spare - handed, i = 0; extra > 0; --extra, ++i) freq[by_remainder[i % kSymbols]] += 1u;
}

// Optimal prefix-code lengths by repeatedly joining the two lightest trees (ties: the older tree first).
void huffman_lengths(const uint64_t *hist, std::array<int, kSymbols> &length) {
    struct Tree { uint64_t weight; int id; };
    std::array<uint64_t, 2 * kSymbols> weight{};
    std::array<int, 2 * kSymbols> parent{};
    std::vector<Tree> live;
    live.reserve(kSymbols);
    for (int s = 0; s < kSymbols; ++s) {
        weight[s] = 2 * hist[s] + 1;
        live.push_back({weight[s], s});
    }
    auto heavier = [](const Tree &a, const Tree &b) { return a.weight != b.weight ? a.weight > b.weight : a.id > b.id; };
    std::make_heap(live.begin(), live.end(), heavier);
    int next = kSymbols;
    while (live.size() > 1) {
        std::pop_heap(live.begin(), live.end(), heavier);
        const Tree a = live.back();
        live.pop_back();
        std::pop_heap(live.begin(), live.end(), heavier);
        const Tree b = live.back();
        live.pop_back();
        weight[next] = a.weight + b.weight;
        parent[a.id] = parent[b.id] = next;
        live.push_back({weight[next], next});
        std::push_heap(live.begin(), live.end(), heavier);
        ++next;
    }
    const int root = next - 1;
    for (int s = 0; s < kSymbols; ++s) {
        int depth = 0;
        for (int n = s; n != root; n = parent[n]) ++depth;
        length[s] = depth;
    }
}

void limit_lengths(const uint64_t *hist, std::array<int, kSymbols> &length) {
    const uint64_t full = uint64_t{1} << kMaxLen;
    uint64_t kraft = 0;
    for (int s = 0; s < kSymbols; ++s) {
        length[s] = std::min(length[s], kMaxLen);
        kraft += full >> length[s];
    }
    std::array<int, kSymbols> lightest, heaviest;
    std::iota(lightest.begin(), lightest.end(), 0);
    heaviest = lightest;
    std::stable_sort(lightest.begin(), lightest.end(),
                     [&](int a, int b) { return hist[a] != hist[b] ? hist[a] < hist[b] : a > b; });
    std::stable_sort(heaviest.begin(), heaviest.end(),
                     [&](int a, int b) { return hist[a] != hist[b] ? hist[a] > hist[b] : a < b; });
    while (kraft > full) {  // over-subscribed after the cut: lengthen the lightest symbol that still can grow
        for (int s : lightest) {
            if (length[s] < kMaxLen) {
                kraft -= full >> (length[s] + 1);
                ++length[s];
                break;
            }
        }
    }
    for (bool again = true; again;) {  // hand unused code space back to the heaviest symbols
        again = false;
        for (int s : heaviest) {
            if (length[s] > 1 && kraft + (full >> length[s]) <= full) {
                kraft += full >> length[s];
                --length[s];
                again = true;
            }
        }
    }
}

}  // namespace

extern "C" cf_status cf_b200_codebook_build(const uint64_t histogram[256], cf_b200_codebook_tables *out) {
    if (histogram == nullptr || out == nullptr) return CF_ERR_INVALID_ARGUMENT;
    std::memset(out, 0, sizeof *out);

    std::array<uint32_t, kSymbols> freq;
    normalise_frequencies(histogram, freq);
    uint32_t start = 0;
    for (int s = 0; s < kSymbols; ++s) {
        out->rans_freq[s] = static_cast<uint16_t>(freq[s]);
        out->rans_cum[s] = static_cast<uint16_t>(start);
        for (uint32_t k = 0; k < freq[s]; ++k)
            out->rans_slot[start + k] = static_cast<uint32_t>(s) | (freq[s] << 8) | (k << 20);
        // the sealer's side: division by freq as a multiplication (sealed_page_format.h)
        if (freq[s] < 2u) {
            out->rans_enc[s][0] = 0xffffffffu;
            out->rans_enc[s][1] = (start + 4095u) | (4095u << 13);
        } else {
            uint32_t shift = 0;
            while ((1u << shift) < freq[s]) ++shift;
            out->rans_enc[s][0] = static_cast<uint32_t>(((1ull << (31u + shift)) + freq[s] - 1u) / freq[s]);
            out->rans_enc[s][1] = start | ((4096u - freq[s]) << 13) | ((shift - 1u) << 25);
        }
        start += freq[s];
    }
    if (start != kSlots) return CF_ERR_UNSUPPORTED;

    std::array<int, kSymbols> length;
    huffman_lengths(histogram, length);
    limit_lengths(histogram, length);
    std::array<int, kSymbols> canonical;
    std::iota(canonical.begin(), canonical.end(), 0);
    std::stable_sort(canonical.begin(), canonical.end(),
                     [&](int a, int b) { return length[a] != length[b] ? length[a] < length[b] : a < b; });
    uint32_t code = 0;
    int previous = length[canonical[0]];
    for (int s : canonical) {
        code <<= (length[s] - previous);
        previous = length[s];
        out->huff_code[s] = code | (static_cast<uint32_t>(length[s]) << 16);
        const uint32_t first = code << (kMaxLen - length[s]);
        const uint32_t span = 1u << (kMaxLen - length[s]);
        for (uint32_t e = 0; e < span; ++e)
            out->huff_lut[first + e] = static_cast<uint16_t>(s | (length[s] << 8));
        ++code;
    }
    return CF_OK;
}
