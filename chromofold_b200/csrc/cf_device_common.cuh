// cf_device_common.cuh — small device/host helpers shared by the kernels of this library.
#ifndef CHROMOFOLD_B200_DEVICE_COMMON_CUH
#define CHROMOFOLD_B200_DEVICE_COMMON_CUH

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "chromofold_b200/sealed_kv.h"

namespace cfb {

constexpr uint32_t kRansL = CF_B200_RANS_L;
constexpr int kZero = CF_B200_ZERO_POINT;

__host__ __device__ inline uint32_t align_up_u32(uint32_t v, uint32_t a) { return (v + a - 1) / a * a; }

// Split-KV workspace. One chunk = `pages_per_unit` consecutive pages of one sequence; one unit = (chunk, kv head).
//   [0, 64)                       PlanHeader
//   [64, 64 + 4*(seq_count+1))    chunk_prefix: number of chunks before each sequence
//   [shared_offset, ...)          shared-prefix partials, per (cell, sequence, local query head), when asked for (SharedSplit)
//   [partials_offset, ...)        per chunk and local query head: float m, float l, float acc[head_dim]
struct PlanHeader {
    uint32_t chunk_count;
    uint32_t pages_per_unit;
    uint32_t next_unit;      // work counter for the attention kernel; the plan kernel clears it
    uint32_t chunk_capacity;
    uint32_t overflow;
    uint32_t shared_pages;            // pages at the head of every sequence that the shared-prefix kernel handles (0 = none)
    uint32_t shared_ctas;             // CTAs of the shared-prefix kernel that take a share of it (0 = none), and
    uint32_t shared_rounds;           // rounds of eight pages that the shared pages make for one (kv head, row tile)
    uint32_t reserved_shared;         // unused
    uint32_t pad[7];
};

// How the shared-prefix kernel's work is cut. The rounds of all (kv head, row tile) pairs form one line, head-tile major:
// round x belongs to head-tile x / rounds. CTA b of `ctas` takes the rounds [first_round(b), first_round(b + 1)): every CTA
// gets the same number of rounds to within one, whatever the number of head-tiles. A CTA's stretch inside one head-tile is
// a unit; it leaves one partial per row, in cell (b - cta_of(the head-tile's first round)) of the row's shared partials.
// The plan kernel picks `ctas` so that no head-tile meets more than CF_B200_SHARED_CHUNKS_MAX CTAs.
struct SharedSplit {
    uint32_t rounds, head_tiles, ctas;
    __host__ __device__ uint64_t total() const { return static_cast<uint64_t>(rounds) * head_tiles; }
    __host__ __device__ uint64_t first_round(uint32_t b) const { return total() * b / ctas; }
    // the CTA whose stretch holds round x: the last b with first_round(b) <= x
    __host__ __device__ uint32_t cta_of(uint64_t x) const {
        return static_cast<uint32_t>(((x + 1ull) * ctas + total() - 1ull) / total()) - 1u;
    }
};
// Number of CTAs for the split: all `sm_count` of them where that keeps a head-tile within `cells` CTAs, else a multiple
// of the head-tiles (stretches then start and end on head-tile boundaries, `cells` or `cells - 1` CTAs per head-tile).
__host__ __device__ inline uint32_t shared_split_ctas(uint32_t rounds, uint32_t head_tiles, uint32_t sm_count, uint32_t cells) {
    const uint64_t total = static_cast<uint64_t>(rounds) * head_tiles;
    if (total == 0 || sm_count == 0) return 0;
    if (static_cast<uint64_t>(cells) * head_tiles <= sm_count) return head_tiles * (rounds < cells ? rounds : cells);
    const uint32_t ctas = total < sm_count ? static_cast<uint32_t>(total) : sm_count;
    if ((ctas + head_tiles - 1u) / head_tiles + 1u <= cells) return ctas;
    return head_tiles * (cells - 1u);
}

// What a (chunk, kv head) unit needs to start, written per chunk by the plan kernel so that the attention kernel's
// warps read one 32-byte record instead of searching the chunk prefix and chasing four dependent loads.
struct ChunkInfo {
    uint32_t seq, slot, sealed, qpos;      // batch entry, its sequence slot, its sealed tokens, its query position
    uint32_t page_begin, reserved[3];      // first page (index into the slot's page-table row) of the chunk
};
static_assert(sizeof(ChunkInfo) == 32, "one chunk record is two 16-byte loads");

struct WorkspaceLayout {
    uint64_t prefix_offset;
    uint64_t shared_offset;          // 0 = no room was set aside for shared-prefix partials
    uint64_t partials_offset;
    uint64_t partial_stride_floats;  // per (chunk, local query head)
    uint64_t chunk_capacity;
    uint64_t info_offset;            // ChunkInfo[chunk_capacity], behind the partials
};

__host__ __device__ inline WorkspaceLayout workspace_layout(uint32_t seq_count, uint32_t local_q_heads,
                                                            uint32_t head_dim, uint64_t workspace_bytes,
                                                            bool shared_prefix = false) {
    WorkspaceLayout w;
    w.prefix_offset = sizeof(PlanHeader);
    w.partials_offset = (w.prefix_offset + 4ull * (seq_count + 1) + 255ull) / 256ull * 256ull;
    w.partial_stride_floats = head_dim + 2ull;
    w.shared_offset = 0;
    if (shared_prefix) {
        w.shared_offset = w.partials_offset;
        w.partials_offset += (static_cast<uint64_t>(CF_B200_SHARED_CHUNKS_MAX) * seq_count * local_q_heads *
                              w.partial_stride_floats * 4ull + 255ull) / 256ull * 256ull;
    }
    const uint64_t per_chunk = w.partial_stride_floats * 4ull * local_q_heads;
    w.chunk_capacity = workspace_bytes > w.partials_offset + 32ull
                           ? (workspace_bytes - w.partials_offset - 32ull) / (per_chunk + sizeof(ChunkInfo)) : 0;
    w.info_offset = (w.partials_offset + w.chunk_capacity * per_chunk + 31ull) / 32ull * 32ull;
    return w;
}

// One-time set-up of a launcher, kept per device: kernel attributes (the dynamic shared-memory opt-in) and the SM
// count belong to a device, and one process may drive several. Returns the current device's slot, or nullptr with *error
// set. Concurrent first calls repeat the same idempotent set-up.
struct LauncherState {
    bool configured = false;
    int sm_count = 0;
};
inline LauncherState *launcher_state(LauncherState (&table)[64], cudaError_t *error) {
    int device = 0;
    *error = cudaGetDevice(&device);
    if (*error != cudaSuccess) return nullptr;
    if (device < 0 || device >= 64) {
        *error = cudaErrorInvalidDevice;
        return nullptr;
    }
    LauncherState *state = &table[device];
    if (state->sm_count == 0) {
        *error = cudaDeviceGetAttribute(&state->sm_count, cudaDevAttrMultiProcessorCount, device);
        if (*error != cudaSuccess) return nullptr;
    }
    return state;
}

// The unit size the WORKSPACE is sized for when the caller leaves the choice to the library: 16 pages, or fewer (down
// to 4) when the batch is so small that units of 16 pages would not give every resident warp of the attention kernel
// (148 SMs x 16 warps) about four units. (The plan kernel makes the actual choice, among the sizes that fit.)
__host__ __device__ inline uint32_t default_pages_per_unit(uint64_t total_pages, uint32_t kv_head_span) {
    const uint64_t slots = 4ull * 148ull * 16ull;
    const uint64_t wanted = (total_pages * kv_head_span + slots - 1ull) / slots;
    return static_cast<uint32_t>(wanted < 4ull ? 4ull : wanted > 16ull ? 16ull : wanted);
}

// A device pointer against the current device: false when it is memory of ANOTHER GPU. Kernels are launched on the
// current device and must only be given that device's memory, so the entry points refuse such a pointer instead of
// launching (host, managed and unregistered pointers are left to the usual CUDA checks).
inline bool on_current_device(const void *ptr) {
    if (ptr == nullptr) return true;
    cudaPointerAttributes attr;
    int device = -1;
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess || cudaGetDevice(&device) != cudaSuccess) {
        cudaGetLastError();
        return true;
    }
    return attr.type != cudaMemoryTypeDevice || attr.device == device;
}

// First token a query at `query_token` may see (src/cuda/paged_kv_attention.cu:50-52).
__host__ __device__ inline uint32_t window_begin(uint32_t query_token, uint32_t causal_window) {
    return causal_window == 0 || query_token + 1u <= causal_window ? 0u : query_token + 1u - causal_window;
}

#ifdef __CUDACC__

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- scalar block decoders: one thread walks one block ----------------------------------------------

// One rANS symbol: src/cuda/rans.cu:20-23 with the three table reads folded into one packed word
// (sym | freq << 8 | (slot - cum) << 20).
// Records are not trusted: a start offset past the payload is pulled back to its end, bytes past the end read as 0, and
// the renormalisation runs at most three times per symbol (a valid stream needs two: the state is >= 2^11 after the
// update), so a corrupt record yields wrong symbols but neither a stray read nor an endless loop.
template <class Emit>
__device__ __forceinline__ void rans_decode_block(const uint8_t *payload, uint32_t payload_bytes, uint32_t pos, uint32_t state,
                                                  const uint32_t *slot_table, int count, Emit emit) {
    pos = min(pos, payload_bytes);
    for (int j = 0; j < count; ++j) {
        const uint32_t e = slot_table[state & (CF_B200_RANS_M - 1u)];
        state = ((e >> 8) & 0xfffu) * (state >> CF_B200_RANS_PROB_BITS) + (e >> 20);
        for (int r = 0; r < 3 && state < kRansL; ++r) {
            state = (state << 8) | (pos < payload_bytes ? payload[pos] : 0u);
            ++pos;
        }
        emit(j, e & 0xffu);
    }
}

// One Huffman symbol per step: the next 12 bits MSB-first index the LUT
// (include/chromofold/detail/block_huffman_device.cuh:12-19), read here from two words at once.
template <class Emit>
__device__ __forceinline__ void huffman_decode_block(const uint32_t *words, uint32_t word_count, uint32_t bit, const uint16_t *lut,
                                                     int count, Emit emit) {
    bit = min(bit, 32u * word_count);   // an untrusted start offset stays inside the part; words past its end read as 0
    for (int j = 0; j < count; ++j) {
        const uint32_t w = bit >> 5;
        const uint64_t two = (static_cast<uint64_t>(w < word_count ? words[w] : 0u) << 32) | (w + 1u < word_count ? words[w + 1] : 0u);
        const uint32_t look = static_cast<uint32_t>(two >> (64u - CF_B200_HUFF_MAXLEN - (bit & 31u))) &
                              (CF_B200_HUFF_LUT_SIZE - 1u);
        const uint32_t sl = lut[look];
        emit(j, sl & 0xffu);
        bit += sl >> 8;
    }
}

// Fixed 8-bit symbols, MSB-first in u32 words (src/runtime/kv_gpu_fixture.cpp:110-116).
template <class Emit>
__device__ __forceinline__ void fixed8_decode_block(const uint32_t *words, uint32_t first_symbol, int count,
                                                    Emit emit) {
    for (int j = 0; j < count; ++j) {
        const uint32_t i = first_symbol + j;
        emit(j, (words[i >> 2] >> (24u - 8u * (i & 3u))) & 0xffu);
    }
}

// Start offset of block `b` against the part's length, and (rANS) its start state against [2^23, 2^31), the range every
// state the sealer leaves lies in: false = the record's block table is corrupt.
__device__ __forceinline__ bool part_block_start_ok(const uint8_t *part, uint32_t part_bytes, uint32_t coder, uint32_t nblocks,
                                                    uint32_t b, uint32_t symbols) {
    if (coder == CF_B200_CODER_RANS || coder == CF_B200_CODER_RANS_SPLIT4) {
        if (part_bytes < align_up_u32(6u * nblocks, 4u)) return false;
        const uint32_t state0 = reinterpret_cast<const uint32_t *>(part)[b];
        if (state0 < kRansL || state0 >= (kRansL << 8)) return false;
    }
    if (coder == CF_B200_CODER_RANS) {
        const uint32_t head = align_up_u32(6u * nblocks, 4u);
        return part_bytes >= head && reinterpret_cast<const uint16_t *>(part + 4u * nblocks)[b] <= part_bytes - head;
    }
    if (coder == CF_B200_CODER_HUFFMAN) {
        const uint32_t head = align_up_u32(2u * nblocks, 4u);
        return part_bytes >= head && reinterpret_cast<const uint16_t *>(part)[b] <= 8u * (part_bytes - head);
    }
    if (coder == CF_B200_CODER_RANS_SPLIT4) {   // block table | raw low-nibble plane (symbols / 2 bytes) | payload
        const uint32_t head = align_up_u32(6u * nblocks, 4u) + symbols / 2u;
        return part_bytes >= head && reinterpret_cast<const uint16_t *>(part + 4u * nblocks)[b] <= part_bytes - head;
    }
    if (coder == CF_B200_CODER_HUFFMAN_SPLIT4) {
        const uint32_t head = align_up_u32(2u * nblocks, 4u) + symbols / 2u;
        return part_bytes >= head && reinterpret_cast<const uint16_t *>(part)[b] <= 8u * (part_bytes - head);
    }
    return part_bytes >= align_up_u32(symbols, 4u);
}

// Decode block `b` of one stream part of part_bytes bytes (layout in sealed_page_format.h). `part` must be 16-byte
// aligned. Nothing outside [part, part + part_bytes) is read, whatever the part's block table says.
template <class Emit>
__device__ __forceinline__ void decode_part_block(const uint8_t *part, uint32_t part_bytes, uint32_t coder, uint32_t nblocks, uint32_t b,
                                                  uint32_t block_size, uint32_t symbols,
                                                  const cf_b200_codebook_tables *tables, Emit emit) {
    const uint32_t base = b * block_size;
    const int count = static_cast<int>(min(block_size, symbols - base));
    if (coder == CF_B200_CODER_RANS) {
        const uint32_t *state0 = reinterpret_cast<const uint32_t *>(part);
        const uint16_t *off = reinterpret_cast<const uint16_t *>(part + 4u * nblocks);
        const uint32_t head = align_up_u32(6u * nblocks, 4u);
        if (part_bytes < head) return;
        rans_decode_block(part + head, part_bytes - head, off[b], state0[b], tables->rans_slot, count, emit);
    } else if (coder == CF_B200_CODER_HUFFMAN) {
        const uint16_t *off = reinterpret_cast<const uint16_t *>(part);
        const uint32_t head = align_up_u32(2u * nblocks, 4u);
        if (part_bytes < head) return;
        huffman_decode_block(reinterpret_cast<const uint32_t *>(part + head), (part_bytes - head) / 4u, off[b], tables->huff_lut,
                             count, emit);
    } else if (coder == CF_B200_CODER_RANS_SPLIT4 || coder == CF_B200_CODER_HUFFMAN_SPLIT4) {
        // nibble-split: the stream codes pairs of high nibbles (count / 2 steps); the low nibbles come from the raw plane,
        // word lo[j][b] = symbols 8j..8j+7 of block b (symbol 8j+i at bits 8i..8i+3 for i < 4, 8j+4+i at bits 8i+4..8i+7)
        const bool rans = coder == CF_B200_CODER_RANS_SPLIT4;
        const uint32_t head = align_up_u32(rans ? 6u * nblocks : 2u * nblocks, 4u), plane_bytes = (block_size / 8u) * nblocks * 4u;
        if (part_bytes < head + plane_bytes) return;
        const uint32_t *plane = reinterpret_cast<const uint32_t *>(part + head);
        auto emit_pair = [&](int k, uint32_t pair) {
            const uint32_t w = plane[(static_cast<uint32_t>(k) >> 2) * nblocks + b], at = (2u * static_cast<uint32_t>(k)) & 7u;
            const uint32_t shift = at < 4u ? 8u * at : 8u * (at - 4u) + 4u;   // at is even: at + 1 sits 8 bits further
            emit(2 * k, (pair & 0xf0u) | ((w >> shift) & 0x0fu));
            emit(2 * k + 1, ((pair & 0x0fu) << 4) | ((w >> (shift + 8u)) & 0x0fu));
        };
        const uint8_t *payload = part + head + plane_bytes;
        if (rans)
            rans_decode_block(payload, part_bytes - head - plane_bytes, reinterpret_cast<const uint16_t *>(part + 4u * nblocks)[b],
                              reinterpret_cast<const uint32_t *>(part)[b], tables->rans_slot, count / 2, emit_pair);
        else
            huffman_decode_block(reinterpret_cast<const uint32_t *>(payload), (part_bytes - head - plane_bytes) / 4u,
                                 reinterpret_cast<const uint16_t *>(part)[b], tables->huff_lut, count / 2, emit_pair);
    } else {
        if (part_bytes < align_up_u32(symbols, 4u)) return;
        fixed8_decode_block(reinterpret_cast<const uint32_t *>(part), base, count, emit);
    }
}

#endif  // __CUDACC__

}  // namespace cfb

#endif
