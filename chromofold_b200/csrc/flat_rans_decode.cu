// flat_rans_decode.cu — the fast path of cf_rans_decode_async (src/cuda/rans.cu:38-50: a flat stream of block-rANS
// coded symbols, `data | byte_off[nb] | state0[nb]` with the three coding tables in global memory, int32 symbols out)
// for the block size the sealed pages use, 64. The reference decodes one block per thread with three dependent
// global-memory table look-ups and byte loads per symbol, and every thread writes its own 256-byte run of the output.
// Here:
//   * the three tables are folded once per CTA into the packed 4096-entry slot table of the lane-per-block decoders
//     (sym | (slot - cum) << 8 | freq << 20) in shared memory;
//   * a warp takes 64 consecutive blocks: their payload bytes (contiguous in `data`) are copied to shared memory with
//     coalesced word loads, laid out as two "parts" of 32 blocks in the sealed-page layout, so that the same RansLane
//     decoder runs on them, two blocks per lane interleaved symbol by symbol;
//   * the 64 x 64 symbols go through a shared-memory tile and leave as coalesced 128-byte stores.
// Other block sizes, and the blocks after the last whole group of 64 (the end of their bytes is not known to the
// callee), go to the reference-shaped kernel in compat_kv.cu. A table with a frequency of 4096 or a symbol above 255
// does not fit the packed entry: this kernel then decodes its groups the reference's way, one block per lane.
#include "lanes_decoders.cuh"

namespace cfb {
namespace {

using namespace lanes;

constexpr uint32_t kFlatWarps = 8;
constexpr uint32_t kFlatThreads = kFlatWarps * 32;
constexpr uint32_t kGroupBlocks = 64;                 // rANS blocks per warp pass
constexpr uint32_t kPartPayload = 3328;               // 32 blocks x 64 symbols x 12 bits = 3072 bytes at most, + start skew + read-ahead
constexpr uint32_t kPartBytes = 192 + kPartPayload;   // u32 state0[32] | u16 byte_off[32] | payload
constexpr uint32_t kTileWords = 16 + 1;               // 16 packed quads per block, padded against bank conflicts
constexpr uint32_t kWarpBytes = 2 * kPartBytes + kGroupBlocks * kTileWords * 4;
constexpr uint32_t kFlatSmem = 4096 * 4 + kFlatWarps * kWarpBytes + 16;

__global__ void __launch_bounds__(kFlatThreads, 2)
flat_rans_decode_kernel(const uint8_t *data, const int32_t *byte_off, const uint32_t *state0, const int32_t *slot2sym,
                        const int32_t *freq, const int32_t *cum, uint32_t groups, int32_t *out) {
    extern __shared__ __align__(16) uint8_t smem[];
    uint32_t *table = reinterpret_cast<uint32_t *>(smem);
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    uint8_t *mine = smem + 4096 * 4 + warp * kWarpBytes;
    uint32_t *tile = reinterpret_cast<uint32_t *>(mine + 2 * kPartBytes);

    int bad = 0;
    {   // 16 slots per thread; the loads of each level are issued together, so the CTA pays two memory latencies, not 32
        uint32_t sym[16], f[16], c[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) sym[i] = static_cast<uint32_t>(slot2sym[tid + i * kFlatThreads]);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            f[i] = sym[i] < 256u ? static_cast<uint32_t>(freq[sym[i]]) : 4096u;
            c[i] = sym[i] < 256u ? static_cast<uint32_t>(cum[sym[i]]) : 0u;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            const uint32_t slot = tid + i * kFlatThreads;
            bad |= sym[i] >= 256u || f[i] >= 4096u || slot - c[i] >= 4096u;
            table[slot] = (sym[i] & 0xffu) | ((slot - c[i]) & 0xfffu) << 8 | (f[i] & 0xfffu) << 20;
        }
    }
    const bool packed_ok = !__syncthreads_or(bad);   // false: the tables do not fit the packed entry, every group goes the slow way

    for (uint32_t group = blockIdx.x * kFlatWarps + warp; group < groups; group += gridDim.x * kFlatWarps) {
        const uint32_t b0 = group * kGroupBlocks;
        bool fits = packed_ok;
        for (uint32_t part = 0; part < 2; ++part) {
            uint8_t *dst = mine + part * kPartBytes;
            const uint32_t first = b0 + 32u * part;
            if (!fits) break;
            const uint32_t start = static_cast<uint32_t>(byte_off[first]), end = static_cast<uint32_t>(byte_off[first + 32u]);
            const uint32_t skew = static_cast<uint32_t>(reinterpret_cast<uintptr_t>(data + start) & 3u), length = end - start;
            fits = end >= start && skew + length + 16u <= kPartPayload;   // whole words are copied: the bytes keep their alignment
            if (!fits) break;
            // the ABI does not promise ordered offsets: a block that starts outside [start, end] sends the group the slow way
            const uint32_t mine_off = static_cast<uint32_t>(byte_off[first + lane]);
            fits = __all_sync(0xffffffffu, mine_off >= start && mine_off <= end);
            if (!fits) break;
            reinterpret_cast<uint32_t *>(dst)[lane] = state0[first + lane];
            reinterpret_cast<uint16_t *>(dst + 128)[lane] = static_cast<uint16_t>(mine_off - start + skew);
            const uint32_t *src = reinterpret_cast<const uint32_t *>(data + (start - skew));
            uint32_t *payload = reinterpret_cast<uint32_t *>(dst + 192);
            for (uint32_t w = lane; w < (skew + length + 3u) / 4u; w += 32u) payload[w] = src[w];
        }
        __syncwarp();
        if (!fits) {   // a group whose bytes do not look like block-64 rANS: one block per lane, the reference's way
            for (uint32_t pass = 0; pass < 2; ++pass) {
                const uint32_t b = b0 + 32u * pass + lane;
                uint32_t x = state0[b];
                const uint8_t *bytes = data + byte_off[b];
                for (uint32_t j = 0; j < 64u; ++j) {
                    const uint32_t slot = x & (CF_B200_RANS_M - 1u);
                    const int s = slot2sym[slot];
                    const uint32_t si = static_cast<uint32_t>(s) & 255u;   // a symbol outside the tables must not index past them
                    x = static_cast<uint32_t>(freq[si]) * (x >> CF_B200_RANS_PROB_BITS) + slot - static_cast<uint32_t>(cum[si]);
                    // a valid stream needs at most two bytes here (the state is >= 2^11 after the update); the bound keeps
                    // a corrupt table (frequency 0) from reading on without end
                    for (int r = 0; r < 3 && x < (1u << 23); ++r) x = (x << 8) | *bytes++;
                    out[static_cast<uint64_t>(b) * 64u + j] = s;
                }
            }
            continue;
        }
        RansLane a, b;   // blocks b0 + lane and b0 + 32 + lane
        a.open(mine, kPartBytes, lane, table);
        b.open(mine + kPartBytes, kPartBytes, lane, table);
#pragma unroll 4
        for (uint32_t q = 0; q < 16; ++q) {
            a.reload();
            b.reload();
            uint32_t ea[4], eb[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                ea[i] = a.symbol();
                eb[i] = b.symbol();
            }
            tile[lane * kTileWords + q] = pack_low_bytes(ea[0], ea[1], ea[2], ea[3]);
            tile[(32u + lane) * kTileWords + q] = pack_low_bytes(eb[0], eb[1], eb[2], eb[3]);
        }
        __syncwarp();
        // block r of the group: 64 symbols = two coalesced stores of 32 int32
        int32_t *dst = out + static_cast<uint64_t>(b0) * 64u;
        const uint8_t *bytes = reinterpret_cast<const uint8_t *>(tile);
#pragma unroll 4
        for (uint32_t r = 0; r < kGroupBlocks; ++r) {
            dst[r * 64u + lane] = bytes[r * kTileWords * 4u + lane];
            dst[r * 64u + 32u + lane] = bytes[r * kTileWords * 4u + 32u + lane];
        }
        __syncwarp();   // the tile and the parts are reused by the next group
    }
}

}  // namespace

// Decodes the first `groups` * 64 blocks (block size 64) of the stream; block groups * 64 must exist (its byte offset
// ends the last group's bytes).
cudaError_t launch_flat_rans_decode(const uint8_t *data, const int32_t *byte_off, const uint32_t *state0, const int32_t *slot2sym,
                                    const int32_t *freq, const int32_t *cum, uint32_t groups, int32_t *out, cudaStream_t stream) {
    static LauncherState table[64];
    cudaError_t e;
    LauncherState *state = launcher_state(table, &e);
    if (!state) return e;
    if (!state->configured) {
        e = cudaFuncSetAttribute(flat_rans_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kFlatSmem));
        if (e != cudaSuccess) return e;
        state->configured = true;
    }
    const int sm_count = state->sm_count;
    const uint32_t wanted = (groups + kFlatWarps - 1) / kFlatWarps;
    const uint32_t grid = std::max(1u, std::min(wanted, static_cast<uint32_t>(2 * sm_count)));
    flat_rans_decode_kernel<<<grid, kFlatThreads, kFlatSmem, stream>>>(data, byte_off, state0, slot2sym, freq, cum, groups, out);
    return cudaPeekAtLastError();
}

}  // namespace cfb
