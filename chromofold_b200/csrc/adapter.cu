// adapter.cu — the llama.cpp-facing KV adapter (include/chromofold_b200/compat_adapter.h) on top of the sealed-KV
// entry points. Host logic mirrors the reference's adapter and single-sequence cache
// (integrations/llama.cpp/chromofold_kv_adapter.cpp, src/runtime/compressed_kv_cache.cu) — same checks, same error
// strings where a caller could match on them — while every byte of KV lives on the GPU: appended rows go straight
// into a device tail, full tiles are sealed by cf_b200_seal_pages_async, attention is cf_b200_sealed_attention_async.

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "chromofold_b200/compat_adapter.h"
#include "chromofold_b200/compat_kv.h"
#include "chromofold_b200/sealed_kv.h"

namespace {

void cuda_check(cudaError_t e, const char *what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

template <class T>
struct DeviceBuffer {  // grow-only device array; growing copies the old contents (set-up and append path only)
    T *ptr = nullptr;
    size_t count = 0;
    ~DeviceBuffer() { if (ptr) cudaFree(ptr); }
    void ensure(size_t wanted, cudaStream_t s) {
        if (wanted <= count) return;
        size_t next = std::max(wanted, count ? count * 2 : wanted);
        T *fresh = nullptr;
        cuda_check(cudaMalloc(reinterpret_cast<void **>(&fresh), next * sizeof(T)), "cudaMalloc");
        cuda_check(cudaMemsetAsync(fresh, 0, next * sizeof(T), s), "cudaMemsetAsync");
        if (ptr) {
            cuda_check(cudaMemcpyAsync(fresh, ptr, count * sizeof(T), cudaMemcpyDeviceToDevice, s), "cudaMemcpyAsync");
            cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
            cudaFree(ptr);
        }
        ptr = fresh;
        count = next;
    }
};

// ---- the reference's own page quantiser on the GPU ---------------------------------------------------------------
// What the reference's adapter stores for kv_bits 4 / 8 (integrations/llama.cpp/chromofold_kv_adapter.cpp:30-31) is what
// gpu_fixture::encode_int{4,8}_page makes on the host (src/runtime/kv_gpu_fixture.cpp:46-95): K with one fp32 scale per
// channel, V with one per token, scale = absmax / qmax (1 when the row or column is all zero), symbol =
// clamp(lrint(x / scale), -(qmax+1), qmax) + 2^(bits-1), symbols packed MSB-first at `bits` bits, block offsets
// b * 64 * bits, the LUT s | bits << 8. The kernel below makes the same page, bit for bit, from rows already on the GPU.
struct KiviLayout {
    size_t k_words, v_words, k_scales, v_scales, k_offsets, v_offsets, total;   // byte offsets inside a page block
    uint32_t word_count, block_count;
};
inline KiviLayout kivi_layout(uint32_t tokens, uint32_t dim, uint32_t bits) {
    KiviLayout l{};
    const uint64_t symbols = static_cast<uint64_t>(tokens) * dim;
    l.word_count = static_cast<uint32_t>((symbols * bits + 31u) / 32u);
    l.block_count = static_cast<uint32_t>((symbols + 63u) / 64u);
    size_t at = 0;
    auto take = [&](size_t bytes) { const size_t here = at; at += (bytes + 15u) / 16u * 16u; return here; };
    l.k_words = take(4ull * l.word_count);
    l.v_words = take(4ull * l.word_count);
    l.k_scales = take(4ull * dim);
    l.v_scales = take(4ull * tokens);
    l.k_offsets = take(4ull * l.block_count);
    l.v_offsets = take(4ull * l.block_count);
    l.total = at;
    return l;
}

// One CTA per page. rows: K / V as [token][row_stride floats], this head's `dim` values first in each row.
__global__ void __launch_bounds__(256) kivi_quantise_kernel(const float *k_rows, const float *v_rows, uint32_t row_stride,
                                                            uint32_t tokens, uint32_t dim, uint32_t bits, uint8_t *block,
                                                            KiviLayout lay, uint32_t *status) {
    extern __shared__ float scales[];   // [dim] K scales | [tokens] V scales
    float *k_scale = scales, *v_scale = scales + dim;
    const int qmax = (1 << (bits - 1)) - 1, zero = 1 << (bits - 1);
    int bad = 0;
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) {   // per channel over the tokens
        float m = 0.0f;
        for (uint32_t t = 0; t < tokens; ++t) {
            const float x = k_rows[static_cast<size_t>(t) * row_stride + d];
            bad |= !isfinite(x);
            m = fmaxf(m, fabsf(x));
        }
        k_scale[d] = m == 0.0f ? 1.0f : __fdiv_rn(m, static_cast<float>(qmax));
    }
    for (uint32_t t = threadIdx.x / 32u; t < tokens; t += blockDim.x / 32u) {   // per token over the channels: a warp each
        float m = 0.0f;
        for (uint32_t d = threadIdx.x % 32u; d < dim; d += 32u) {
            const float x = v_rows[static_cast<size_t>(t) * row_stride + d];
            bad |= !isfinite(x);
            m = fmaxf(m, fabsf(x));
        }
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (threadIdx.x % 32u == 0) v_scale[t] = m == 0.0f ? 1.0f : __fdiv_rn(m, static_cast<float>(qmax));
    }
    if (__syncthreads_or(bad)) {   // kv_gpu_fixture.cpp:13: a non-finite value is an error; nothing of the page is used
        if (threadIdx.x == 0) atomicOr(status, 1u);
        return;
    }
    const uint32_t per_word = 32u / bits;
    uint32_t *kw = reinterpret_cast<uint32_t *>(block + lay.k_words), *vw = reinterpret_cast<uint32_t *>(block + lay.v_words);
    const uint64_t symbols = static_cast<uint64_t>(tokens) * dim;
    auto symbol = [&](float x, float scale) {
        const int q = max(-(qmax + 1), min(qmax, __float2int_rn(__fdiv_rn(x, scale))));   // lrint(x / scale), clamped
        return static_cast<uint32_t>(q + zero);
    };
    for (uint32_t w = threadIdx.x; w < lay.word_count; w += blockDim.x) {
        uint32_t kword = 0, vword = 0;
        for (uint32_t j = 0; j < per_word; ++j) {
            const uint64_t i = static_cast<uint64_t>(w) * per_word + j;
            if (i >= symbols) break;
            const uint32_t t = static_cast<uint32_t>(i / dim), d = static_cast<uint32_t>(i % dim);
            const uint32_t shift = (32u - bits) - j * bits;
            kword |= symbol(k_rows[static_cast<size_t>(t) * row_stride + d], k_scale[d]) << shift;
            vword |= symbol(v_rows[static_cast<size_t>(t) * row_stride + d], v_scale[t]) << shift;
        }
        kw[w] = kword;
        vw[w] = vword;
    }
    for (uint32_t d = threadIdx.x; d < dim; d += blockDim.x) reinterpret_cast<float *>(block + lay.k_scales)[d] = k_scale[d];
    for (uint32_t t = threadIdx.x; t < tokens; t += blockDim.x) reinterpret_cast<float *>(block + lay.v_scales)[t] = v_scale[t];
    for (uint32_t b = threadIdx.x; b < lay.block_count; b += blockDim.x) {
        reinterpret_cast<int32_t *>(block + lay.k_offsets)[b] = static_cast<int32_t>(b * 64u * bits);
        reinterpret_cast<int32_t *>(block + lay.v_offsets)[b] = static_cast<int32_t>(b * 64u * bits);
    }
}

struct HeadState {   // per (layer, kv head), in tokens
    uint64_t appended = 0;      // everything ever appended
    uint32_t sealed = 0;        // tokens in sealed tiles
    uint32_t tail = 0;          // tokens in the device tail
    uint32_t next_token = 0;    // position the next append must start at
    bool started = false;
    bool flushed_partial = false;
};

struct LayerState {
    bool calibrated = false;
    std::vector<uint32_t> page_ids;   // tile index -> page id
    uint32_t device_sealed = 0xffffffffu, device_tail = 0xffffffffu;  // what the device scalars hold
};

}  // namespace

struct cf_llama_kv_adapter {
    cf_llama_kv_options opt{};
    uint32_t tile_tokens = 0;     // T: tokens per record, T * head_dim <= 4096, T divides page_size
    uint32_t coder = CF_B200_CODER_RANS;
    std::string last_error;
    std::vector<HeadState> heads;
    std::vector<LayerState> layers;
    uint32_t next_page_id = 1;
    uint64_t sealed_tiles = 0;

    DeviceBuffer<uint8_t> arena;
    DeviceBuffer<uint64_t> page_dir;
    DeviceBuffer<uint32_t> page_table;      // [layer][stride]
    uint32_t stride = 0;
    DeviceBuffer<uint32_t> scalars;          // [0,L): sealed tokens per layer; [L,2L): tail tokens per layer
    DeviceBuffer<float> tail_k, tail_v;      // [layer][kv_head][T][head_dim]
    DeviceBuffer<cf_b200_codebook_tables> tables;  // [layer][2]
    DeviceBuffer<uint32_t> slots;            // [layer][max_queries]: the layer index repeated
    DeviceBuffer<uint32_t> positions;        // iota
    DeviceBuffer<uint32_t> jobs;             // scratch for seal jobs: slot, page, tokens, head
    DeviceBuffer<unsigned long long> cursor; // [0] arena cursor, [1..512] histograms
    DeviceBuffer<uint32_t> status;
    DeviceBuffer<uint8_t> workspace;
    static constexpr uint32_t kMaxQueries = 4096;

    // Reference-exact mode (the default): pages as the reference's own fixed-width descriptors, made by
    // kivi_quantise_kernel, attended by cf_kv_paged_attention_async. CHROMOFOLD_B200_CODER switches to format v1.
    bool kivi = true;
    uint32_t kivi_bits = 4;
    static constexpr size_t kKiviChunk = 32u << 20;
    std::vector<uint8_t *> kivi_chunks;      // page blocks never move: descriptors hold their addresses
    size_t kivi_chunk_index = 0, kivi_chunk_used = 0;
    DeviceBuffer<float> kivi_tail_k, kivi_tail_v;   // [layer][page_size][kv_head][head_dim]: the layout the attention reads
    DeviceBuffer<int32_t> kivi_lut;
    std::vector<std::unique_ptr<DeviceBuffer<cf_kv_device_page>>> kivi_descs;   // per layer, device
    std::vector<std::vector<cf_kv_device_page>> kivi_host_descs;                // per layer, the same on the host
    uint64_t kivi_resident_bytes = 0;

    ~cf_llama_kv_adapter() {
        for (uint8_t *c : kivi_chunks) cudaFree(c);
    }
    size_t kivi_row_floats() const { return static_cast<size_t>(opt.kv_head_count) * opt.head_dim; }
    float *kivi_tail(DeviceBuffer<float> &buffer, uint32_t layer) const {
        return buffer.ptr + static_cast<size_t>(layer) * opt.page_size * kivi_row_floats();
    }
    uint8_t *kivi_take(size_t bytes) {
        if (bytes > kKiviChunk) throw std::runtime_error("page is larger than an adapter memory chunk");
        if (kivi_chunk_index < kivi_chunks.size() && kivi_chunk_used + bytes > kKiviChunk) {
            ++kivi_chunk_index;
            kivi_chunk_used = 0;
        }
        if (kivi_chunk_index >= kivi_chunks.size()) {
            uint8_t *fresh = nullptr;
            cuda_check(cudaMalloc(reinterpret_cast<void **>(&fresh), kKiviChunk), "cudaMalloc");
            kivi_chunks.push_back(fresh);
            kivi_chunk_used = 0;
        }
        uint8_t *at = kivi_chunks[kivi_chunk_index] + kivi_chunk_used;
        kivi_chunk_used += (bytes + 255u) / 256u * 256u;
        return at;
    }
    void kivi_create() {
        cudaStream_t s = nullptr;
        const size_t tail = static_cast<size_t>(opt.layer_count) * opt.page_size * kivi_row_floats();
        kivi_tail_k.ensure(tail, s);
        kivi_tail_v.ensure(tail, s);
        const uint32_t levels = 1u << kivi_bits;
        std::vector<int32_t> lut(levels);
        for (uint32_t v = 0; v < levels; ++v) lut[v] = static_cast<int32_t>(v | (kivi_bits << 8));
        kivi_lut.ensure(levels, s);
        cuda_check(cudaMemcpy(kivi_lut.ptr, lut.data(), levels * 4, cudaMemcpyHostToDevice), "upload lut");
        status.ensure(1, s);
        kivi_descs.clear();
        for (uint32_t l = 0; l < opt.layer_count; ++l) {
            kivi_descs.push_back(std::make_unique<DeviceBuffer<cf_kv_device_page>>());
            kivi_descs.back()->ensure(64, s);
        }
        kivi_host_descs.assign(opt.layer_count, {});
        if (const char *reserve = std::getenv("CHROMOFOLD_B200_RESERVE_TOKENS")) {   // page memory and descriptors up front
            const unsigned long long tokens = std::strtoull(reserve, nullptr, 10);
            const size_t pages = static_cast<size_t>((tokens + opt.page_size - 1) / opt.page_size);   // per layer and kv head
            const size_t page_bytes = (kivi_layout(opt.page_size, opt.head_dim, kivi_bits).total + 255u) / 256u * 256u;
            const size_t per_chunk = kKiviChunk / page_bytes;
            const size_t chunks = per_chunk ? (pages * opt.layer_count * opt.kv_head_count + per_chunk - 1) / per_chunk : 0;
            for (size_t i = kivi_chunks.size(); i < chunks; ++i) {
                uint8_t *fresh = nullptr;
                cuda_check(cudaMalloc(reinterpret_cast<void **>(&fresh), kKiviChunk), "cudaMalloc");
                kivi_chunks.push_back(fresh);
            }
            for (uint32_t l = 0; l < opt.layer_count; ++l) kivi_descs[l]->ensure(std::max<size_t>(64, pages * opt.kv_head_count), s);
        }
        cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    }
    void kivi_reset() {
        kivi_chunk_index = 0;
        kivi_chunk_used = 0;
        kivi_resident_bytes = 0;
        for (auto &d : kivi_host_descs) d.clear();
    }
    // Quantise the tail rows of (layer, kv_head) into one page (the reference's seal_full_pages / flush for one head).
    void kivi_seal(uint32_t layer, uint32_t kv_head, cudaStream_t s) {
        HeadState &h = head(layer, kv_head);
        if (h.tail == 0) return;
        const uint32_t D = opt.head_dim, tokens = h.tail;
        const KiviLayout lay = kivi_layout(tokens, D, kivi_bits);
        uint8_t *block = kivi_take(lay.total);
        cuda_check(cudaMemsetAsync(status.ptr, 0, 4, s), "clear status");
        const size_t smem = (static_cast<size_t>(D) + tokens) * sizeof(float);
        kivi_quantise_kernel<<<1, 256, smem, s>>>(kivi_tail(kivi_tail_k, layer) + static_cast<size_t>(kv_head) * D,
                                                  kivi_tail(kivi_tail_v, layer) + static_cast<size_t>(kv_head) * D,
                                                  static_cast<uint32_t>(kivi_row_floats()), tokens, D, kivi_bits, block, lay, status.ptr);
        cuda_check(cudaGetLastError(), "page quantise launch");
        uint32_t bad = 0;   // the reference quantises on the host and throws at once; so does this front
        cuda_check(cudaMemcpyAsync(&bad, status.ptr, 4, cudaMemcpyDeviceToHost, s), "read status");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        if (bad) throw std::invalid_argument("invalid quantization input");
        cf_kv_device_page page{};
        page.k_words = reinterpret_cast<const uint32_t *>(block + lay.k_words);
        page.v_words = reinterpret_cast<const uint32_t *>(block + lay.v_words);
        page.k_scales = reinterpret_cast<const float *>(block + lay.k_scales);
        page.v_scales = reinterpret_cast<const float *>(block + lay.v_scales);
        page.k_block_offsets = reinterpret_cast<const int32_t *>(block + lay.k_offsets);
        page.v_block_offsets = reinterpret_cast<const int32_t *>(block + lay.v_offsets);
        page.k_lut = page.v_lut = kivi_lut.ptr;
        page.token_begin = h.next_token - h.tail;
        page.token_count = tokens;
        page.head_dim = D;
        page.block_size = 64;
        page.k_max_code_length = page.v_max_code_length = page.fixed_code_length = kivi_bits;
        page.zero_point = 1u << (kivi_bits - 1);
        page.kv_head = kv_head;
        std::vector<cf_kv_device_page> &host = kivi_host_descs[layer];
        host.push_back(page);
        DeviceBuffer<cf_kv_device_page> &dev = *kivi_descs[layer];
        dev.ensure(host.size(), s);
        cuda_check(cudaMemcpyAsync(dev.ptr + host.size() - 1, &host.back(), sizeof page, cudaMemcpyHostToDevice, s), "publish page");
        // EncodedKvPage::resident_bytes: words, offsets, both LUTs, scales
        kivi_resident_bytes += 8ull * lay.word_count + 8ull * lay.block_count + 8ull * (1u << kivi_bits) + 4ull * (D + tokens);
        if (h.tail < opt.page_size) h.flushed_partial = true;
        h.sealed += h.tail;
        h.tail = 0;
        ++sealed_tiles;
    }

    HeadState &head(uint32_t layer, uint32_t h) { return heads[static_cast<size_t>(layer) * opt.kv_head_count + h]; }
    size_t tile_values() const { return static_cast<size_t>(tile_tokens) * opt.head_dim; }
    size_t max_record_bytes() const { return 16 + 2 * ((tile_values() + 15) / 16 * 16); }

    void reset(cudaStream_t s) {
        heads.assign(static_cast<size_t>(opt.layer_count) * opt.kv_head_count, HeadState{});
        layers.assign(opt.layer_count, LayerState{});
        next_page_id = 1;
        sealed_tiles = 0;
        kivi_reset();
        if (cursor.ptr) cuda_check(cudaMemsetAsync(cursor.ptr, 0, sizeof(unsigned long long), s), "memset cursor");
        if (page_dir.ptr) cuda_check(cudaMemsetAsync(page_dir.ptr, 0, page_dir.count * sizeof(uint64_t), s), "memset dir");
        if (status.ptr) cuda_check(cudaMemsetAsync(status.ptr, 0, sizeof(uint32_t), s), "memset status");
    }

    void create_buffers() {
        cudaStream_t s = nullptr;
        const uint32_t L = opt.layer_count, H = opt.kv_head_count;
        stride = 4096;
        page_table.ensure(static_cast<size_t>(L) * stride, s);
        scalars.ensure(2 * L, s);
        tail_k.ensure(static_cast<size_t>(L) * H * tile_values(), s);
        tail_v.ensure(static_cast<size_t>(L) * H * tile_values(), s);
        tables.ensure(2 * L, s);
        cursor.ensure(1 + 512, s);
        status.ensure(1, s);
        jobs.ensure(4 * 64, s);
        arena.ensure(64u << 20, s);
        page_dir.ensure(static_cast<size_t>(65536) * H, s);
        std::vector<uint32_t> host(static_cast<size_t>(L) * kMaxQueries);
        for (uint32_t l = 0; l < L; ++l) std::fill_n(host.begin() + static_cast<size_t>(l) * kMaxQueries, kMaxQueries, l);
        slots.ensure(host.size(), s);
        cuda_check(cudaMemcpy(slots.ptr, host.data(), host.size() * 4, cudaMemcpyHostToDevice), "upload slots");
        grow_positions(1u << 16, s);
        // workspace: one chunk per query row is the floor; give 16-tile chunks room for 1M tokens
        cf_b200_sealed_attention_desc d{};
        d.kv_head_count = H;
        d.query_head_count = opt.query_head_count;
        d.head_dim = opt.head_dim;
        d.seq_count = kMaxQueries;
        uint64_t bytes = 0;
        cf_b200_sealed_attention_workspace_bytes(&d, 65536, &bytes);
        workspace.ensure(bytes + 256, s);
        cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    }

    void grow_positions(size_t wanted, cudaStream_t s) {
        if (wanted <= positions.count) return;
        const size_t old = positions.count;
        positions.ensure(wanted, s);
        std::vector<uint32_t> host(positions.count - old);
        for (size_t i = 0; i < host.size(); ++i) host[i] = static_cast<uint32_t>(old + i);
        cuda_check(cudaMemcpyAsync(positions.ptr + old, host.data(), host.size() * 4, cudaMemcpyHostToDevice, s), "upload positions");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
    }

    // Make sure `tiles` more tiles fit: arena by the worst-case record size, directory and page table by count.
    void reserve(uint32_t layer, uint32_t tile_index, cudaStream_t s) {
        arena.ensure((sealed_tiles + 1) * max_record_bytes() + 4096, s);
        page_dir.ensure(static_cast<size_t>(next_page_id + 2) * opt.kv_head_count, s);
        if (tile_index >= stride) {  // widen every row of the page table
            const uint32_t wider = stride * 2;
            DeviceBuffer<uint32_t> fresh;
            fresh.ensure(static_cast<size_t>(opt.layer_count) * wider, s);
            cuda_check(cudaMemcpy2DAsync(fresh.ptr, wider * 4, page_table.ptr, stride * 4, stride * 4, opt.layer_count,
                                         cudaMemcpyDeviceToDevice, s), "widen page table");
            cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
            std::swap(fresh.ptr, page_table.ptr);
            std::swap(fresh.count, page_table.count);
            stride = wider;
        }
        (void)layer;
    }

    cf_b200_seal_desc seal_desc(uint32_t layer) const {
        cf_b200_seal_desc d{};
        d.struct_size = sizeof d;
        d.abi_version = CF_B200_ABI_VERSION;
        d.kv_head_count = opt.kv_head_count;
        d.head_dim = opt.head_dim;
        d.page_tokens = tile_tokens;
        d.block_size = 64;
        d.coder = coder;
        d.codebook_id = layer;
        d.k_tables = tables.ptr + 2 * layer;
        d.v_tables = tables.ptr + 2 * layer + 1;
        d.tail_k = tail_k.ptr;
        d.tail_v = tail_v.ptr;
        d.tail_type = CF_B200_F32;
        d.arena = arena.ptr;
        d.arena_units = arena.count / 16;
        d.arena_cursor_units = cursor.ptr;
        d.page_dir = page_dir.ptr;
        d.status = status.ptr;
        return d;
    }

    void upload_job(uint32_t slot, uint32_t page, uint32_t tokens, uint32_t kv_head, cudaStream_t s) {
        const uint32_t host[4] = {slot, page, tokens, kv_head};
        cuda_check(cudaMemcpyAsync(jobs.ptr, &host[0], 4, cudaMemcpyHostToDevice, s), "job");
        cuda_check(cudaMemcpyAsync(jobs.ptr + 64, &host[1], 4, cudaMemcpyHostToDevice, s), "job");
        cuda_check(cudaMemcpyAsync(jobs.ptr + 128, &host[2], 4, cudaMemcpyHostToDevice, s), "job");
        cuda_check(cudaMemcpyAsync(jobs.ptr + 192, &host[3], 4, cudaMemcpyHostToDevice, s), "job");
    }

    // First tile of a layer: histogram its quantised symbols on the GPU, build the layer's codebooks.
    void calibrate(uint32_t layer, uint32_t kv_head, uint32_t tokens, cudaStream_t s) {
        cf_b200_seal_desc d = seal_desc(layer);
        upload_job(layer, 0, tokens, kv_head, s);
        d.job_slots = jobs.ptr;
        d.job_tokens = jobs.ptr + 128;
        d.job_heads = jobs.ptr + 192;
        d.job_count = 1;
        cuda_check(cudaMemsetAsync(cursor.ptr + 1, 0, 512 * sizeof(unsigned long long), s), "memset hist");
        if (cf_b200_histogram_async(&d, cursor.ptr + 1, cursor.ptr + 257, s) != CF_OK)
            throw std::runtime_error("ChromoFold histogram launch rejected");
        unsigned long long hist[512];
        cuda_check(cudaMemcpyAsync(hist, cursor.ptr + 1, sizeof hist, cudaMemcpyDeviceToHost, s), "download hist");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        std::vector<cf_b200_codebook_tables> host(2);
        uint64_t hk[256], hv[256];
        for (int i = 0; i < 256; ++i) { hk[i] = hist[i]; hv[i] = hist[256 + i]; }
        if (cf_b200_codebook_build(hk, &host[0]) != CF_OK || cf_b200_codebook_build(hv, &host[1]) != CF_OK)
            throw std::runtime_error("ChromoFold codebook build failed");
        cuda_check(cudaMemcpyAsync(tables.ptr + 2 * layer, host.data(), 2 * sizeof(cf_b200_codebook_tables),
                                   cudaMemcpyHostToDevice, s), "upload codebooks");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        layers[layer].calibrated = true;
    }

    // Seal the tail of (layer, kv_head): `tokens` rows become tile number sealed / T.
    void seal_tail(uint32_t layer, uint32_t kv_head, cudaStream_t s) {
        HeadState &h = head(layer, kv_head);
        if (h.tail == 0) return;
        LayerState &ls = layers[layer];
        const uint32_t tile_index = h.sealed / tile_tokens;
        reserve(layer, tile_index, s);
        if (!ls.calibrated) calibrate(layer, kv_head, h.tail, s);
        if (tile_index >= ls.page_ids.size()) {  // first head to reach this tile names the page
            ls.page_ids.push_back(next_page_id);
            cuda_check(cudaMemcpyAsync(page_table.ptr + static_cast<size_t>(layer) * stride + tile_index, &next_page_id, 4,
                                       cudaMemcpyHostToDevice, s), "publish page id");
            ++next_page_id;
        }
        cf_b200_seal_desc d = seal_desc(layer);
        upload_job(layer, ls.page_ids[tile_index], h.tail, kv_head, s);
        d.job_slots = jobs.ptr;
        d.job_pages = jobs.ptr + 64;
        d.job_tokens = jobs.ptr + 128;
        d.job_heads = jobs.ptr + 192;
        d.job_count = 1;
        if (cf_b200_seal_pages_async(&d, s) != CF_OK) throw std::runtime_error("ChromoFold seal launch rejected");
        if (h.tail < tile_tokens) h.flushed_partial = true;
        h.sealed += h.tail;
        h.tail = 0;
        ++sealed_tiles;
    }
};

namespace {

template <class Operation>
int guarded(cf_llama_kv_adapter *adapter, Operation &&operation) {  // chromofold_kv_adapter.cpp:35-49
    if (adapter == nullptr) return -1;
    try {
        operation();
        adapter->last_error.clear();
        return 0;
    } catch (const std::exception &error) {
        adapter->last_error = error.what();
        return -1;
    } catch (...) {
        adapter->last_error = "unknown ChromoFold KV error";
        return -1;
    }
}

uint32_t choose_tile_tokens(uint32_t page_size, uint32_t head_dim) {
    // 16-token records at head_dim 128, 96, 64 and 32 are the geometries of the lane-per-block attention kernels
    if ((head_dim == 128 || head_dim == 96 || head_dim == 64 || head_dim == 32) && page_size % 16 == 0) return 16;
    const uint32_t limit = CF_B200_MAX_STREAM_SYMBOLS / head_dim;
    for (uint32_t t = std::min(page_size, limit); t >= 1; --t)
        if (page_size % t == 0) return t;
    return 1;
}

}  // namespace

extern "C" int cf_llama_kv_options_validate(const cf_llama_kv_options *options) {
    if (options == nullptr || options->struct_size != sizeof(cf_llama_kv_options)) return -1;
    if (options->backend == CF_LLAMA_KV_BACKEND_DENSE) return 0;
    if (options->backend != CF_LLAMA_KV_BACKEND_CHROMOFOLD || options->layer_count == 0 || options->kv_head_count == 0 ||
        options->query_head_count == 0 || options->head_dim == 0 || options->page_size == 0 ||
        options->gqa_group_size == 0 || options->query_head_count != options->kv_head_count * options->gqa_group_size)
        return -1;
    return 0;
}

extern "C" cf_llama_kv_adapter *cf_llama_kv_create(const cf_llama_kv_options *options) {
    if (cf_llama_kv_options_validate(options) != 0 || options->backend != CF_LLAMA_KV_BACKEND_CHROMOFOLD) return nullptr;
    if (options->head_dim > CF_KV_MAX_HEAD_DIM || options->gqa_group_size > 16) return nullptr;
    try {
        auto *a = new cf_llama_kv_adapter();
        a->opt = *options;
        a->tile_tokens = choose_tile_tokens(options->page_size, options->head_dim);
        a->kivi_bits = options->kv_bits == 8 ? 8u : 4u;   // chromofold_kv_adapter.cpp:30-31: 8 selects int8, anything else int4
        if (const char *env = std::getenv("CHROMOFOLD_B200_CODER")) {   // opt in to entropy-coded format-v1 pages
            a->kivi = false;
            if (std::strcmp(env, "huffman") == 0) a->coder = CF_B200_CODER_HUFFMAN;
            else if (std::strcmp(env, "fixed8") == 0) a->coder = CF_B200_CODER_FIXED8;
            else if (std::strcmp(env, "rans4") == 0) a->coder = CF_B200_CODER_RANS_SPLIT4;
            else if (std::strcmp(env, "huffman4") == 0) a->coder = CF_B200_CODER_HUFFMAN_SPLIT4;
            else if (std::strcmp(env, "rans") != 0) a->kivi = true;   // not a coder name: the default stands
        }
        if (a->kivi) a->tile_tokens = options->page_size;
        try {
            if (a->kivi) a->kivi_create();
            else a->create_buffers();
            a->reset(nullptr);
        } catch (...) {
            delete a;
            return nullptr;  // no usable CUDA device: there is no host fallback
        }
        return a;
    } catch (...) {
        return nullptr;
    }
}

extern "C" void cf_llama_kv_destroy(cf_llama_kv_adapter *adapter) { delete adapter; }

extern "C" int cf_llama_kv_append(cf_llama_kv_adapter *adapter, uint32_t layer, uint32_t kv_head, uint32_t token_begin,
                                  const float *keys, const float *values, uint32_t token_count, void *stream) {
    return guarded(adapter, [&] {
        if (keys == nullptr || values == nullptr || token_count == 0) throw std::invalid_argument("invalid KV append");
        if (layer >= adapter->opt.layer_count || kv_head >= adapter->opt.kv_head_count)
            throw std::out_of_range("KV layer or head out of range");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        HeadState &h = adapter->head(layer, kv_head);
        if (h.started && token_begin != h.next_token) throw std::invalid_argument("KV append must be logically contiguous");
        if (h.flushed_partial && !adapter->kivi)
            throw std::runtime_error("append after a partial flush is not supported by the sealed format");
        if (!h.started) {
            h.started = true;
            h.next_token = token_begin;
        }
        const uint32_t D = adapter->opt.head_dim, T = adapter->tile_tokens;
        if (adapter->kivi) {   // rows into the [token][kv head][dim] tail the attention reads; a full tail becomes a page
            const size_t row = adapter->kivi_row_floats();
            uint32_t done = 0;
            while (done < token_count) {
                const uint32_t take = std::min(token_count - done, T - h.tail);
                const size_t at = static_cast<size_t>(h.tail) * row + static_cast<size_t>(kv_head) * D;
                cuda_check(cudaMemcpy2DAsync(adapter->kivi_tail(adapter->kivi_tail_k, layer) + at, row * 4, keys + static_cast<size_t>(done) * D,
                                             D * 4ull, D * 4ull, take, cudaMemcpyHostToDevice, s), "append keys");
                cuda_check(cudaMemcpy2DAsync(adapter->kivi_tail(adapter->kivi_tail_v, layer) + at, row * 4, values + static_cast<size_t>(done) * D,
                                             D * 4ull, D * 4ull, take, cudaMemcpyHostToDevice, s), "append values");
                h.tail += take;
                h.next_token += take;
                done += take;
                if (h.tail == T) adapter->kivi_seal(layer, kv_head, s);
            }
            h.appended += token_count;
            return;
        }
        const size_t tile = (static_cast<size_t>(layer) * adapter->opt.kv_head_count + kv_head) * adapter->tile_values();
        uint32_t done = 0;
        while (done < token_count) {
            const uint32_t take = std::min(token_count - done, T - h.tail);
            const size_t dst = tile + static_cast<size_t>(h.tail) * D;
            cuda_check(cudaMemcpyAsync(adapter->tail_k.ptr + dst, keys + static_cast<size_t>(done) * D, sizeof(float) * take * D,
                                       cudaMemcpyHostToDevice, s), "append keys");
            cuda_check(cudaMemcpyAsync(adapter->tail_v.ptr + dst, values + static_cast<size_t>(done) * D,
                                       sizeof(float) * take * D, cudaMemcpyHostToDevice, s), "append values");
            h.tail += take;
            done += take;
            if (h.tail == T) adapter->seal_tail(layer, kv_head, s);
        }
        h.appended += token_count;
        h.next_token += token_count;
    });
}

extern "C" int cf_llama_kv_attention(cf_llama_kv_adapter *adapter, uint32_t layer, const float *queries_device,
                                     float *output_device, uint32_t query_count, uint32_t query_head_count,
                                     uint32_t gqa_group_size, uint32_t query_token_begin, float softmax_scale,
                                     uint32_t causal_window, void *stream) {
    return guarded(adapter, [&] {
        if (queries_device == nullptr || output_device == nullptr || gqa_group_size == 0 || query_head_count == 0 ||
            query_head_count % gqa_group_size != 0)
            throw std::invalid_argument("invalid ChromoFold attention request");
        if (layer >= adapter->opt.layer_count) throw std::out_of_range("KV layer out of range");
        if (query_head_count != adapter->opt.query_head_count || gqa_group_size != adapter->opt.gqa_group_size ||
            query_count == 0 || query_count > cf_llama_kv_adapter::kMaxQueries)
            throw std::invalid_argument("invalid ChromoFold attention request");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const HeadState &h0 = adapter->head(layer, 0);
        for (uint32_t k = 1; k < adapter->opt.kv_head_count; ++k) {
            const HeadState &h = adapter->head(layer, k);
            if (h.sealed != h0.sealed || h.tail != h0.tail) throw std::runtime_error("KV active tails are not aligned across heads");
        }
        if (adapter->kivi) {   // the reference's own call over the reference's own page descriptors (its adapter, :107-131)
            cf_kv_paged_attention_desc desc{};
            desc.struct_size = sizeof desc;
            desc.abi_version = CF_KV_CUDA_ABI_VERSION;
            desc.pages = adapter->kivi_descs[layer]->ptr;
            desc.page_count = static_cast<uint32_t>(adapter->kivi_host_descs[layer].size());
            desc.kv_head_count = adapter->opt.kv_head_count;
            desc.query_head_count = query_head_count;
            desc.gqa_group_size = gqa_group_size;
            desc.active_k = h0.tail ? adapter->kivi_tail(adapter->kivi_tail_k, layer) : nullptr;
            desc.active_v = h0.tail ? adapter->kivi_tail(adapter->kivi_tail_v, layer) : nullptr;
            desc.active_token_begin = h0.next_token - h0.tail;
            desc.active_token_count = h0.tail;
            desc.queries = queries_device;
            desc.output = output_device;
            desc.query_token_begin = query_token_begin;
            desc.query_count = query_count;
            desc.head_dim = adapter->opt.head_dim;
            desc.causal_window = causal_window;
            desc.softmax_scale = softmax_scale;
            if (cf_kv_paged_attention_async(&desc, s) != CF_OK) throw std::runtime_error("ChromoFold paged attention launch rejected");
            return;
        }
        LayerState &ls = adapter->layers[layer];
        const uint32_t L = adapter->opt.layer_count;
        if (ls.device_sealed != h0.sealed || ls.device_tail != h0.tail) {
            cuda_check(cudaMemcpyAsync(adapter->scalars.ptr + layer, &h0.sealed, 4, cudaMemcpyHostToDevice, s), "sealed count");
            cuda_check(cudaMemcpyAsync(adapter->scalars.ptr + L + layer, &h0.tail, 4, cudaMemcpyHostToDevice, s), "tail count");
            ls.device_sealed = h0.sealed;
            ls.device_tail = h0.tail;
        }
        adapter->grow_positions(static_cast<size_t>(query_token_begin) + query_count + 1, s);

        cf_b200_sealed_attention_desc d{};
        d.struct_size = sizeof d;
        d.abi_version = CF_B200_ABI_VERSION;
        d.kv_head_count = adapter->opt.kv_head_count;
        d.query_head_count = query_head_count;
        d.head_dim = adapter->opt.head_dim;
        d.page_tokens = adapter->tile_tokens;
        d.block_size = 64;
        d.codebook_id = layer;
        d.arena = adapter->arena.ptr;
        d.page_dir = adapter->page_dir.ptr;
        d.page_table = adapter->page_table.ptr;
        d.seq_sealed_tokens = adapter->scalars.ptr;
        d.seq_slots = adapter->slots.ptr + static_cast<size_t>(layer) * cf_llama_kv_adapter::kMaxQueries;
        d.page_table_stride = adapter->stride;
        d.seq_count = query_count;
        d.k_tables = adapter->tables.ptr + 2 * layer;
        d.v_tables = adapter->tables.ptr + 2 * layer + 1;
        d.tail_k = adapter->tail_k.ptr;
        d.tail_v = adapter->tail_v.ptr;
        d.tail_tokens = adapter->scalars.ptr + L;
        d.tail_type = CF_B200_F32;
        d.query_positions = adapter->positions.ptr + query_token_begin;
        d.queries = queries_device;
        d.output = output_device;
        d.query_type = CF_B200_F32;
        d.output_type = CF_B200_F32;
        d.softmax_scale = softmax_scale;
        d.causal_window = causal_window;
        // Prefill (llama.cpp evaluates a prompt in batches of query tokens): they all see the layer's sealed records in
        // full, which the shared-prefix kernel then decodes once per 128 query rows instead of once per query token.
        // Only a hint (the plan kernel checks it), given where it pays and the workspace has or can get the room.
        if (query_count >= 4 && causal_window == 0) {
            const uint32_t tiles = std::min(h0.sealed / adapter->tile_tokens, (query_token_begin + 1u) / adapter->tile_tokens);
            if (tiles >= 8 && tiles <= adapter->stride) {
                cf_b200_sealed_attention_desc room = d;   // the workspace grows for the extra partials, up to 1 GiB
                room.shared_prefix_pages = 1;
                uint64_t bytes = 0;
                if (cf_b200_sealed_attention_workspace_bytes(&room, 65536, &bytes) == CF_OK && bytes + 256 <= (1ull << 30)) {
                    adapter->workspace.ensure(bytes + 256, s);
                    d.shared_prefix_pages = tiles;
                }
            }
        }
        const uintptr_t ws = reinterpret_cast<uintptr_t>(adapter->workspace.ptr);
        const uintptr_t aligned = (ws + 255) / 256 * 256;
        d.workspace = reinterpret_cast<void *>(aligned);
        d.workspace_bytes = adapter->workspace.count - (aligned - ws);
        d.status = adapter->status.ptr;
        if (cf_b200_sealed_attention_async(&d, s) != CF_OK) throw std::runtime_error("ChromoFold paged attention launch rejected");
    });
}

extern "C" int cf_llama_kv_attention_host(cf_llama_kv_adapter *adapter, uint32_t layer, const float *queries_host,
                                          float *output_host, uint32_t query_count, uint32_t query_head_count,
                                          uint32_t gqa_group_size, uint32_t query_token_begin, float softmax_scale,
                                          uint32_t causal_window, void *stream) {
    return guarded(adapter, [&] {
        if (queries_host == nullptr || output_host == nullptr) throw std::invalid_argument("null host attention buffer");
        const size_t bytes = static_cast<size_t>(query_count) * query_head_count * adapter->opt.head_dim * sizeof(float);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        float *dq = nullptr, *dout = nullptr;
        if (cudaMalloc(reinterpret_cast<void **>(&dq), bytes) != cudaSuccess ||
            cudaMalloc(reinterpret_cast<void **>(&dout), bytes) != cudaSuccess) {
            if (dq) cudaFree(dq);
            throw std::runtime_error("failed to allocate attention scratch");
        }
        cudaMemcpyAsync(dq, queries_host, bytes, cudaMemcpyHostToDevice, s);
        const int rc = cf_llama_kv_attention(adapter, layer, dq, dout, query_count, query_head_count, gqa_group_size,
                                             query_token_begin, softmax_scale, causal_window, stream);
        const std::string inner = adapter->last_error;
        if (rc == 0) {
            cudaMemcpyAsync(output_host, dout, bytes, cudaMemcpyDeviceToHost, s);
            cudaStreamSynchronize(s);
        }
        cudaFree(dq);
        cudaFree(dout);
        if (rc != 0) throw std::runtime_error(inner.empty() ? "attention failed" : inner);
    });
}

extern "C" int cf_llama_kv_flush(cf_llama_kv_adapter *adapter, void *stream) {
    return guarded(adapter, [&] {
        for (uint32_t layer = 0; layer < adapter->opt.layer_count; ++layer)
            for (uint32_t h = 0; h < adapter->opt.kv_head_count; ++h) {
                if (adapter->kivi) adapter->kivi_seal(layer, h, static_cast<cudaStream_t>(stream));
                else adapter->seal_tail(layer, h, static_cast<cudaStream_t>(stream));
            }
    });
}

extern "C" int cf_llama_kv_seq_rm(cf_llama_kv_adapter *adapter, uint64_t sequence_id) {
    return guarded(adapter, [&] {  // compressed_kv_cache.cu:180-183
        if (sequence_id != 0) throw std::invalid_argument("current ChromoFold cache supports sequence 0 only");
        cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        adapter->reset(nullptr);
    });
}

extern "C" int cf_llama_kv_seq_cp(cf_llama_kv_adapter *adapter, uint64_t source_id, uint64_t destination_id) {
    return guarded(adapter, [&] {  // compressed_kv_cache.cu:185-188
        if (source_id == destination_id) return;
        throw std::runtime_error("sequence copy requires the forthcoming shared-page table");
    });
}

extern "C" int cf_llama_kv_seq_shift(cf_llama_kv_adapter *adapter, uint64_t sequence_id, int32_t delta) {
    return guarded(adapter, [&] {  // compressed_kv_cache.cu:190-192
        if (sequence_id != 0 || delta != 0) throw std::runtime_error("non-zero context shift is not implemented");
    });
}

extern "C" int cf_llama_kv_clear(cf_llama_kv_adapter *adapter) {
    return guarded(adapter, [&] {
        cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        adapter->reset(nullptr);
    });
}

// Statistics in the reference's units (compressed_kv_cache.cu:198-210): a page is page_size tokens of one kv head.
extern "C" int cf_llama_kv_get_stats(const cf_llama_kv_adapter *adapter, cf_llama_kv_stats *stats) {
    if (adapter == nullptr || stats == nullptr) return -1;
    cf_llama_kv_stats out{};
    const uint32_t page = adapter->opt.page_size;
    for (const HeadState &h : adapter->heads) {
        out.appended_tokens += h.appended;
        const uint64_t whole = h.flushed_partial ? (h.sealed + page - 1) / page : h.sealed / page;
        const uint64_t sealed_tokens = h.flushed_partial ? h.sealed : whole * page;
        out.sealed_pages += whole;
        out.sealed_tokens += sealed_tokens;
        out.active_tokens += h.sealed + h.tail - sealed_tokens;
    }
    out.dense_active_bytes = out.active_tokens * adapter->opt.head_dim * 2 * sizeof(float);
    if (adapter->kivi) {
        out.compressed_bytes = adapter->kivi_resident_bytes;
        for (const auto &layer : adapter->kivi_host_descs) out.descriptor_bytes += layer.size() * sizeof(cf_kv_device_page);
    } else {
        unsigned long long units = 0;
        if (adapter->cursor.ptr) cudaMemcpy(&units, adapter->cursor.ptr, sizeof units, cudaMemcpyDeviceToHost);
        out.compressed_bytes = units * 16ull;
        out.descriptor_bytes = static_cast<uint64_t>(adapter->next_page_id) * adapter->opt.kv_head_count * sizeof(uint64_t);
    }
    *stats = out;
    return 0;
}

extern "C" const char *cf_llama_kv_last_error(const cf_llama_kv_adapter *adapter) {
    return adapter == nullptr ? "invalid ChromoFold KV adapter" : adapter->last_error.c_str();
}


// Additive: the device descriptor of a page of reference-exact mode (the reference's cf_kv_device_page: fixed-width words,
// K per-channel and V per-token fp32 scales), so that a test or a tool can read back exactly what was stored.
// page_index counts the pages of `layer` in the order they were sealed, over all kv heads. Returns -1 in format-v1 mode.
extern "C" uint64_t cf_b200_llama_kv_reserved_bytes(const cf_llama_kv_adapter *adapter) {
    return adapter ? static_cast<uint64_t>(adapter->kivi_chunks.size()) * cf_llama_kv_adapter::kKiviChunk : 0;
}

extern "C" int cf_b200_llama_kv_reference_page(const cf_llama_kv_adapter *adapter, uint32_t layer, uint32_t page_index,
                                               cf_kv_device_page *out_page) {
    if (adapter == nullptr || out_page == nullptr || !adapter->kivi || layer >= adapter->kivi_host_descs.size() ||
        page_index >= adapter->kivi_host_descs[layer].size())
        return -1;
    *out_page = adapter->kivi_host_descs[layer][page_index];
    return 0;
}
