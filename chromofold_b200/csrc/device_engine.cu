// device_engine.cu — the reference's device-resident KV ABIs (include/chromofold_b200/compat_device.h):
// cf_device_tensor_validate, cf_device_kv_* (src/cuda/device_kv_dataplane.cu) and cf_device_seal_*
// (src/cuda/device_kv_seal_attention.cu), both as thin fronts of one core: a single-sequence, multi-layer store whose
// active page lives on the GPU as fp32 rows, whose full pages are sealed by cf_b200_seal_pages_async and whose
// attention is cf_b200_sealed_attention_async.

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "cf_device_common.cuh"
#include "engine_common.cuh"

using namespace cfb_engine;

namespace {

struct CoreConfig { uint32_t layers, kv_heads, query_heads, head_dim, page_size, group; };

struct LayerHost {
    uint32_t active_begin = 0, active_count = 0;   // the unsealed page: first token and rows held
    uint32_t sealed_tokens = 0;                    // tokens in sealed tiles
    uint32_t base = 0;                             // logical position of the layer's first stored token (its first append's)
    uint32_t state = CF_SEAL_ACTIVE_FILLING;
    uint64_t generation = 0;
    bool calibrated = false;
    uint32_t descriptor_capacity = 0;              // pages the reference's descriptor table would hold (0, 4, 8, 16, ...)
    std::vector<uint32_t> page_ids;                // tile index -> page id
    uint32_t dev_sealed = 0xffffffffu, dev_tail = 0xffffffffu;
};

// What a seal reports back to the ABI front that called it.
struct SealReport { uint64_t values = 0, bytes_written = 0; bool nonfinite = false, table_grew = false; };

struct Core {
    static constexpr uint32_t kMaxQueries = 4096;
    CoreConfig cfg{};
    uint32_t tile = 0, tiles_per_page = 0;
    std::vector<LayerHost> layers;
    bool ready = false;
    uint32_t next_page_id = 1, stride = 1024;
    uint64_t sealed_records = 0, bytes_sealed = 0;
    Buffer<uint8_t> arena, workspace;
    Buffer<uint64_t> page_dir;
    Buffer<uint32_t> page_table, scalars, slots, positions, jobs, status;
    Buffer<float> tail_k, tail_v, q_dense, o_dense;
    Buffer<cf_b200_codebook_tables> tables;
    Buffer<unsigned long long> cursor;  // [0] arena cursor, [1..512] histograms

    explicit Core(const CoreConfig &c) : cfg(c), layers(c.layers) {
        tile = choose_tile_tokens(c.page_size, c.head_dim);
        tiles_per_page = c.page_size / tile;
    }
    size_t page_values() const { return static_cast<size_t>(cfg.kv_heads) * cfg.page_size * cfg.head_dim; }
    size_t max_record_bytes() const { return 16 + 2 * ((static_cast<size_t>(tile) * cfg.head_dim + 15) / 16 * 16); }
    uint64_t owned_bytes() const {
        return arena.bytes() + workspace.bytes() + page_dir.bytes() + page_table.bytes() + tail_k.bytes() + tail_v.bytes() +
               tables.bytes() + q_dense.bytes() + o_dense.bytes();
    }

    // Device memory is taken on first use, so handles can be created (and their contracts tested) without a GPU.
    void ensure_ready(cudaStream_t s) {
        if (ready) return;
        const uint32_t L = cfg.layers;
        page_table.ensure(static_cast<size_t>(L) * stride, s);
        scalars.ensure(2 * L, s);
        tail_k.ensure(L * page_values(), s);
        tail_v.ensure(L * page_values(), s);
        tables.ensure(2 * L, s);
        cursor.ensure(513, s);
        status.ensure(1, s);
        jobs.ensure(5 * 256, s);
        arena.ensure(16u << 20, s);
        page_dir.ensure(static_cast<size_t>(4096) * cfg.kv_heads, s);
        std::vector<uint32_t> host(static_cast<size_t>(L) * kMaxQueries);
        for (uint32_t l = 0; l < L; ++l) std::fill_n(host.begin() + static_cast<size_t>(l) * kMaxQueries, kMaxQueries, l);
        slots.ensure(host.size(), s);
        cuda_check(cudaMemcpyAsync(slots.ptr, host.data(), host.size() * 4, cudaMemcpyHostToDevice, s), "upload slots");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        grow_positions(1u << 16, s);
        cf_b200_sealed_attention_desc d{};
        d.kv_head_count = cfg.kv_heads;
        d.query_head_count = cfg.query_heads;
        d.head_dim = cfg.head_dim;
        d.seq_count = kMaxQueries;
        uint64_t bytes = 0;
        cf_b200_sealed_attention_workspace_bytes(&d, 65536, &bytes);
        workspace.ensure(bytes + 256, s);
        ready = true;
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
    float *tail_of(Buffer<float> &b, uint32_t layer) { return b.ptr + layer * page_values(); }
};

}  // namespace

namespace {

// Rows of a strided view into the active page of `layer`, starting at active row `row0`.
void core_copy_rows(Core &c, uint32_t layer, const cf_device_tensor_view &k, const cf_device_tensor_view &v, uint32_t row0,
                    cudaStream_t s) {
    c.ensure_ready(s);
    const uint64_t count = static_cast<uint64_t>(k.token_count) * k.head_count * k.head_dim;
    const int threads = 256, blocks = static_cast<int>((count + threads - 1) / threads);
    rows_to_tail_kernel<<<blocks, threads, 0, s>>>(k, c.tail_of(c.tail_k, layer), c.cfg.page_size, row0);
    rows_to_tail_kernel<<<blocks, threads, 0, s>>>(v, c.tail_of(c.tail_v, layer), c.cfg.page_size, row0);
    cuda_check(cudaGetLastError(), "device KV conversion launch");
}

cf_b200_seal_desc core_seal_desc(Core &c, uint32_t layer) {
    cf_b200_seal_desc d{};
    d.struct_size = sizeof d;
    d.abi_version = CF_B200_ABI_VERSION;
    d.kv_head_count = c.cfg.kv_heads;
    d.head_dim = c.cfg.head_dim;
    d.page_tokens = c.tile;
    d.block_size = 64;
    d.coder = engine_coder(c.tile * c.cfg.head_dim);
    d.codebook_id = layer;
    d.k_tables = c.tables.ptr + 2 * layer;
    d.v_tables = c.tables.ptr + 2 * layer + 1;
    d.tail_k = c.tail_k.ptr;
    d.tail_v = c.tail_v.ptr;
    d.tail_type = CF_B200_F32;
    d.tail_capacity = c.cfg.page_size;
    d.arena = c.arena.ptr;
    d.arena_units = c.arena.count / 16;
    d.arena_cursor_units = c.cursor.ptr;
    d.page_dir = c.page_dir.ptr;
    d.status = c.status.ptr;
    return d;
}

// Seal the full active page of `layer`: tiles_per_page jobs, every kv head. `inject(point)` is the front's host-side
// fault hook; it throws to abort. Everything before the publish step leaves host and device tables untouched.
template <class Inject>
SealReport core_seal_page(Core &c, uint32_t layer, cudaStream_t s, Inject inject) {
    c.ensure_ready(s);
    LayerHost &L = c.layers[layer];
    SealReport report;
    report.values = 2ull * c.page_values();
    inject(CF_SEAL_FAULT_CANDIDATE_ALLOC);
    const uint32_t n = c.tiles_per_page;
    const uint32_t first_tile = L.sealed_tokens / c.tile;
    L.state = CF_SEAL_VALIDATING;
    inject(CF_SEAL_FAULT_FINITE_VALIDATION);
    // room: arena by the worst-case record size, directory by page count, page table by tile index
    c.arena.ensure((c.sealed_records + static_cast<uint64_t>(n) * c.cfg.kv_heads) * c.max_record_bytes() + 4096, s);
    c.page_dir.ensure(static_cast<size_t>(c.next_page_id + n + 1) * c.cfg.kv_heads, s);
    if (first_tile + n > c.stride) {
        uint32_t wider = c.stride;
        while (first_tile + n > wider) wider *= 2;
        Buffer<uint32_t> fresh;
        fresh.ensure(static_cast<size_t>(c.cfg.layers) * wider, s);
        cuda_check(cudaMemcpy2DAsync(fresh.ptr, wider * 4, c.page_table.ptr, c.stride * 4, c.stride * 4, c.cfg.layers,
                                     cudaMemcpyDeviceToDevice, s), "widen page table");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        std::swap(fresh.ptr, c.page_table.ptr);
        std::swap(fresh.count, c.page_table.count);
        c.stride = wider;
    }
    // job arrays: slot (= layer), page id, rows, first row
    std::vector<uint32_t> host(4 * n);
    for (uint32_t j = 0; j < n; ++j) {
        host[j] = layer;
        host[n + j] = c.next_page_id + j;
        host[2 * n + j] = c.tile;
        host[3 * n + j] = j * c.tile;
    }
    c.jobs.ensure(4 * n, s);
    cuda_check(cudaMemcpyAsync(c.jobs.ptr, host.data(), host.size() * 4, cudaMemcpyHostToDevice, s), "upload seal jobs");
    cf_b200_seal_desc d = core_seal_desc(c, layer);
    d.job_slots = c.jobs.ptr;
    d.job_pages = c.jobs.ptr + n;
    d.job_tokens = c.jobs.ptr + 2 * n;
    d.job_rows = c.jobs.ptr + 3 * n;
    d.job_count = n;
    if (!L.calibrated) {  // first page of the layer: histogram its symbols, build the layer's codebooks
        cuda_check(cudaMemsetAsync(c.cursor.ptr + 1, 0, 512 * sizeof(unsigned long long), s), "clear histograms");
        if (cf_b200_histogram_async(&d, c.cursor.ptr + 1, c.cursor.ptr + 257, s) != CF_OK)
            throw std::runtime_error("histogram launch rejected");
        unsigned long long hist[512];
        cuda_check(cudaMemcpyAsync(hist, c.cursor.ptr + 1, sizeof hist, cudaMemcpyDeviceToHost, s), "read histograms");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        std::vector<cf_b200_codebook_tables> tables(2);
        uint64_t hk[256], hv[256];
        for (int i = 0; i < 256; ++i) { hk[i] = hist[i]; hv[i] = hist[256 + i]; }
        if (cf_b200_codebook_build(hk, &tables[0]) != CF_OK || cf_b200_codebook_build(hv, &tables[1]) != CF_OK)
            throw std::runtime_error("codebook build failed");
        cuda_check(cudaMemcpyAsync(c.tables.ptr + 2 * layer, tables.data(), 2 * sizeof(cf_b200_codebook_tables),
                                   cudaMemcpyHostToDevice, s), "upload codebooks");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        L.calibrated = true;
    }
    unsigned long long cursor_before = 0;
    cuda_check(cudaMemcpyAsync(&cursor_before, c.cursor.ptr, sizeof cursor_before, cudaMemcpyDeviceToHost, s), "read cursor");
    c.sealed_records += static_cast<uint64_t>(n) * c.cfg.kv_heads;  // arena room is budgeted per launch, kept or not
    if (cf_b200_seal_pages_async(&d, s) != CF_OK) throw std::runtime_error("seal launch rejected");
    // The reference learns about NaN / Inf through a synchronisation right after its finite scan, before any later
    // fault point (device_kv_seal_attention.cu:262-268); so does this front: the device status word and the arena cursor
    // of the one fused launch come back together, and a page that is not finite is refused whatever fault is armed
    // beyond FINITE_VALIDATION.
    uint32_t status = 0;
    unsigned long long cursor_after = 0;
    cuda_check(cudaMemcpyAsync(&status, c.status.ptr, 4, cudaMemcpyDeviceToHost, s), "read status");
    cuda_check(cudaMemcpyAsync(&cursor_after, c.cursor.ptr, sizeof cursor_after, cudaMemcpyDeviceToHost, s), "read cursor");
    cuda_check(cudaStreamSynchronize(s), "finite validation sync");
    report.bytes_written = (cursor_after - cursor_before) * 16ull;
    auto unpublish = [&] {  // directory entries of the candidate pages back to "not there"; the bytes stay as garbage
        cuda_check(cudaMemsetAsync(c.page_dir.ptr + static_cast<size_t>(c.next_page_id) * c.cfg.kv_heads, 0,
                                   static_cast<size_t>(n) * c.cfg.kv_heads * sizeof(uint64_t), s), "unpublish");
        cuda_check(cudaMemsetAsync(c.status.ptr, 0, 4, s), "clear status");
    };
    if (status & (CF_B200_DEVSTAT_NONFINITE | CF_B200_DEVSTAT_ARENA_FULL)) {
        unpublish();
        report.nonfinite = (status & CF_B200_DEVSTAT_NONFINITE) != 0;
        throw std::runtime_error(report.nonfinite ? "active page contains NaN or Inf" : "arena is full");
    }
    try {   // the later fault points, in the reference's order (:270-312)
        L.state = CF_SEAL_QUANTIZING;
        inject(CF_SEAL_FAULT_SCALE_ALLOC);
        inject(CF_SEAL_FAULT_QUANTIZE_LAUNCH);
        L.state = CF_SEAL_PACKING;
        inject(CF_SEAL_FAULT_PAYLOAD_ALLOC);
        inject(CF_SEAL_FAULT_PACK_LAUNCH);
        inject(CF_SEAL_FAULT_DESCRIPTOR_VALIDATE);
        L.state = CF_SEAL_PUBLISHING;
        // PAGE_TABLE_GROW fires where the reference's descriptor table would grow: at a layer's 1st, 5th, 9th, 17th ...
        // page (capacity 0 -> 4 -> 8 -> 16 ..., :300-307); a growth that happened stays even if a later point aborts
        const uint32_t needed = L.sealed_tokens / c.cfg.page_size + 1u;
        if (needed > L.descriptor_capacity) {
            inject(CF_SEAL_FAULT_PAGE_TABLE_GROW);
            uint32_t next = std::max<uint32_t>(4u, L.descriptor_capacity ? L.descriptor_capacity * 2u : 4u);
            while (next < needed) next *= 2u;
            L.descriptor_capacity = next;
            report.table_grew = true;
        }
        inject(CF_SEAL_FAULT_ACTIVE_REPLACEMENT);
        inject(CF_SEAL_FAULT_DESCRIPTOR_PUBLISH);
    } catch (...) {
        unpublish();
        throw;
    }
    // publish: page ids into the layer's page table row, then host bookkeeping
    cuda_check(cudaMemcpyAsync(c.page_table.ptr + static_cast<size_t>(layer) * c.stride + first_tile, host.data() + n, n * 4,
                               cudaMemcpyHostToDevice, s), "publish page ids");
    for (uint32_t j = 0; j < n; ++j) L.page_ids.push_back(c.next_page_id + j);
    c.next_page_id += n;
    c.bytes_sealed += report.bytes_written;
    L.sealed_tokens += c.cfg.page_size;
    L.active_begin += L.active_count;
    L.active_count = 0;
    L.generation++;
    L.state = CF_SEAL_ACTIVE_FILLING;
    return report;
}

// Attention of `count` query rows at positions query_begin.. over layer `layer`. q: contiguous [count][Hq][D] of
// q_type (F16 or F32); out: contiguous fp32.
void core_attention(Core &c, uint32_t layer, const void *q, uint32_t q_type, float *out, uint32_t count, uint32_t query_begin,
                    float softmax_scale, uint32_t window, cudaStream_t s) {
    c.ensure_ready(s);
    if (count == 0 || count > Core::kMaxQueries) throw std::runtime_error("query token count out of range");
    LayerHost &L = c.layers[layer];
    const uint32_t N = c.cfg.layers;
    if (L.dev_sealed != L.sealed_tokens || L.dev_tail != L.active_count) {
        cuda_check(cudaMemcpyAsync(c.scalars.ptr + layer, &L.sealed_tokens, 4, cudaMemcpyHostToDevice, s), "sealed count");
        cuda_check(cudaMemcpyAsync(c.scalars.ptr + N + layer, &L.active_count, 4, cudaMemcpyHostToDevice, s), "tail count");
        L.dev_sealed = L.sealed_tokens;
        L.dev_tail = L.active_count;
    }
    c.grow_positions(static_cast<size_t>(query_begin) + count + 1, s);
    cf_b200_sealed_attention_desc d{};
    d.struct_size = sizeof d;
    d.abi_version = CF_B200_ABI_VERSION;
    d.kv_head_count = c.cfg.kv_heads;
    d.query_head_count = c.cfg.query_heads;
    d.head_dim = c.cfg.head_dim;
    d.page_tokens = c.tile;
    d.block_size = 64;
    d.codebook_id = layer;
    d.arena = c.arena.ptr;
    d.page_dir = c.page_dir.ptr;
    d.page_table = c.page_table.ptr;
    d.seq_sealed_tokens = c.scalars.ptr;
    d.seq_slots = c.slots.ptr + static_cast<size_t>(layer) * Core::kMaxQueries;
    d.page_table_stride = c.stride;
    d.seq_count = count;
    d.k_tables = c.tables.ptr + 2 * layer;
    d.v_tables = c.tables.ptr + 2 * layer + 1;
    d.tail_k = c.tail_k.ptr;
    d.tail_v = c.tail_v.ptr;
    d.tail_tokens = c.scalars.ptr + N;
    d.tail_type = CF_B200_F32;
    d.tail_capacity = c.cfg.page_size;
    d.query_positions = c.positions.ptr + query_begin;
    d.queries = q;
    d.query_type = q_type;
    d.output = out;
    d.output_type = CF_B200_F32;
    d.softmax_scale = softmax_scale;
    d.causal_window = window;
    // Prefill: the query tokens of one call all see the layer's sealed records in full, so those records are decoded
    // once per 128 query rows by the shared-prefix kernel instead of once per query token. Only a hint (the plan kernel
    // checks it), given where it pays and where the workspace has or can get room for the extra partials.
    if (count >= 4 && window == 0) {
        const uint32_t tiles = std::min(L.sealed_tokens / c.tile, (query_begin + 1u) / c.tile);
        if (tiles >= 8 && tiles <= c.stride && shared_prefix_room(c.workspace, count, c.cfg.kv_heads, c.cfg.query_heads, c.cfg.head_dim, s))
            d.shared_prefix_pages = tiles;
    }
    const uintptr_t ws = reinterpret_cast<uintptr_t>(c.workspace.ptr), aligned = (ws + 255) / 256 * 256;
    d.workspace = reinterpret_cast<void *>(aligned);
    d.workspace_bytes = c.workspace.count - (aligned - ws);
    d.status = c.status.ptr;
    if (cf_b200_sealed_attention_async(&d, s) != CF_OK) throw std::runtime_error("compressed attention launch rejected");
}

void core_clear(Core &c, cudaStream_t s) {
    for (auto &L : c.layers) L = LayerHost{};
    c.next_page_id = 1;
    c.sealed_records = c.bytes_sealed = 0;
    if (!c.ready) return;
    cuda_check(cudaMemsetAsync(c.cursor.ptr, 0, sizeof(unsigned long long), s), "clear cursor");
    cuda_check(cudaMemsetAsync(c.page_dir.ptr, 0, c.page_dir.bytes(), s), "clear directory");
    cuda_check(cudaMemsetAsync(c.status.ptr, 0, 4, s), "clear status");
}

bool config_ok(uint32_t layers, uint32_t kv, uint32_t q, uint32_t dim, uint32_t page, uint32_t group) {
    return layers && kv && q && dim && page && group && q == kv * group && dim <= CF_KV_MAX_HEAD_DIM && group <= 16;
}

bool view_is_dense(const cf_device_tensor_view &v) {
    const uint64_t w = scalar_bytes(v.scalar_type);
    return v.element_stride_bytes == w && v.head_stride_bytes == w * v.head_dim &&
           v.token_stride_bytes == w * v.head_dim * v.head_count;
}

}  // namespace

// ------------------------------------------------------------------------------------------------------------------
// cf_device_tensor_validate + cf_device_kv_*  (src/cuda/device_kv_dataplane.cu:112-247)
// ------------------------------------------------------------------------------------------------------------------
struct cf_device_kv_dataplane {
    Core core;
    cf_device_kv_config config{};
    cf_device_kv_counters counters{};
    std::string last_error;
    explicit cf_device_kv_dataplane(const cf_device_kv_config &c)
        : core(CoreConfig{c.layer_count, c.kv_head_count, c.query_head_count, c.head_dim, c.page_size, c.gqa_group_size}), config(c) {}
    void account() {
        counters.active_bytes = core.tail_k.bytes() + core.tail_v.bytes();
        counters.compressed_bytes = core.bytes_sealed;
        counters.descriptor_bytes = core.page_dir.bytes() + core.page_table.bytes();
        counters.workspace_bytes = core.workspace.bytes();
        counters.peak_owned_bytes = std::max<uint64_t>(counters.peak_owned_bytes, core.owned_bytes());
    }
};

extern "C" int cf_device_tensor_validate(const cf_device_tensor_view *v) {
    if (!v || !v->data || v->token_count == 0 || v->head_count == 0 || v->head_dim == 0) return -1;
    const uint64_t w = scalar_bytes(v->scalar_type);
    if (w == 0 || v->element_stride_bytes < w) return -1;
    const uint64_t row = static_cast<uint64_t>(v->head_dim - 1) * v->element_stride_bytes + w;
    if (v->head_stride_bytes < row) return -1;
    if (v->token_stride_bytes < static_cast<uint64_t>(v->head_count - 1) * v->head_stride_bytes + row) return -1;
    return 0;
}

extern "C" cf_device_kv_dataplane *cf_device_kv_create(const cf_device_kv_config *c) {
    if (!c || !config_ok(c->layer_count, c->kv_head_count, c->query_head_count, c->head_dim, c->page_size, c->gqa_group_size))
        return nullptr;
    try { return new cf_device_kv_dataplane(*c); } catch (...) { return nullptr; }
}

extern "C" void cf_device_kv_destroy(cf_device_kv_dataplane *p, void *) { delete p; }

extern "C" int cf_device_kv_append_async(cf_device_kv_dataplane *p, uint32_t layer, uint32_t token_begin,
                                         const cf_device_tensor_view *keys, const cf_device_tensor_view *values, void *stream) {
    if (!p || layer >= p->core.layers.size() || cf_device_tensor_validate(keys) != 0 || cf_device_tensor_validate(values) != 0)
        return -1;
    try {
        if (keys->token_count != values->token_count || keys->head_count != values->head_count ||
            keys->head_dim != values->head_dim || keys->head_count != p->config.kv_head_count ||
            keys->head_dim != p->config.head_dim)
            throw std::runtime_error("device K/V topology mismatch");
        LayerHost &L = p->core.layers[layer];
        const uint32_t next = L.active_begin + L.active_count;
        if ((L.active_count != 0 || L.sealed_tokens != 0) && token_begin != next)
            throw std::runtime_error("non-contiguous device token append");
        // The reference adopts the caller's position whenever the active page is empty (src/cuda/device_kv_dataplane.cu:160-168).
        // Sealed records here carry no position, so a layer's tokens stay contiguous: the first append fixes where the
        // layer starts, and an append after a seal has to continue it (a gap is the one thing that is still refused).
        if (L.active_count + keys->token_count > p->config.page_size)
            throw std::runtime_error("append crosses active page boundary; seal before retry");
        if (L.active_count == 0 && L.sealed_tokens == 0) {
            L.active_begin = token_begin;
            L.base = token_begin;
        }
        core_copy_rows(p->core, layer, *keys, *values, L.active_count, static_cast<cudaStream_t>(stream));
        L.active_count += keys->token_count;
        L.state = L.active_count == p->config.page_size ? CF_SEAL_ACTIVE_FULL : CF_SEAL_ACTIVE_FILLING;
        const uint64_t n = static_cast<uint64_t>(keys->token_count) * keys->head_count * keys->head_dim;
        for (const cf_device_tensor_view *v : {keys, values}) {
            if (v->scalar_type == CF_DEVICE_F16) p->counters.fp16_values_converted += n;
            else if (v->scalar_type == CF_DEVICE_BF16) p->counters.bf16_values_converted += n;
            else p->counters.fp32_values_copied += n;
        }
        p->counters.device_append_calls++;
        p->counters.device_values_appended += 2 * n;
        p->account();
        p->last_error.clear();
        return 0;
    } catch (const std::exception &e) {
        p->last_error = e.what();
        p->counters.cuda_errors++;
        return -1;
    }
}

extern "C" int cf_device_kv_seal_full_pages_async(cf_device_kv_dataplane *p, void *stream) {
    if (!p) return -1;
    p->counters.seal_attempts++;
    try {
        for (uint32_t layer = 0; layer < p->core.layers.size(); ++layer) {
            if (p->core.layers[layer].active_count != p->config.page_size) continue;
            core_seal_page(p->core, layer, static_cast<cudaStream_t>(stream), [](uint32_t) {});
            p->counters.quantization_launches++;
            p->counters.huffman_pack_launches++;
            p->counters.descriptor_publications++;
            p->counters.seal_successes++;
        }
        p->account();
        p->last_error.clear();
        return 0;
    } catch (const std::exception &e) {
        for (auto &L : p->core.layers)
            if (L.state != CF_SEAL_ACTIVE_FILLING) L.state = CF_SEAL_ACTIVE_FULL;
        p->last_error = e.what();
        p->counters.seal_failures++;
        return -1;
    }
}

extern "C" int cf_device_kv_attention_async(cf_device_kv_dataplane *p, uint32_t layer, const float *query, float *output,
                                            uint32_t query_token_count, uint32_t query_token_begin, float softmax_scale,
                                            uint32_t causal_window, void *stream) {
    if (!p || layer >= p->core.layers.size() || !query || !output) return -1;
    try {
        const LayerHost &L = p->core.layers[layer];
        if (query_token_begin < L.base) throw std::runtime_error("query position lies before the layer's first token");
        core_attention(p->core, layer, query, CF_B200_F32, output, query_token_count, query_token_begin - L.base, softmax_scale,
                       causal_window, static_cast<cudaStream_t>(stream));
        p->counters.compressed_attention_launches++;
        p->counters.sealed_values_consumed += 2ull * L.sealed_tokens * p->config.kv_head_count * p->config.head_dim;
        p->counters.active_values_consumed += 2ull * L.active_count * p->config.kv_head_count * p->config.head_dim;
        p->last_error.clear();
        return 0;
    } catch (const std::exception &e) {
        p->last_error = e.what();
        p->counters.cuda_errors++;
        return -1;
    }
}

extern "C" int cf_device_kv_clear_async(cf_device_kv_dataplane *p, void *stream) {
    if (!p) return -1;
    try {
        core_clear(p->core, static_cast<cudaStream_t>(stream));
        p->account();
        return 0;
    } catch (const std::exception &e) {
        p->last_error = e.what();
        return -1;
    }
}

extern "C" int cf_device_kv_get_counters(const cf_device_kv_dataplane *p, cf_device_kv_counters *out) {
    if (!p || !out) return -1;
    *out = p->counters;
    return 0;
}

extern "C" const char *cf_device_kv_last_error(const cf_device_kv_dataplane *p) {
    return p ? p->last_error.c_str() : "null device KV dataplane";
}

// ------------------------------------------------------------------------------------------------------------------
// cf_device_seal_*  (src/cuda/device_kv_seal_attention.cu:203-373)
// ------------------------------------------------------------------------------------------------------------------
struct cf_device_seal_engine {
    Core core;
    cf_device_seal_config config{};
    cf_device_seal_counters counters{};
    uint32_t fault = CF_SEAL_FAULT_NONE;
    std::string error;
    explicit cf_device_seal_engine(const cf_device_seal_config &c)
        : core(CoreConfig{c.layer_count, c.kv_head_count, c.query_head_count, c.head_dim, c.page_size, c.gqa_group_size}), config(c) {}
};

extern "C" cf_device_seal_engine *cf_device_seal_create(const cf_device_seal_config *c) {
    if (!c || !c->block_size ||
        !config_ok(c->layer_count, c->kv_head_count, c->query_head_count, c->head_dim, c->page_size, c->gqa_group_size))
        return nullptr;
    try { return new cf_device_seal_engine(*c); } catch (...) { return nullptr; }
}

extern "C" void cf_device_seal_destroy(cf_device_seal_engine *e, void *) { delete e; }

extern "C" int cf_device_seal_stage_active_page(cf_device_seal_engine *e, uint32_t layer, uint32_t token_begin, const float *k,
                                                const float *v, uint32_t token_count, void *stream) {
    if (!e || layer >= e->core.layers.size() || !k || !v || !token_count || token_count > e->config.page_size) return -1;
    try {
        // the staged rows replace the active page: [token][kv head][dim] fp32 on the device (:228-242)
        cf_device_tensor_view view{};
        view.scalar_type = CF_DEVICE_F32;
        view.token_count = token_count;
        view.head_count = e->config.kv_head_count;
        view.head_dim = e->config.head_dim;
        view.element_stride_bytes = 4;
        view.head_stride_bytes = 4ull * view.head_dim;
        view.token_stride_bytes = view.head_stride_bytes * view.head_count;
        cf_device_tensor_view kv = view, vv = view;
        kv.data = k;
        vv.data = v;
        LayerHost &L = e->core.layers[layer];
        // The reference stages a page at any position (:233-241). Sealed tiles carry no position of their own here, so a
        // layer's history is contiguous from the position of its first page: a layer without sealed pages takes any
        // position, one with sealed pages only the next one.
        if (L.sealed_tokens == 0) L.base = token_begin;
        else if (token_begin != L.base + L.sealed_tokens)
            throw std::runtime_error("active page must continue the sealed history of the layer");
        core_copy_rows(e->core, layer, kv, vv, 0, static_cast<cudaStream_t>(stream));
        L.active_begin = token_begin;
        L.active_count = token_count;
        L.state = token_count == e->config.page_size ? CF_SEAL_ACTIVE_FULL : CF_SEAL_ACTIVE_FILLING;
        e->counters.workspace_bytes = e->core.workspace.bytes();
        e->error.clear();
        return 0;
    } catch (const std::exception &ex) {
        e->error = ex.what();
        e->counters.cuda_errors++;
        return -1;
    }
}

extern "C" int cf_device_seal_full_page_async(cf_device_seal_engine *e, uint32_t layer, void *stream) {
    if (!e || layer >= e->core.layers.size()) return -1;
    LayerHost &L = e->core.layers[layer];
    cf_device_seal_counters &n = e->counters;
    n.seal_attempts++;
    if (L.active_count != e->config.page_size || L.state != CF_SEAL_ACTIVE_FULL) {
        e->error = "layer does not contain a full active page";
        n.seal_failures++;
        return -1;
    }
    try {
        // One launch does what the reference splits over finite_scan, quantize and pack launches; the counters are booked
        // where the reference books them, so an attempt that a later fault point aborts still counts the work it passed
        // (device_kv_seal_attention.cu:262, 275, 284, 298).
        const uint64_t values = 2ull * e->core.page_values();
        const SealReport r = core_seal_page(e->core, layer, static_cast<cudaStream_t>(stream), [&](uint32_t point) {
            if (point == CF_SEAL_FAULT_FINITE_VALIDATION) { n.finite_validation_launches++; n.values_scanned += values; }
            if (point == CF_SEAL_FAULT_QUANTIZE_LAUNCH) { n.quantization_launches++; n.values_quantized += values; }
            if (point == CF_SEAL_FAULT_PACK_LAUNCH) { n.packing_launches++; n.symbols_packed += values; }
            if (point == CF_SEAL_FAULT_DESCRIPTOR_VALIDATE) n.descriptor_validations++;
            if (e->fault == point) throw std::runtime_error("injected transactional seal failure");
        });
        if (r.table_grew) n.page_table_reallocations++;
        n.payload_bytes_written += r.bytes_written;
        n.descriptor_publications++;
        n.page_table_generation = L.generation;
        n.seal_successes++;
        n.compressed_bytes += r.bytes_written;
        n.descriptor_bytes = e->core.page_dir.bytes() + e->core.page_table.bytes();
        n.workspace_bytes = e->core.workspace.bytes();
        n.peak_owned_bytes = std::max<uint64_t>(n.peak_owned_bytes, e->core.owned_bytes());
        e->error.clear();
        return 0;
    } catch (const std::exception &ex) {
        L.state = CF_SEAL_ACTIVE_FULL;  // the active page is intact, the table generation unchanged (:328-333)
        e->error = ex.what();
        n.seal_failures++;
        if (e->error == "active page contains NaN or Inf") {
            n.invalid_pages_rejected++;
            n.nan_values++;  // the device reports "not finite" as one flag; it is booked here
        }
        return -1;
    }
}

extern "C" int cf_device_seal_attention_async(cf_device_seal_engine *e, uint32_t layer, const cf_device_tensor_view *query,
                                              void *output, uint32_t output_type, uint64_t ots, uint64_t ohs, uint64_t oes,
                                              uint32_t query_begin, float softmax_scale, uint32_t window, void *stream) {
    if (!e || layer >= e->core.layers.size() || cf_device_tensor_validate(query) != 0 || !output || !scalar_bytes(output_type))
        return -1;
    try {
        Core &c = e->core;
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        if (query->head_count != e->config.query_head_count || query->head_dim != e->config.head_dim)
            throw std::runtime_error("query topology mismatch");
        const uint64_t ow = scalar_bytes(output_type);
        if (ots < static_cast<uint64_t>(query->head_count - 1) * ohs + static_cast<uint64_t>(query->head_dim - 1) * oes + ow)
            throw std::runtime_error("output stride is too small");
        c.ensure_ready(s);
        const uint64_t count = static_cast<uint64_t>(query->token_count) * query->head_count * query->head_dim;
        const int threads = 256, blocks = static_cast<int>((count + threads - 1) / threads);
        const void *q = query->data;
        uint32_t q_type = query->scalar_type == CF_DEVICE_F16 ? CF_B200_F16 : CF_B200_F32;
        if (query->scalar_type == CF_DEVICE_BF16 || !view_is_dense(*query)) {  // gather / widen into a dense fp32 copy
            c.q_dense.ensure(count, s);
            view_to_dense_kernel<<<blocks, threads, 0, s>>>(*query, c.q_dense.ptr);
            cuda_check(cudaGetLastError(), "query conversion launch");
            q = c.q_dense.ptr;
            q_type = CF_B200_F32;
        }
        const bool out_dense = output_type == CF_DEVICE_F32 && oes == 4 && ohs == 4ull * query->head_dim &&
                               ots == ohs * query->head_count;
        float *out = static_cast<float *>(output);
        if (!out_dense) {
            c.o_dense.ensure(count, s);
            out = c.o_dense.ptr;
        }
        const uint32_t first_position = c.layers[layer].base;
        if (query_begin < first_position) throw std::runtime_error("query position lies before the layer's first token");
        core_attention(c, layer, q, q_type, out, query->token_count, query_begin - first_position, softmax_scale, window, s);
        if (!out_dense) {
            dense_to_view_kernel<<<blocks, threads, 0, s>>>(out, output, output_type, query->token_count, query->head_count,
                                                            query->head_dim, ots, ohs, oes);
            cuda_check(cudaGetLastError(), "output conversion launch");
        }
        const LayerHost &L = c.layers[layer];
        cf_device_seal_counters &n = e->counters;
        n.compressed_attention_launches++;
        n.sealed_pages_consumed += L.sealed_tokens / e->config.page_size;
        n.sealed_values_consumed += 2ull * L.sealed_tokens * e->config.kv_head_count * e->config.head_dim;
        n.active_values_consumed += 2ull * L.active_count * e->config.kv_head_count * e->config.head_dim;
        if (query->scalar_type != CF_DEVICE_F32) n.query_conversion_launches++;
        if (output_type != CF_DEVICE_F32) n.output_conversion_launches++;
        e->error.clear();
        return 0;
    } catch (const std::exception &ex) {
        e->error = ex.what();
        e->counters.cuda_errors++;
        return -1;
    }
}

extern "C" int cf_device_seal_clear_async(cf_device_seal_engine *e, void *stream) {
    if (!e) return -1;
    try {
        core_clear(e->core, static_cast<cudaStream_t>(stream));
        e->counters.compressed_bytes = e->counters.descriptor_bytes = 0;
        return 0;
    } catch (const std::exception &ex) {
        e->error = ex.what();
        return -1;
    }
}

extern "C" int cf_device_seal_set_fault(cf_device_seal_engine *e, uint32_t fault) {
    if (!e || fault > CF_SEAL_FAULT_ACTIVE_REPLACEMENT) return -1;
    e->fault = fault;
    return 0;
}

extern "C" int cf_device_seal_get_state(const cf_device_seal_engine *e, uint32_t layer, uint32_t *state) {
    if (!e || layer >= e->core.layers.size() || !state) return -1;
    *state = e->core.layers[layer].state;
    return 0;
}

extern "C" int cf_device_seal_get_counters(const cf_device_seal_engine *e, cf_device_seal_counters *out) {
    if (!e || !out) return -1;
    *out = e->counters;
    return 0;
}

extern "C" const char *cf_device_seal_last_error(const cf_device_seal_engine *e) { return e ? e->error.c_str() : "null seal engine"; }
