// ms_resolver.cu — the reference's device sequence resolver ABI (include/chromofold_b200/compat_ms.h) on this
// library's multi-sequence page store. Host semantics follow src/cuda/multisequence_cuda_resolver.cu (shared pages
// with logical / in-flight references, snapshots released on events, deferred reclamation, copy-on-write tails);
// the data path is new: pages are format-v1 records in one arena, every sequence has a row in a device page table,
// and a batch is one cf_b200_sealed_attention_async launch per layer instead of one kernel per item.

#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "chromofold_b200/compat_ms.h"
#include "cf_device_common.cuh"
#include "engine_common.cuh"

using namespace cfb_engine;

namespace {

constexpr uint32_t kMaxBatchTokens = 2048;

struct SharedPage;
// `page` is the entry of cf_ms_cuda_resolver::pages for page_id (entries of that map do not move; set when the reference
// is made), so that the per-batch bookkeeping over thousands of pages does not pay a hash look-up per page.
struct PageRef { uint64_t page_id; int64_t logical_begin; uint32_t tokens; uint32_t first_tile, tiles; SharedPage *page = nullptr; };
struct SharedPage {
    uint64_t logical_refs = 0, in_flight_refs = 0, resident_bytes = 0, seal_generation = 0;
    bool retired = false;
    uint64_t record_bytes = 0;        // what the sealer wrote into the page's arena slot
    std::vector<uint32_t> store_ids;  // page ids of its tiles in the arena's directory
};
struct LayerSeq {
    std::vector<PageRef> pages;
    uint32_t pins = 0;   // unreleased snapshots that still hold this list as "its first n pages" (see Snapshot)
    uint32_t sealed_tokens = 0, tiles = 0;
    bool partial_last = false;
    uint32_t active_begin = 0, active_count = 0;
    uint64_t active_generation = 0, descriptor_generation = 0;
};
struct Sequence {
    int64_t id = 0;
    uint32_t slot = 0;
    bool dispatchable = true;
    uint64_t topology_generation = 0;
    std::vector<LayerSeq> layers;
};
// What a batch item reads: the first page_count pages of a (sequence, layer) list at the time of the launch. Taking it
// costs nothing per page: the list is pinned (LayerSeq::pins) and only when the sequence is about to DROP pages while a
// snapshot is still out are the page ids written down and each page's in-flight count raised (materialise_pins), so
// a decode step over long sequences does not walk tens of thousands of page objects on the host. A page list only
// grows at its end between drops, which is what makes "the first n pages" a stable name.
struct Snapshot { int64_t sequence_id; uint32_t layer; uint32_t page_count; bool lazy; std::vector<uint64_t> page_ids; };
struct Pending { std::vector<Snapshot> snapshots; cudaEvent_t event = nullptr; };   // one event per batch

// Reference int4 page (all kv heads): value = (nibble - 8) * scale[flat / block_size], flat = (token*Hkv + head)*D + d,
// two nibbles per byte, low nibble first (src/cuda/device_kv_seal_attention.cu:106-118). Written as fp32 rows into
// a scratch tail [kv head][capacity][dim].
__global__ void unpack_reference_page_kernel(cf_device_page_descriptor page, float *tail_k, float *tail_v, uint32_t capacity) {
    const uint64_t count = static_cast<uint64_t>(page.token_count) * page.kv_head_count * page.head_dim;
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const uint32_t d = i % page.head_dim, h = (i / page.head_dim) % page.kv_head_count;
    const uint32_t t = i / (static_cast<uint64_t>(page.head_dim) * page.kv_head_count);
    const uint32_t shift = (i & 1) ? 4u : 0u;
    const float k = static_cast<float>(static_cast<int>((page.key_payload[i >> 1] >> shift) & 0xfu) - 8) * page.key_scales[i / page.block_size];
    const float v = static_cast<float>(static_cast<int>((page.value_payload[i >> 1] >> shift) & 0xfu) - 8) * page.value_scales[i / page.block_size];
    const uint64_t dst = (static_cast<uint64_t>(h) * capacity + t) * page.head_dim + d;
    tail_k[dst] = k;
    tail_v[dst] = v;
}

struct ItemIo {   // one batch item's query view and output placement, as the gather / scatter kernels see them
    cf_device_tensor_view query;
    void *output;
    uint32_t output_type, first_row;
    uint64_t ots, ohs, oes;
};

__global__ void gather_queries_kernel(const ItemIo *items, float *dense, uint32_t heads, uint32_t dim) {
    const ItemIo it = items[blockIdx.y];
    const uint64_t count = static_cast<uint64_t>(it.query.token_count) * heads * dim;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t d = i % dim, h = (i / dim) % heads;
        const uint32_t t = i / (static_cast<uint64_t>(dim) * heads);
        dense[static_cast<uint64_t>(it.first_row) * heads * dim + i] = load_scalar(
            it.query.data, t * it.query.token_stride_bytes + h * it.query.head_stride_bytes + d * it.query.element_stride_bytes,
            it.query.scalar_type);
    }
}
__global__ void scatter_outputs_kernel(const ItemIo *items, const float *dense, uint32_t heads, uint32_t dim) {
    const ItemIo it = items[blockIdx.y];
    const uint64_t count = static_cast<uint64_t>(it.query.token_count) * heads * dim;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t d = i % dim, h = (i / dim) % heads;
        const uint32_t t = i / (static_cast<uint64_t>(dim) * heads);
        store_scalar(it.output, t * it.ots + h * it.ohs + d * it.oes, it.output_type,
                     dense[static_cast<uint64_t>(it.first_row) * heads * dim + i]);
    }
}

}  // namespace

struct cf_ms_cuda_resolver {
    cf_ms_cuda_config config{};
    mutable std::mutex mutex;
    std::map<int64_t, Sequence> sequences;
    std::unordered_map<uint64_t, SharedPage> pages;
    std::vector<Pending> pending;
    std::vector<uint32_t> free_slots;
    uint64_t next_page_id = 1;
    uint32_t next_slot = 0;
    uint64_t ref_increments = 0, ref_decrements = 0;   // page references taken / dropped by sequences
    cf_ms_cuda_counters counters{};
    std::string error;
    // device side
    uint32_t tile = 0, tiles_per_page = 0, slot_capacity = 0, stride = 256;
    // Arena room is handed out in page slots: a slot holds the records of one page (tiles_per_page tiles x kv heads, each
    // at its largest possible size) at a fixed place, store ids slot * tiles_per_page + 1 + tile. A reclaimed page gives
    // its slot back, and the next page sealed into it overwrites the old bytes: the arena stops growing once the number
    // of live pages does, however many sequences come and go.
    uint32_t next_page_slot = 0;
    std::vector<uint32_t> free_page_slots;
    uint64_t live_record_bytes = 0;      // bytes the sealer actually wrote into live slots
    uint32_t device_status_seen = 0;     // CF_B200_DEVSTAT_* bits read back at the resolver's synchronisation points
    std::vector<bool> calibrated;
    bool ready = false;
    Buffer<uint8_t> arena, workspace;
    Buffer<uint64_t> page_dir;
    Buffer<uint32_t> page_table, sealed, tails, jobs, status, slot_list, positions;   // tables are [layer][slot]
    Buffer<float> tail_k, tail_v, scratch_k, scratch_v, q_dense, o_dense;          // tails are [layer][slot][Hkv][page][D]
    Buffer<cf_b200_codebook_tables> tables;
    Buffer<unsigned long long> cursor;
    Buffer<ItemIo> item_io;

    size_t page_values() const { return static_cast<size_t>(config.kv_head_count) * config.page_size * config.head_dim; }
    size_t max_record_bytes() const { return 16 + 2 * ((static_cast<size_t>(tile) * config.head_dim + 15) / 16 * 16); }
    size_t row(uint32_t layer, uint32_t slot) const { return static_cast<size_t>(layer) * slot_capacity + slot; }

    void ensure_ready(cudaStream_t s) {
        if (ready) return;
        tile = choose_tile_tokens(config.page_size, config.head_dim);
        tiles_per_page = config.page_size / tile;
        calibrated.assign(config.layer_count, false);
        tables.ensure(2 * config.layer_count, s);
        cursor.ensure(513, s);
        status.ensure(1, s);
        jobs.ensure(4 * 64, s);
        arena.ensure(16u << 20, s);
        page_dir.ensure(static_cast<size_t>(4096) * config.kv_head_count, s);
        scratch_k.ensure(page_values(), s);
        scratch_v.ensure(page_values(), s);
        slot_list.ensure(kMaxBatchTokens, s);
        positions.ensure(kMaxBatchTokens, s);
        item_io.ensure(1024, s);
        q_dense.ensure(static_cast<size_t>(kMaxBatchTokens) * config.query_head_count * config.head_dim, s);
        o_dense.ensure(q_dense.count, s);
        cf_b200_sealed_attention_desc d{};
        d.kv_head_count = config.kv_head_count;
        d.query_head_count = config.query_head_count;
        d.head_dim = config.head_dim;
        d.seq_count = kMaxBatchTokens;
        uint64_t bytes = 0;
        cf_b200_sealed_attention_workspace_bytes(&d, 65536, &bytes);
        workspace.ensure(bytes + 256, s);
        ready = true;
        grow_slots(std::max(16u, next_slot), s);
    }

    // Tables are laid out [layer][slot]; growing the slot count re-strides them.
    void grow_slots(uint32_t wanted, cudaStream_t s) {
        if (wanted <= slot_capacity) return;
        uint32_t next = std::max(16u, slot_capacity);
        while (next < wanted) next *= 2;
        const uint32_t L = config.layer_count, old = slot_capacity;
        auto restride = [&](auto &buf, size_t per_slot) {
            using T = std::remove_pointer_t<decltype(buf.ptr)>;
            Buffer<T> fresh;
            fresh.ensure(static_cast<size_t>(L) * next * per_slot, s);
            if (old)
                cuda_check(cudaMemcpy2DAsync(fresh.ptr, next * per_slot * sizeof(T), buf.ptr, old * per_slot * sizeof(T),
                                             old * per_slot * sizeof(T), L, cudaMemcpyDeviceToDevice, s), "re-stride table");
            cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
            std::swap(fresh.ptr, buf.ptr);
            std::swap(fresh.count, buf.count);
        };
        restride(page_table, stride);
        restride(sealed, 1);
        restride(tails, 1);
        restride(tail_k, page_values());
        restride(tail_v, page_values());
        slot_capacity = next;
    }

    void grow_stride(uint32_t wanted, cudaStream_t s) {
        if (wanted <= stride) return;
        uint32_t next = stride;
        while (next < wanted) next *= 2;
        Buffer<uint32_t> fresh;
        const size_t rows = static_cast<size_t>(config.layer_count) * slot_capacity;
        fresh.ensure(rows * next, s);
        cuda_check(cudaMemcpy2DAsync(fresh.ptr, next * 4, page_table.ptr, stride * 4, stride * 4, rows, cudaMemcpyDeviceToDevice, s),
                   "widen page table");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        std::swap(fresh.ptr, page_table.ptr);
        std::swap(fresh.count, page_table.count);
        stride = next;
        ++counters.descriptor_table_rebuilds;
    }

    uint32_t take_slot(cudaStream_t s) {
        if (!free_slots.empty()) { const uint32_t v = free_slots.back(); free_slots.pop_back(); return v; }
        const uint32_t slot = next_slot++;
        if (ready) grow_slots(next_slot, s);
        return slot;
    }

    void push_scalars(const Sequence &q, uint32_t layer, cudaStream_t s) {
        const LayerSeq &L = q.layers[layer];
        cuda_check(cudaMemcpyAsync(sealed.ptr + row(layer, q.slot), &L.sealed_tokens, 4, cudaMemcpyHostToDevice, s), "sealed count");
        cuda_check(cudaMemcpyAsync(tails.ptr + row(layer, q.slot), &L.active_count, 4, cudaMemcpyHostToDevice, s), "tail count");
    }

    void release_snapshot(const Snapshot &snap) {
        if (snap.lazy) {   // never written down: the list it pinned is still there (a drop would have materialised it)
            auto q = sequences.find(snap.sequence_id);
            if (q == sequences.end() || snap.layer >= q->second.layers.size() || q->second.layers[snap.layer].pins == 0)
                throw std::runtime_error("snapshot reference underflow");
            --q->second.layers[snap.layer].pins;
            counters.in_flight_page_references -= snap.page_count;
        } else {
            for (uint64_t id : snap.page_ids) {
                auto p = pages.find(id);
                if (p == pages.end() || p->second.in_flight_refs == 0) throw std::runtime_error("snapshot reference underflow");
                --p->second.in_flight_refs;
                --counters.in_flight_page_references;
            }
        }
        ++counters.snapshots_released;
    }

    // Before (sequence, layer) drops pages: every snapshot that still names its list lazily gets its page ids written
    // down and its pages' in-flight counts raised, so that reclamation waits for the launches that read them.
    // `building` = snapshots of a batch that is being assembled (not yet in `pending`).
    void materialise_pins(Sequence &q, uint32_t layer, std::vector<Snapshot> *building = nullptr) {
        LayerSeq &L = q.layers[layer];
        if (L.pins == 0) return;
        auto write_down = [&](Snapshot &snap) {
            if (!snap.lazy || snap.sequence_id != q.id || snap.layer != layer) return;
            snap.page_ids.reserve(snap.page_count);
            for (uint32_t i = 0; i < snap.page_count && i < L.pages.size(); ++i) {
                PageRef &ref = L.pages[i];
                SharedPage &page = ref.page ? *ref.page : pages.at(ref.page_id);
                ++page.in_flight_refs;
                snap.page_ids.push_back(ref.page_id);
            }
            counters.in_flight_page_references -= snap.page_count - snap.page_ids.size();
            snap.lazy = false;
            --L.pins;
        };
        for (Pending &p : pending)
            for (Snapshot &snap : p.snapshots) write_down(snap);
        if (building)
            for (Snapshot &snap : *building) write_down(snap);
    }
    void materialise_pins(Sequence &q) {
        for (uint32_t layer = 0; layer < q.layers.size(); ++layer) materialise_pins(q, layer);
    }
};

namespace {

template <class Fn>
int locked(cf_ms_cuda_resolver *r, bool count_cuda_error, Fn &&fn) {
    std::lock_guard<std::mutex> guard(r->mutex);
    try {
        fn();
        r->error.clear();
        return 0;
    } catch (const std::exception &e) {
        if (count_cuda_error) ++r->counters.cuda_errors;
        r->error = e.what();
        return -1;
    }
}

Sequence &find_sequence(cf_ms_cuda_resolver *r, int64_t id, const char *what) {
    auto it = r->sequences.find(id);
    if (it == r->sequences.end()) throw std::runtime_error(what);
    return it->second;
}

void retire_if_unreferenced(cf_ms_cuda_resolver *r, SharedPage &page) {
    if (page.logical_refs != 0 || page.retired) return;
    page.retired = true;
    ++r->counters.pages_retired;
    r->counters.pending_reclamation_bytes += page.resident_bytes;
    r->counters.pending_reclamation_bytes_peak = std::max(r->counters.pending_reclamation_bytes_peak, r->counters.pending_reclamation_bytes);
}

// Seal `token_count` fp32 rows laid out [kv head][page_size][dim] at src_k / src_v into format-v1 records (one launch),
// append their ids to the sequence's page-table row of `layer` and return the number of tiles. The first page of a
// layer also calibrates the layer's shared codebooks from its own codes.
uint32_t seal_rows(cf_ms_cuda_resolver *r, Sequence &q, uint32_t layer, const float *src_k, const float *src_v,
                   uint32_t token_count, SharedPage &page, cudaStream_t s) {
    LayerSeq &L = q.layers[layer];
    const uint32_t n = (token_count + r->tile - 1) / r->tile;
    r->grow_stride(L.tiles + n, s);
    if (n > r->tiles_per_page) throw std::invalid_argument("more rows than a page holds");
    const bool recycled = !r->free_page_slots.empty();
    const uint32_t page_slot = recycled ? r->free_page_slots.back() : r->next_page_slot;
    const uint64_t slot_units = static_cast<uint64_t>(r->tiles_per_page) * r->config.kv_head_count * (r->max_record_bytes() / 16u);
    const unsigned long long region_begin = 1ull + page_slot * slot_units;   // unit 0 stays unused
    r->arena.ensure((region_begin + slot_units) * 16u + 4096, s);
    std::vector<uint32_t> host(4 * n);
    for (uint32_t j = 0; j < n; ++j) {
        const uint32_t id = page_slot * r->tiles_per_page + 1u + j;
        page.store_ids.push_back(id);
        host[j] = 0;
        host[n + j] = id;
        host[2 * n + j] = std::min(r->tile, token_count - j * r->tile);
        host[3 * n + j] = j * r->tile;
    }
    r->page_dir.ensure((static_cast<size_t>(page_slot + 1) * r->tiles_per_page + 2) * r->config.kv_head_count, s);
    r->jobs.ensure(4 * n, s);
    cuda_check(cudaMemcpyAsync(r->jobs.ptr, host.data(), host.size() * 4, cudaMemcpyHostToDevice, s), "upload seal jobs");
    cf_b200_seal_desc sd{};
    sd.struct_size = sizeof sd;
    sd.abi_version = CF_B200_ABI_VERSION;
    sd.kv_head_count = r->config.kv_head_count;
    sd.head_dim = r->config.head_dim;
    sd.page_tokens = r->tile;
    sd.block_size = 64;
    sd.coder = engine_coder(r->tile * r->config.head_dim);
    sd.codebook_id = layer;
    sd.k_tables = r->tables.ptr + 2 * layer;
    sd.v_tables = r->tables.ptr + 2 * layer + 1;
    sd.tail_k = src_k;
    sd.tail_v = src_v;
    sd.tail_type = CF_B200_F32;
    sd.tail_capacity = r->config.page_size;
    sd.job_slots = r->jobs.ptr;
    sd.job_pages = r->jobs.ptr + n;
    sd.job_tokens = r->jobs.ptr + 2 * n;
    sd.job_rows = r->jobs.ptr + 3 * n;
    sd.job_count = n;
    sd.arena = r->arena.ptr;
    sd.arena_units = region_begin + slot_units;   // the sealer takes room from the cursor: it starts at the slot and may not leave it
    sd.arena_cursor_units = r->cursor.ptr;
    sd.page_dir = r->page_dir.ptr;
    sd.status = r->status.ptr;
    if (!r->calibrated[layer]) {
        cuda_check(cudaMemsetAsync(r->cursor.ptr + 1, 0, 512 * sizeof(unsigned long long), s), "clear histograms");
        if (cf_b200_histogram_async(&sd, r->cursor.ptr + 1, r->cursor.ptr + 257, s) != CF_OK) throw std::runtime_error("histogram launch rejected");
        unsigned long long hist[512];
        cuda_check(cudaMemcpyAsync(hist, r->cursor.ptr + 1, sizeof hist, cudaMemcpyDeviceToHost, s), "read histograms");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        std::vector<cf_b200_codebook_tables> tables(2);
        uint64_t hk[256], hv[256];
        for (int i = 0; i < 256; ++i) { hk[i] = hist[i]; hv[i] = hist[256 + i]; }
        if (cf_b200_codebook_build(hk, &tables[0]) != CF_OK || cf_b200_codebook_build(hv, &tables[1]) != CF_OK)
            throw std::runtime_error("codebook build failed");
        cuda_check(cudaMemcpyAsync(r->tables.ptr + 2 * layer, tables.data(), 2 * sizeof(cf_b200_codebook_tables),
                                   cudaMemcpyHostToDevice, s), "upload codebooks");
        cuda_check(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        r->calibrated[layer] = true;
    }
    cuda_check(cudaMemcpyAsync(r->cursor.ptr, &region_begin, sizeof region_begin, cudaMemcpyHostToDevice, s), "place arena cursor");
    if (cf_b200_seal_pages_async(&sd, s) != CF_OK) throw std::runtime_error("seal launch rejected");
    // The sealer publishes nothing for a tile that holds NaN / Inf or found no room, so its outcome is read back before
    // the page becomes part of the sequence (the reference synchronises at the same point,
    // src/cuda/device_kv_seal_attention.cu:265). A refused page leaves the sequence, the slot list and the counters as
    // they were.
    uint32_t status = 0;
    unsigned long long cursor_after = 0;
    cuda_check(cudaMemcpyAsync(&status, r->status.ptr, 4, cudaMemcpyDeviceToHost, s), "read seal status");
    cuda_check(cudaMemcpyAsync(&cursor_after, r->cursor.ptr, sizeof cursor_after, cudaMemcpyDeviceToHost, s), "read arena cursor");
    cuda_check(cudaStreamSynchronize(s), "seal validation sync");
    r->device_status_seen |= status;
    if (status & (CF_B200_DEVSTAT_NONFINITE | CF_B200_DEVSTAT_ARENA_FULL)) {
        for (uint32_t id : page.store_ids)   // whatever some kv heads of the page did publish goes back to "not there"
            cuda_check(cudaMemsetAsync(r->page_dir.ptr + static_cast<size_t>(id) * r->config.kv_head_count, 0,
                                       r->config.kv_head_count * sizeof(uint64_t), s), "unpublish refused page");
        cuda_check(cudaMemsetAsync(r->status.ptr, 0, 4, s), "clear status");
        page.store_ids.clear();
        throw std::runtime_error(status & CF_B200_DEVSTAT_NONFINITE ? "page contains NaN or Inf" : "arena slot is too small for the page");
    }
    if (recycled) r->free_page_slots.pop_back();
    else ++r->next_page_slot;
    page.record_bytes = (cursor_after - region_begin) * 16ull;
    r->live_record_bytes += page.record_bytes;
    cuda_check(cudaMemcpyAsync(r->page_table.ptr + r->row(layer, q.slot) * r->stride + L.tiles, host.data() + n, n * 4,
                               cudaMemcpyHostToDevice, s), "publish page ids");
    return n;
}

}  // namespace

extern "C" cf_ms_cuda_resolver *cf_ms_cuda_create(const cf_ms_cuda_config *c) {
    if (!c || !c->layer_count || !c->kv_head_count || !c->query_head_count || !c->head_dim || !c->page_size ||
        !c->gqa_group_size || c->query_head_count != c->kv_head_count * c->gqa_group_size || c->head_dim > CF_KV_MAX_HEAD_DIM ||
        c->gqa_group_size > 16)
        return nullptr;
    try {
        auto *r = new cf_ms_cuda_resolver();
        r->config = *c;
        return r;
    } catch (...) {
        return nullptr;
    }
}

extern "C" void cf_ms_cuda_destroy(cf_ms_cuda_resolver *r, void *stream) {
    if (!r) return;
    if (r->ready) cudaStreamSynchronize(static_cast<cudaStream_t>(stream));
    for (auto &p : r->pending)
        if (p.event) cudaEventDestroy(p.event);
    delete r;
}

extern "C" int cf_ms_cuda_sequence_create(cf_ms_cuda_resolver *r, int64_t id) {
    if (!r) return -1;
    return locked(r, false, [&] {
        if (r->sequences.count(id)) throw std::runtime_error("sequence already exists");
        Sequence q;
        q.id = id;
        q.slot = r->take_slot(nullptr);
        q.layers.resize(r->config.layer_count);
        r->sequences.emplace(id, std::move(q));
    });
}

extern "C" int cf_ms_cuda_publish_page_async(cf_ms_cuda_resolver *r, const cf_ms_page_publication *pub, void *stream) {
    if (!r || !pub) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    try {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        auto it = r->sequences.find(pub->sequence_id);
        if (it == r->sequences.end() || pub->layer >= it->second.layers.size()) throw std::runtime_error("publication target is invalid");
        const cf_device_page_descriptor &d = pub->descriptor;
        if (!d.key_payload || !d.value_payload || !d.key_scales || !d.value_scales) throw std::runtime_error("publication descriptor is incomplete");
        if (d.kv_head_count != r->config.kv_head_count || d.head_dim != r->config.head_dim || d.token_count == 0 ||
            d.token_count > r->config.page_size || d.block_size == 0)
            throw std::runtime_error("publication descriptor does not match the resolver topology");
        Sequence &q = it->second;
        LayerSeq &L = q.layers[pub->layer];
        if (L.partial_last) throw std::runtime_error("a short page can only be the last page of a layer");
        if (d.token_begin != L.sealed_tokens) throw std::runtime_error("published page must continue the sealed history of the layer");
        r->ensure_ready(s);
        // transcode: int4 page -> fp32 scratch rows -> format-v1 records
        const uint64_t count = static_cast<uint64_t>(d.token_count) * d.kv_head_count * d.head_dim;
        unpack_reference_page_kernel<<<static_cast<int>((count + 255) / 256), 256, 0, s>>>(d, r->scratch_k.ptr, r->scratch_v.ptr,
                                                                                         r->config.page_size);
        cuda_check(cudaGetLastError(), "page unpack launch");
        SharedPage page;
        const uint32_t n = seal_rows(r, q, pub->layer, r->scratch_k.ptr, r->scratch_v.ptr, d.token_count, page, s);
        page.seal_generation = pub->seal_generation;
        page.resident_bytes = pub->resident_bytes;
        page.logical_refs = 1;
        ++r->ref_increments;
        const uint64_t id = r->next_page_id++;
        L.pages.push_back({id, static_cast<int64_t>(d.token_begin), d.token_count, L.tiles, n});
        L.pages.back().page = &r->pages.emplace(id, std::move(page)).first->second;
        L.tiles += n;
        L.sealed_tokens += d.token_count;
        L.partial_last = d.token_count % r->tile != 0;
        if (L.active_count && L.active_begin < L.sealed_tokens) L.active_count = 0;  // the staged rows were this page
        ++L.descriptor_generation;
        r->push_scalars(q, pub->layer, s);
        ++q.topology_generation;
        ++r->counters.pages_registered;
        ++r->counters.descriptor_tables_built;
        r->error.clear();
        return 0;
    } catch (const std::exception &e) {
        ++r->counters.page_registration_failures;
        r->error = e.what();
        return -1;
    }
}

extern "C" int cf_ms_cuda_stage_active_async(cf_ms_cuda_resolver *r, int64_t id, uint32_t layer, uint32_t token_begin,
                                             const float *keys, const float *values, uint32_t token_count, void *stream) {
    if (!r || !keys || !values || !token_count || token_count > r->config.page_size) return -1;
    return locked(r, true, [&] {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        auto it = r->sequences.find(id);
        if (it == r->sequences.end() || layer >= it->second.layers.size()) throw std::runtime_error("active target is invalid");
        Sequence &q = it->second;
        LayerSeq &L = q.layers[layer];
        if (token_begin != L.sealed_tokens) throw std::runtime_error("active rows must continue the sealed history of the layer");
        r->ensure_ready(s);
        cf_device_tensor_view view{};
        view.scalar_type = CF_DEVICE_F32;
        view.token_count = token_count;
        view.head_count = r->config.kv_head_count;
        view.head_dim = r->config.head_dim;
        view.element_stride_bytes = 4;
        view.head_stride_bytes = 4ull * view.head_dim;
        view.token_stride_bytes = view.head_stride_bytes * view.head_count;
        const uint64_t count = static_cast<uint64_t>(token_count) * view.head_count * view.head_dim;
        const int blocks = static_cast<int>((count + 255) / 256);
        const size_t base = r->row(layer, q.slot) * r->page_values();
        view.data = keys;
        rows_to_tail_kernel<<<blocks, 256, 0, s>>>(view, r->tail_k.ptr + base, r->config.page_size, 0);
        view.data = values;
        rows_to_tail_kernel<<<blocks, 256, 0, s>>>(view, r->tail_v.ptr + base, r->config.page_size, 0);
        cuda_check(cudaGetLastError(), "stage sequence active rows");
        L.active_begin = token_begin;
        L.active_count = token_count;
        ++L.active_generation;
        r->push_scalars(q, layer, s);
    });
}

// ---- additive entry points: the append / seal / truncate seam of a data-bearing sequence cache ---------------------
// (what cf_sequence_append_async + the device seal engine + cf_ms_cuda_publish_page_async do together in the
// reference, without the int4 detour: rows are appended to the active tail and the tail is sealed in one launch)

extern "C" int cf_b200_ms_append_active_async(cf_ms_cuda_resolver *r, int64_t id, uint32_t layer, uint32_t token_begin,
                                              const cf_device_tensor_view *keys, const cf_device_tensor_view *values, void *stream) {
    if (!r || !keys || !values) return -1;
    if (cf_device_tensor_validate(keys) != 0 || cf_device_tensor_validate(values) != 0) return -1;
    return locked(r, true, [&] {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        auto it = r->sequences.find(id);
        if (it == r->sequences.end() || layer >= it->second.layers.size()) throw std::invalid_argument("append target is invalid");
        if (keys->token_count != values->token_count || keys->head_count != r->config.kv_head_count ||
            values->head_count != r->config.kv_head_count || keys->head_dim != r->config.head_dim ||
            values->head_dim != r->config.head_dim || keys->token_count == 0)
            throw std::invalid_argument("append tensor topology mismatch");
        Sequence &q = it->second;
        LayerSeq &L = q.layers[layer];
        if (L.partial_last) throw std::invalid_argument("a layer whose last page is short cannot grow");
        if (token_begin != L.sealed_tokens + L.active_count) throw std::invalid_argument("non-contiguous sequence append");
        if (L.active_count + keys->token_count > r->config.page_size)
            throw std::invalid_argument("append crosses sequence active-page boundary");
        r->ensure_ready(s);
        const uint64_t count = static_cast<uint64_t>(keys->token_count) * keys->head_count * keys->head_dim;
        const int blocks = static_cast<int>((count + 255) / 256);
        const size_t base = r->row(layer, q.slot) * r->page_values();
        rows_to_tail_kernel<<<blocks, 256, 0, s>>>(*keys, r->tail_k.ptr + base, r->config.page_size, L.active_count);
        rows_to_tail_kernel<<<blocks, 256, 0, s>>>(*values, r->tail_v.ptr + base, r->config.page_size, L.active_count);
        cuda_check(cudaGetLastError(), "append sequence rows");
        if (!L.active_count) L.active_begin = L.sealed_tokens;
        L.active_count += keys->token_count;
        ++L.active_generation;
        r->push_scalars(q, layer, s);
    });
}

extern "C" int cf_b200_ms_seal_active_async(cf_ms_cuda_resolver *r, int64_t id, uint32_t layer, void *stream) {
    if (!r) return -1;
    return locked(r, true, [&] {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        auto it = r->sequences.find(id);
        if (it == r->sequences.end() || layer >= it->second.layers.size()) throw std::invalid_argument("seal target is invalid");
        Sequence &q = it->second;
        LayerSeq &L = q.layers[layer];
        if (!L.active_count) throw std::invalid_argument("no active rows to seal");
        if (L.partial_last) throw std::invalid_argument("a short page can only be the last page of a layer");
        r->ensure_ready(s);
        const size_t base = r->row(layer, q.slot) * r->page_values();
        SharedPage page;
        const uint32_t n = seal_rows(r, q, layer, r->tail_k.ptr + base, r->tail_v.ptr + base, L.active_count, page, s);
        page.logical_refs = 1;
        ++r->ref_increments;
        page.resident_bytes = static_cast<uint64_t>(n) * r->config.kv_head_count * r->max_record_bytes();
        const uint64_t page_id = r->next_page_id++;
        L.pages.push_back({page_id, static_cast<int64_t>(L.sealed_tokens), L.active_count, L.tiles, n});
        L.pages.back().page = &r->pages.emplace(page_id, std::move(page)).first->second;
        L.tiles += n;
        L.sealed_tokens += L.active_count;
        L.partial_last = L.active_count % r->tile != 0;
        L.active_count = 0;
        L.active_begin = L.sealed_tokens;
        ++L.descriptor_generation;
        r->push_scalars(q, layer, s);
        ++q.topology_generation;
        ++r->counters.pages_registered;
        ++r->counters.descriptor_tables_built;
    });
}

// Keep the first `token_count` tokens of every layer of the sequence: later whole pages lose this sequence's
// reference, the active tail is shortened; a cut inside a sealed page is refused (pages are immutable,
// src/multisequence_cache.cpp:318-321).
extern "C" int cf_b200_ms_truncate_async(cf_ms_cuda_resolver *r, int64_t id, uint32_t token_count, void *stream) {
    if (!r) return -1;
    return locked(r, false, [&] {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        Sequence &q = find_sequence(r, id, "sequence is missing");
        for (const LayerSeq &L : q.layers) {   // validate every layer before changing any
            if (token_count >= L.sealed_tokens) continue;
            uint32_t end = 0;
            bool boundary = token_count == 0;
            for (const PageRef &ref : L.pages) {
                end += ref.tokens;
                if (end == token_count) boundary = true;
            }
            if (!boundary) throw std::invalid_argument("removal inside immutable page is not supported");
        }
        for (uint32_t layer = 0; layer < q.layers.size(); ++layer) {
            LayerSeq &L = q.layers[layer];
            if (token_count >= L.sealed_tokens + L.active_count) continue;
            if (token_count >= L.sealed_tokens) {
                L.active_count = token_count - L.sealed_tokens;
            } else {
                r->materialise_pins(q, layer);
                L.active_count = 0;
                while (!L.pages.empty() && L.sealed_tokens > token_count) {
                    const PageRef ref = L.pages.back();
                    L.pages.pop_back();
                    L.sealed_tokens -= ref.tokens;
                    L.tiles -= ref.tiles;
                    SharedPage &page = r->pages.at(ref.page_id);
                    --page.logical_refs;
                    ++r->ref_decrements;
                    retire_if_unreferenced(r, page);
                }
                L.partial_last = !L.pages.empty() && L.pages.back().tokens % (r->tile ? r->tile : 1u) != 0;
                L.active_begin = L.sealed_tokens;
                ++L.descriptor_generation;
            }
            ++L.active_generation;
            if (r->ready) r->push_scalars(q, layer, s);
        }
        ++q.topology_generation;
    });
}

// Forget the first `token_count` tokens of every layer (whole pages only, all of them sealed): the sequence drops its
// reference to those pages, the later pages move to the front of its page-table row, and device token 0 becomes what
// was token `token_count` — the caller keeps the logical position of that token (a copy of a range that does not start
// at token 0, src/multisequence_cache.cpp:257-258).
extern "C" int cf_b200_ms_drop_prefix_async(cf_ms_cuda_resolver *r, int64_t id, uint32_t token_count, void *stream) {
    if (!r) return -1;
    return locked(r, false, [&] {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        Sequence &q = find_sequence(r, id, "sequence is missing");
        if (token_count == 0) return;
        for (const LayerSeq &L : q.layers) {   // the whole cut is checked before anything changes
            uint32_t covered = 0;
            for (const PageRef &ref : L.pages) {
                if (covered >= token_count) break;
                covered += ref.tokens;
            }
            if (covered != token_count && !(L.pages.empty() && L.sealed_tokens == 0 && L.active_count == 0))
                throw std::invalid_argument("a prefix cut must fall on a page boundary of sealed pages");
        }
        for (uint32_t layer = 0; layer < q.layers.size(); ++layer) {
            LayerSeq &L = q.layers[layer];
            if (L.pages.empty()) continue;
            r->materialise_pins(q, layer);
            uint32_t dropped_tokens = 0, dropped_tiles = 0;
            size_t dropped_pages = 0;
            while (dropped_tokens < token_count) {
                const PageRef &ref = L.pages[dropped_pages++];
                dropped_tokens += ref.tokens;
                dropped_tiles += ref.tiles;
                SharedPage &page = r->pages.at(ref.page_id);
                --page.logical_refs;
                ++r->ref_decrements;
                retire_if_unreferenced(r, page);
            }
            L.pages.erase(L.pages.begin(), L.pages.begin() + static_cast<std::ptrdiff_t>(dropped_pages));
            std::vector<uint32_t> row;
            for (PageRef &ref : L.pages) {
                ref.logical_begin -= token_count;
                ref.first_tile -= dropped_tiles;
                const SharedPage &page = r->pages.at(ref.page_id);
                row.insert(row.end(), page.store_ids.begin(), page.store_ids.end());
            }
            L.sealed_tokens -= dropped_tokens;
            L.tiles -= dropped_tiles;
            L.active_begin = L.sealed_tokens;
            ++L.descriptor_generation;
            if (r->ready) {
                if (!row.empty())
                    cuda_check(cudaMemcpyAsync(r->page_table.ptr + r->row(layer, q.slot) * r->stride, row.data(), row.size() * 4,
                                               cudaMemcpyHostToDevice, s), "re-base page table row");
                r->push_scalars(q, layer, s);
            }
        }
        ++q.topology_generation;
    });
}

extern "C" int cf_b200_ms_page_sharing(const cf_ms_cuda_resolver *r, uint64_t *shared_pages, uint64_t *shared_references,
                                       uint64_t *reference_increments, uint64_t *reference_decrements) {
    if (!r || !shared_pages || !shared_references || !reference_increments || !reference_decrements) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    *shared_pages = *shared_references = 0;
    for (const auto &entry : r->pages)
        if (entry.second.logical_refs >= 2) {
            ++*shared_pages;
            *shared_references += entry.second.logical_refs;
        }
    *reference_increments = r->ref_increments;
    *reference_decrements = r->ref_decrements;
    return 0;
}

extern "C" int cf_b200_ms_sequence_tokens(const cf_ms_cuda_resolver *r, int64_t id, uint32_t layer, uint32_t *sealed_tokens,
                                          uint32_t *active_tokens) {
    if (!r || !sealed_tokens || !active_tokens) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    auto it = r->sequences.find(id);
    if (it == r->sequences.end() || layer >= it->second.layers.size()) return -1;
    *sealed_tokens = it->second.layers[layer].sealed_tokens;
    *active_tokens = it->second.layers[layer].active_count;
    return 0;
}

extern "C" int cf_ms_cuda_copy_sequence_async(cf_ms_cuda_resolver *r, int64_t source_id, int64_t destination_id, void *stream) {
    if (!r || source_id == destination_id) return -1;
    return locked(r, true, [&] {
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        Sequence &src = find_sequence(r, source_id, "source sequence is missing");
        Sequence candidate;
        candidate.id = destination_id;
        auto old = r->sequences.find(destination_id);
        if (old != r->sequences.end()) {  // the old destination is replaced: its pages lose one reference each
            old->second.dispatchable = false;
            r->materialise_pins(old->second);
            for (auto &layer : old->second.layers)
                for (const auto &ref : layer.pages) {
                    SharedPage &page = r->pages.at(ref.page_id);
                    --page.logical_refs;
                    ++r->ref_decrements;
                    retire_if_unreferenced(r, page);
                }
            candidate.slot = old->second.slot;
        } else {
            candidate.slot = r->take_slot(s);
        }
        const Sequence &source = r->sequences.at(source_id);  // take_slot may have re-strided, not re-hashed: still valid
        candidate.layers = source.layers;
        for (uint32_t layer = 0; layer < r->config.layer_count; ++layer) {
            LayerSeq &L = candidate.layers[layer];
            L.pins = 0;   // the snapshots out on the source pin the source's list, not the copy's
            for (const auto &ref : L.pages) {
                ++r->pages.at(ref.page_id).logical_refs;
                ++r->ref_increments;
            }
            if (r->ready) {
                if (L.tiles)
                    cuda_check(cudaMemcpyAsync(r->page_table.ptr + r->row(layer, candidate.slot) * r->stride,
                                               r->page_table.ptr + r->row(layer, source.slot) * r->stride, L.tiles * 4ull,
                                               cudaMemcpyDeviceToDevice, s), "copy page table row");
                if (L.active_count) {  // the unsealed rows are the only bytes that are copied
                    const size_t bytes = r->page_values() * sizeof(float);
                    cuda_check(cudaMemcpyAsync(r->tail_k.ptr + r->row(layer, candidate.slot) * r->page_values(),
                                               r->tail_k.ptr + r->row(layer, source.slot) * r->page_values(), bytes,
                                               cudaMemcpyDeviceToDevice, s), "copy active K");
                    cuda_check(cudaMemcpyAsync(r->tail_v.ptr + r->row(layer, candidate.slot) * r->page_values(),
                                               r->tail_v.ptr + r->row(layer, source.slot) * r->page_values(), bytes,
                                               cudaMemcpyDeviceToDevice, s), "copy active V");
                    ++L.active_generation;
                    ++r->counters.copy_on_write_tail_copies;
                }
                r->push_scalars(candidate, layer, s);
            }
            ++r->counters.descriptor_tables_built;
        }
        (void)src;
        r->sequences[destination_id] = std::move(candidate);
    });
}

// Sealed records that every row of a layer's batch shares: sequences forked from one prompt reference the same pages
// (copy shares pages by reference), and the query tokens of one prefill item all see the item's sealed history. Such
// records are decoded once per 128 query rows by the shared-prefix kernel instead of once per row; the number returned
// here is only a hint, the plan kernel checks it against the page tables. 0 = not worth it or not applicable.
static uint32_t shared_leading_tiles(cf_ms_cuda_resolver *r, const cf_ms_batch_item *items, uint32_t item_count, uint32_t layer,
                                     uint32_t rows, uint32_t window) {
    if (rows < 4 || window != 0) return 0;   // a handful of rows is served faster one by one
    const LayerSeq *first = nullptr;
    size_t common_refs = 0;
    uint32_t lowest_position = 0xffffffffu;
    for (uint32_t i = 0; i < item_count; ++i) {
        if (items[i].layer != layer) continue;
        lowest_position = std::min(lowest_position, items[i].query_token_begin);
        const LayerSeq &L = r->sequences.at(items[i].sequence_id).layers[layer];
        if (!first) {
            first = &L;
            common_refs = L.pages.size();
            continue;
        }
        if (&L == first) continue;
        size_t n = 0;
        while (n < common_refs && n < L.pages.size() && L.pages[n].page_id == first->pages[n].page_id) ++n;
        common_refs = n;
    }
    if (!first) return 0;
    uint32_t tiles = 0;
    for (size_t n = 0; n < common_refs; ++n) {
        const PageRef &ref = first->pages[n];
        if (ref.tokens != ref.tiles * r->tile) break;   // a record that is not full ends the run of whole records
        tiles += ref.tiles;
    }
    tiles = std::min(tiles, (lowest_position + 1u) / r->tile);   // every query token must see the shared records in full
    return tiles >= 8 ? tiles : 0;
}

extern "C" int cf_ms_cuda_execute_batch_async(cf_ms_cuda_resolver *r, const cf_ms_batch_item *items, uint32_t item_count,
                                              void *stream) {
    if (!r || !items || !item_count) return -1;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> guard(r->mutex);
    std::vector<Snapshot> snapshots;
    try {
        // validate everything and take every snapshot before the first launch (:381-390)
        uint32_t total_rows = 0;
        for (uint32_t i = 0; i < item_count; ++i) {
            const cf_ms_batch_item &it = items[i];
            if (cf_device_tensor_validate(&it.query) != 0 || !it.output || !scalar_bytes(it.output_type))
                throw std::runtime_error("invalid batch tensor");
            auto q = r->sequences.find(it.sequence_id);
            if (q == r->sequences.end() || !q->second.dispatchable) throw std::runtime_error("sequence is unavailable for dispatch");
            if (it.layer >= q->second.layers.size()) throw std::runtime_error("layer out of range");
            if (it.query.head_count != r->config.query_head_count || it.query.head_dim != r->config.head_dim)
                throw std::runtime_error("query topology mismatch");
            total_rows += it.query.token_count;
        }
        if (total_rows > kMaxBatchTokens || item_count > 1024) throw std::runtime_error("batch is larger than the resolver's staging buffers");
        snapshots.reserve(item_count);
        for (uint32_t i = 0; i < item_count; ++i) {
            LayerSeq &L = r->sequences.at(items[i].sequence_id).layers[items[i].layer];
            snapshots.push_back(Snapshot{items[i].sequence_id, items[i].layer, static_cast<uint32_t>(L.pages.size()), true, {}});
            ++L.pins;
            r->counters.in_flight_page_references += L.pages.size();
            ++r->counters.snapshots_acquired;
        }
        ++r->counters.server_batches_received;
        r->counters.tokens_per_batch_peak = std::max<uint64_t>(r->counters.tokens_per_batch_peak, item_count);
        r->ensure_ready(s);

        // rows of the batch, grouped by layer: [layer 0 items..., layer 1 items..., ...]
        std::vector<ItemIo> io(item_count);
        std::vector<uint32_t> slots, positions, order;
        std::vector<std::pair<uint32_t, uint32_t>> layer_rows(r->config.layer_count, {0u, 0u});  // first row, count
        for (uint32_t layer = 0; layer < r->config.layer_count; ++layer) {
            layer_rows[layer].first = static_cast<uint32_t>(slots.size());
            for (uint32_t i = 0; i < item_count; ++i) {
                const cf_ms_batch_item &it = items[i];
                if (it.layer != layer) continue;
                io[i] = ItemIo{it.query, it.output, it.output_type, static_cast<uint32_t>(slots.size()),
                               it.output_token_stride_bytes, it.output_head_stride_bytes, it.output_element_stride_bytes};
                const uint32_t slot = r->sequences.at(it.sequence_id).slot;
                for (uint32_t t = 0; t < it.query.token_count; ++t) {
                    slots.push_back(slot);
                    positions.push_back(it.query_token_begin + t);
                }
                if (it.query.token_count == 1) ++r->counters.decode_items; else ++r->counters.prefill_items;
            }
            layer_rows[layer].second = static_cast<uint32_t>(slots.size()) - layer_rows[layer].first;
        }
        cuda_check(cudaMemcpyAsync(r->item_io.ptr, io.data(), io.size() * sizeof(ItemIo), cudaMemcpyHostToDevice, s), "upload batch items");
        cuda_check(cudaMemcpyAsync(r->slot_list.ptr, slots.data(), slots.size() * 4, cudaMemcpyHostToDevice, s), "upload batch slots");
        cuda_check(cudaMemcpyAsync(r->positions.ptr, positions.data(), positions.size() * 4, cudaMemcpyHostToDevice, s), "upload batch positions");
        const uint32_t Hq = r->config.query_head_count, D = r->config.head_dim;
        gather_queries_kernel<<<dim3(8, item_count), 256, 0, s>>>(r->item_io.ptr, r->q_dense.ptr, Hq, D);
        cuda_check(cudaGetLastError(), "query gather launch");
        float softmax_scale = items[0].softmax_scale;
        uint32_t window = items[0].causal_window;
        for (uint32_t i = 1; i < item_count; ++i)
            if (items[i].softmax_scale != softmax_scale || items[i].causal_window != window)
                throw std::runtime_error("items of one batch must share softmax_scale and causal_window");
        for (uint32_t layer = 0; layer < r->config.layer_count; ++layer) {
            const auto [first, count] = layer_rows[layer];
            if (!count) continue;
            cf_b200_sealed_attention_desc d{};
            d.struct_size = sizeof d;
            d.abi_version = CF_B200_ABI_VERSION;
            d.kv_head_count = r->config.kv_head_count;
            d.query_head_count = Hq;
            d.head_dim = D;
            d.page_tokens = r->tile;
            d.block_size = 64;
            d.codebook_id = layer;
            d.arena = r->arena.ptr;
            d.page_dir = r->page_dir.ptr;
            d.page_table = r->page_table.ptr + r->row(layer, 0) * r->stride;
            d.seq_sealed_tokens = r->sealed.ptr + r->row(layer, 0);
            d.seq_slots = r->slot_list.ptr + first;
            d.page_table_stride = r->stride;
            d.seq_count = count;
            d.k_tables = r->tables.ptr + 2 * layer;
            d.v_tables = r->tables.ptr + 2 * layer + 1;
            d.tail_k = r->tail_k.ptr + r->row(layer, 0) * r->page_values();
            d.tail_v = r->tail_v.ptr + r->row(layer, 0) * r->page_values();
            d.tail_tokens = r->tails.ptr + r->row(layer, 0);
            d.tail_type = CF_B200_F32;
            d.tail_capacity = r->config.page_size;
            d.query_positions = r->positions.ptr + first;
            d.queries = r->q_dense.ptr + static_cast<size_t>(first) * Hq * D;
            d.output = r->o_dense.ptr + static_cast<size_t>(first) * Hq * D;
            d.query_type = CF_B200_F32;
            d.output_type = CF_B200_F32;
            d.softmax_scale = softmax_scale;
            d.causal_window = window;
            // the shared-prefix partials take their own region of the workspace, which grows for them if it has to
            d.shared_prefix_pages = shared_leading_tiles(r, items, item_count, layer, count, window);
            if (d.shared_prefix_pages && !shared_prefix_room(r->workspace, count, r->config.kv_head_count, Hq, D, s))
                d.shared_prefix_pages = 0;
            const uintptr_t ws = reinterpret_cast<uintptr_t>(r->workspace.ptr), aligned = (ws + 255) / 256 * 256;
            d.workspace = reinterpret_cast<void *>(aligned);
            d.workspace_bytes = r->workspace.count - (aligned - ws);
            d.status = r->status.ptr;
            if (cf_b200_sealed_attention_async(&d, s) != CF_OK) throw std::runtime_error("multi-sequence attention launch rejected");
            ++r->counters.sequence_attention_launches;
        }
        scatter_outputs_kernel<<<dim3(8, item_count), 256, 0, s>>>(r->item_io.ptr, r->o_dense.ptr, Hq, D);
        cuda_check(cudaGetLastError(), "output scatter launch");
        {   // one event for the batch: every snapshot of it is released when the batch's last kernel is done
            Pending p;
            cuda_check(cudaEventCreateWithFlags(&p.event, cudaEventDisableTiming), "create snapshot release event");
            const cudaError_t recorded = cudaEventRecord(p.event, s);
            if (recorded != cudaSuccess) {
                cudaEventDestroy(p.event);
                cuda_check(recorded, "record snapshot release event");
            }
            r->counters.snapshot_release_events += snapshots.size();
            p.snapshots = std::move(snapshots);
            snapshots.clear();
            r->pending.push_back(std::move(p));
        }
        ++r->counters.compressed_batches_executed;
        r->error.clear();
        return 0;
    } catch (const std::exception &e) {
        for (const auto &snap : snapshots) {
            try { r->release_snapshot(snap); } catch (...) {}
        }
        ++r->counters.cuda_errors;
        r->error = e.what();
        return -1;
    }
}

extern "C" int cf_ms_cuda_cancel_sequence_async(cf_ms_cuda_resolver *r, int64_t id, void *) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    auto q = r->sequences.find(id);
    if (q == r->sequences.end()) return -1;
    q->second.dispatchable = false;
    ++r->counters.cancellation_requests;
    return 0;
}

extern "C" int cf_ms_cuda_sequence_remove_async(cf_ms_cuda_resolver *r, int64_t id, void *) {
    if (!r) return -1;
    return locked(r, false, [&] {
        Sequence &q = find_sequence(r, id, "sequence is missing");
        r->materialise_pins(q);
        for (auto &layer : q.layers)
            for (const auto &ref : layer.pages) {
                SharedPage &page = r->pages.at(ref.page_id);
                if (!page.logical_refs) throw std::runtime_error("page logical reference underflow");
                --page.logical_refs;
                ++r->ref_decrements;
                retire_if_unreferenced(r, page);
            }
        r->free_slots.push_back(q.slot);
        r->sequences.erase(id);
    });
}

extern "C" int cf_ms_cuda_reclaim_async(cf_ms_cuda_resolver *r, void *stream) {
    if (!r) return -1;
    return locked(r, true, [&] {
        for (auto it = r->pending.begin(); it != r->pending.end();) {
            const cudaError_t status = cudaEventQuery(it->event);
            if (status == cudaErrorNotReady) { ++it; continue; }
            cuda_check(status, "query snapshot release event");
            for (const Snapshot &snap : it->snapshots) r->release_snapshot(snap);
            cudaEventDestroy(it->event);
            it = r->pending.erase(it);
        }
        for (auto it = r->pages.begin(); it != r->pages.end();) {
            SharedPage &page = it->second;
            if (page.retired && page.logical_refs == 0 && page.in_flight_refs == 0) {
                // the directory rows of its tiles go back to "not there"; its arena slot is handed to the next page sealed
                for (uint32_t id : page.store_ids)
                    if (r->ready)
                        cuda_check(cudaMemsetAsync(r->page_dir.ptr + static_cast<size_t>(id) * r->config.kv_head_count, 0,
                                                   r->config.kv_head_count * sizeof(uint64_t), static_cast<cudaStream_t>(stream)),
                                   "clear directory rows");
                if (!page.store_ids.empty()) r->free_page_slots.push_back((page.store_ids.front() - 1u) / r->tiles_per_page);
                r->live_record_bytes -= std::min<uint64_t>(r->live_record_bytes, page.record_bytes);
                r->counters.pending_reclamation_bytes -= page.resident_bytes;
                ++r->counters.pages_reclaimed;
                it = r->pages.erase(it);
            } else {
                ++it;
            }
        }
    });
}

extern "C" int cf_b200_ms_arena_stats(const cf_ms_cuda_resolver *r, uint64_t *slots_in_use, uint64_t *slots_free,
                                      uint64_t *live_record_bytes, uint64_t *arena_bytes, uint32_t *device_status_seen) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    if (slots_in_use) *slots_in_use = r->next_page_slot - r->free_page_slots.size();
    if (slots_free) *slots_free = r->free_page_slots.size();
    if (live_record_bytes) *live_record_bytes = r->live_record_bytes;
    if (arena_bytes) *arena_bytes = r->arena.count;
    if (device_status_seen) *device_status_seen = r->device_status_seen;
    return 0;
}

extern "C" int cf_ms_cuda_shift_sequence(cf_ms_cuda_resolver *r, int64_t id, uint32_t begin, uint32_t end, int32_t delta) {
    if (!r || end < begin) return -1;
    return locked(r, false, [&] {
        Sequence &q = find_sequence(r, id, "sequence is missing");
        for (auto &layer : q.layers)
            for (auto &ref : layer.pages) {
                const int64_t ref_end = ref.logical_begin + r->config.page_size;
                if (ref.logical_begin >= begin && ref_end <= end) {
                    if (delta != 0) throw std::runtime_error("sealed records carry no position: a non-zero shift needs a re-seal");
                } else if (ref.logical_begin < end && ref_end > begin) {
                    throw std::runtime_error("shift intersects part of an immutable page");
                }
            }
        ++q.topology_generation;
    });
}

extern "C" int cf_ms_cuda_audit(const cf_ms_cuda_resolver *r) {
    if (!r) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    std::unordered_map<uint64_t, uint64_t> observed;
    std::unordered_map<uint32_t, int> slots;
    for (const auto &[id, q] : r->sequences) {
        if (id != q.id || ++slots[q.slot] > 1) return -1;
        for (const auto &layer : q.layers) {
            uint32_t tokens = 0;
            for (const auto &ref : layer.pages) {
                auto page = r->pages.find(ref.page_id);
                if (page == r->pages.end() || page->second.retired) return -1;
                ++observed[ref.page_id];
                tokens += ref.tokens;
            }
            if (tokens != layer.sealed_tokens) return -1;
        }
    }
    for (const auto &[id, page] : r->pages)
        if (!page.retired && page.logical_refs != observed[id]) return -1;
    return r->counters.cross_sequence_contamination == 0 && r->counters.dense_fallback_launches == 0 ? 0 : -1;
}

extern "C" int cf_ms_cuda_get_counters(const cf_ms_cuda_resolver *r, cf_ms_cuda_counters *out) {
    if (!r || !out) return -1;
    std::lock_guard<std::mutex> guard(r->mutex);
    *out = r->counters;
    return 0;
}

extern "C" const char *cf_ms_cuda_last_error(const cf_ms_cuda_resolver *r) {
    return r ? r->error.c_str() : "null multi-sequence CUDA resolver";
}
