// sealed_multigpu.cu — the batch scheduler of include/chromofold_b200/sealed_kv_multigpu.h: one host process, one
// stream per GPU, sequences or kv heads sharded over the GPUs of a box, query rows out and output rows back as plain
// peer copies. No kernel here reads or writes another GPU's memory; the two row-permutation kernels run on the root
// GPU over the root GPU's own buffers.

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <numeric>
#include <string>
#include <thread>
#include <vector>

#include "attention_params.cuh"
#include "chromofold_b200/sealed_kv_multigpu.h"

namespace {

// dst row j = src row perm[j] (kGather) or dst row perm[j] = src row j (scatter); rows are whole 16-byte units.
template <bool kGather>
__global__ void permute_rows_kernel(const uint4 *src, uint4 *dst, const uint32_t *perm, uint32_t rows, uint32_t units_per_row) {
    for (uint64_t i = blockIdx.x * static_cast<uint64_t>(blockDim.x) + threadIdx.x; i < static_cast<uint64_t>(rows) * units_per_row;
         i += static_cast<uint64_t>(gridDim.x) * blockDim.x) {
        const uint32_t j = static_cast<uint32_t>(i / units_per_row), u = static_cast<uint32_t>(i % units_per_row);
        const uint64_t other = static_cast<uint64_t>(perm[j]) * units_per_row + u;
        if (kGather) dst[i] = src[other];
        else dst[other] = src[i];
    }
}

struct DeviceGuard {   // the calling thread's current device is put back when the call returns
    int saved = -1;
    DeviceGuard() { cudaGetDevice(&saved); }
    ~DeviceGuard() {
        if (saved >= 0) cudaSetDevice(saved);
    }
};

}  // namespace

// What every device does in a step; filled by the calling thread, read by the submitting threads.
struct StepJob {
    const cf_b200_mg_shard *shards = nullptr;
    uint32_t mode = 0, row_count = 0;
    const void *root_queries = nullptr;
    void *root_output = nullptr;
    uint32_t first_row[CF_B200_MG_MAX_DEVICES] = {};   // by-sequence: where the device's rows start in device-major order
    bool direct = false;   // this step's outputs are stored straight into root_output by every device
};

struct cf_b200_mg_scheduler {
    cf_b200_mg_config config{};
    // One submitting thread per device beyond the root: queueing a device's copies and launches takes tens of
    // microseconds of host time, which in one thread would add up to more than a step takes on eight GPUs. A thread
    // spins briefly for the next step, then sleeps.
    std::vector<std::thread> workers;
    std::atomic<uint64_t> step_seq{0};
    std::atomic<uint32_t> pending{0};
    std::atomic<bool> stopping{false};
    std::mutex wake_mutex;
    std::condition_variable wake_cv;
    StepJob job;
    cf_status device_status[CF_B200_MG_MAX_DEVICES] = {};
    std::string device_error[CF_B200_MG_MAX_DEVICES];
    std::vector<int32_t> ordinals;
    std::vector<cudaStream_t> streams;
    std::vector<cudaEvent_t> done;
    std::vector<uint8_t> failed;
    cudaEvent_t ready = nullptr;
    uint8_t *staging_q = nullptr;      // root device, max_rows query rows in device-major order
    float *staging_out = nullptr;      // root device, max_rows output rows in device-major order
    uint32_t *d_perm = nullptr;        // root device
    uint32_t *h_perm = nullptr;        // pinned
    std::vector<uint32_t> last_perm;   // what d_perm holds
    // Direct output (every device can store into the root's memory): a device keeps the whole batch's query rows
    // (one peer copy per step) and the rows of its own entries as a row map; its combine kernel stores the output rows
    // straight into the root's tensor. No staging, no permute kernels, no copies back.
    bool direct = false;
    std::vector<uint8_t *> q_full;             // per device: max_rows query rows (nullptr on the root)
    std::vector<uint32_t *> d_rows, h_rows;    // per device: row map on the device / pinned copy of what it holds
    std::vector<uint32_t> rows_held;           // per device: entries of the row map that are valid (0 = none uploaded)
    void *access_query = nullptr;              // cuPointerGetAttribute, looked up once
    bool access_query_looked_up = false;

    // Whether every other device may STORE to `ptr` (memory of the root): asked of the driver per device
    // (CU_POINTER_ATTRIBUTE_ACCESS_FLAGS with that device current). Anything but a clear "read and write" — an
    // allocation from a pool that was not opened to the peers, a driver that does not answer — keeps the copy path.
    // Asked on every call (a few microseconds of host time): an address can come back from the allocator as a
    // different kind of memory.
    bool every_device_may_store(const void *ptr) {
        using QueryFn = CUresult (*)(void *, CUpointer_attribute, CUdeviceptr);
        if (!access_query_looked_up) {
            cudaDriverEntryPointQueryResult found;
            void *entry = nullptr;
            if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &entry, cudaEnableDefault, &found) == cudaSuccess &&
                found == cudaDriverEntryPointSuccess)
                access_query = entry;
            access_query_looked_up = true;
        }
        void *entry = access_query;
        bool writable = entry != nullptr;
        for (size_t d = 1; d < ordinals.size() && writable; ++d) {
            unsigned long long flags = 0;
            writable = cudaSetDevice(ordinals[d]) == cudaSuccess &&
                       reinterpret_cast<QueryFn>(entry)(&flags, CU_POINTER_ATTRIBUTE_ACCESS_FLAGS,
                                                        reinterpret_cast<CUdeviceptr>(ptr)) == CUDA_SUCCESS &&
                       flags == CU_POINTER_ATTRIBUTE_ACCESS_FLAG_READWRITE;
        }
        cudaGetLastError();
        return writable;
    }
    cf_b200_mg_counters counters{};
    mutable std::mutex mutex;
    std::string error;

    size_t query_row_bytes() const {
        return static_cast<size_t>(config.query_head_count) * config.head_dim * (config.query_type == CF_B200_F32 ? 4u : 2u);
    }
    size_t output_row_bytes() const { return static_cast<size_t>(config.query_head_count) * config.head_dim * 4u; }
    cf_status fail(cf_status code, const std::string &why) {
        error = why;
        return code;
    }
    cf_status cuda_fail(cudaError_t e, const char *where) {
        error = std::string(where) + ": " + cudaGetErrorString(e);
        return CF_ERR_CUDA;
    }
    void stop_workers() {
        stopping.store(true, std::memory_order_release);
        {
            std::lock_guard<std::mutex> lock(wake_mutex);
        }
        wake_cv.notify_all();
        for (std::thread &t : workers)
            if (t.joinable()) t.join();
        workers.clear();
    }
    void release() {
        stop_workers();
        DeviceGuard guard;
        for (size_t d = 0; d < ordinals.size(); ++d) {
            if (cudaSetDevice(ordinals[d]) != cudaSuccess) continue;
            if (d < streams.size() && streams[d]) cudaStreamDestroy(streams[d]);
            if (d < done.size() && done[d]) cudaEventDestroy(done[d]);
        }
        for (size_t d = 0; d < ordinals.size(); ++d) {
            if (cudaSetDevice(ordinals[d]) != cudaSuccess) continue;
            if (d < q_full.size() && q_full[d]) cudaFree(q_full[d]);
            if (d < d_rows.size() && d_rows[d]) cudaFree(d_rows[d]);
            if (d < h_rows.size() && h_rows[d]) cudaFreeHost(h_rows[d]);
        }
        if (!ordinals.empty() && cudaSetDevice(ordinals[0]) == cudaSuccess) {
            if (ready) cudaEventDestroy(ready);
            if (staging_q) cudaFree(staging_q);
            if (staging_out) cudaFree(staging_out);
            if (d_perm) cudaFree(d_perm);
        }
        if (h_perm) cudaFreeHost(h_perm);
    }
};

namespace {

// Queues one device's share of the current step on that device's stream: wait for the root, query rows in, the
// attention launches, output rows (or columns) back to the root, done-event. The calling thread has the device current.
cf_status submit_device(cf_b200_mg_scheduler *s, uint32_t d) {
    const StepJob &job = s->job;
    const cf_b200_sealed_attention_desc &desc = job.shards[d].desc;
    const size_t q_row = s->query_row_bytes(), o_row = s->output_row_bytes();
    cudaStream_t stream = s->streams[d];
    std::string &error = s->device_error[d];
    auto cuda_fail = [&](cudaError_t e, const char *where) {
        error = std::string(where) + ": " + cudaGetErrorString(e);
        return CF_ERR_CUDA;
    };
    cudaError_t e;
    if ((e = cudaStreamWaitEvent(stream, s->ready, 0)) != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
    if (job.direct) {
        cf_b200_sealed_attention_desc local = desc;
        if (d != 0) {   // the batch's query rows, whole: reads stay local to this device
            uint8_t *q = job.mode == CF_B200_MG_BY_SEQUENCE ? s->q_full[d] : static_cast<uint8_t *>(const_cast<void *>(desc.queries));
            e = cudaMemcpyPeerAsync(q, s->ordinals[d], job.root_queries, s->ordinals[0], q_row * job.row_count, stream);
            if (e != cudaSuccess) return cuda_fail(e, "query rows out");
            local.queries = q;
        } else {
            local.queries = job.root_queries;
        }
        local.output = job.root_output;   // rows (or head columns) are stored where the caller wants them
        if (job.mode == CF_B200_MG_BY_SEQUENCE && job.shards[d].rows) {
            const uint32_t *rows = job.shards[d].rows;
            bool changed = s->rows_held[d] != desc.seq_count;
            for (uint32_t i = 0; !changed && i < desc.seq_count; ++i) changed = s->h_rows[d][i] != rows[i];
            if (changed) {   // a new placement: a few hundred bytes, and the pinned copy must not change under a copy in flight
                if ((e = cudaStreamSynchronize(stream)) != cudaSuccess) return cuda_fail(e, "row map upload");
                std::memcpy(s->h_rows[d], rows, sizeof(uint32_t) * desc.seq_count);
                e = cudaMemcpyAsync(s->d_rows[d], s->h_rows[d], sizeof(uint32_t) * desc.seq_count, cudaMemcpyHostToDevice, stream);
                if (e != cudaSuccess) return cuda_fail(e, "row map upload");
                s->rows_held[d] = desc.seq_count;
            }
            local.row_map = s->d_rows[d];
        }
        const cf_status launched = cfb::sealed_attention_stages(&local, CF_B200_STAGE_PLAN | CF_B200_STAGE_ATTENTION | CF_B200_STAGE_COMBINE, stream, d != 0);
        if (launched != CF_OK) {
            error = "attention launch failed on a device";
            return launched;
        }
        if ((e = cudaEventRecord(s->done[d], stream)) != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
        return CF_OK;
    }
    if (job.mode == CF_B200_MG_BY_SEQUENCE) {
        const uint32_t at = job.first_row[d];
        e = cudaMemcpyPeerAsync(const_cast<void *>(desc.queries), s->ordinals[d], s->staging_q + q_row * at, s->ordinals[0],
                                q_row * desc.seq_count, stream);
        if (e != cudaSuccess) return cuda_fail(e, "query rows out");
        const cf_status launched = cf_b200_sealed_attention_async(&desc, stream);
        if (launched != CF_OK) {
            error = "attention launch failed on a device";
            return launched;
        }
        e = cudaMemcpyPeerAsync(s->staging_out + (o_row / 4u) * at, s->ordinals[0], desc.output, s->ordinals[d],
                                o_row * desc.seq_count, stream);
        if (e != cudaSuccess) return cuda_fail(e, "output rows back");
    } else {
        const uint32_t group = desc.query_head_count / desc.kv_head_count;
        const uint32_t span = desc.kv_head_span ? desc.kv_head_span : desc.kv_head_count - desc.kv_head_begin;
        if (desc.queries != job.root_queries) {   // the root device may read the caller's rows in place
            e = cudaMemcpyPeerAsync(const_cast<void *>(desc.queries), s->ordinals[d], job.root_queries, s->ordinals[0],
                                    q_row * job.row_count, stream);
            if (e != cudaSuccess) return cuda_fail(e, "query rows out");
        }
        const cf_status launched = cf_b200_sealed_attention_async(&desc, stream);
        if (launched != CF_OK) {
            error = "attention launch failed on a device";
            return launched;
        }
        if (desc.output != job.root_output) {   // (the root may write in place)
            // columns [kv_head_begin * group, (kv_head_begin + span) * group) of every row: one pitched peer copy
            cudaMemcpy3DPeerParms parms{};
            const size_t column = static_cast<size_t>(desc.kv_head_begin) * group * desc.head_dim * 4u;
            const size_t width = static_cast<size_t>(span) * group * desc.head_dim * 4u;
            parms.srcDevice = s->ordinals[d];
            parms.dstDevice = s->ordinals[0];
            parms.srcPtr = make_cudaPitchedPtr(desc.output, o_row, o_row, job.row_count);
            parms.dstPtr = make_cudaPitchedPtr(job.root_output, o_row, o_row, job.row_count);
            parms.srcPos = make_cudaPos(column, 0, 0);
            parms.dstPos = make_cudaPos(column, 0, 0);
            parms.extent = make_cudaExtent(width, job.row_count, 1);
            if ((e = cudaMemcpy3DPeerAsync(&parms, stream)) != cudaSuccess) return cuda_fail(e, "output columns back");
        }
    }
    if ((e = cudaEventRecord(s->done[d], stream)) != cudaSuccess) return cuda_fail(e, "cudaEventRecord");
    return CF_OK;
}

void worker_main(cf_b200_mg_scheduler *s, uint32_t d) {
    const bool usable = cudaSetDevice(s->ordinals[d]) == cudaSuccess;
    uint64_t seen = 0;
    for (;;) {
        uint32_t spins = 0;
        while (s->step_seq.load(std::memory_order_acquire) == seen && !s->stopping.load(std::memory_order_acquire)) {
            if (++spins < 20000u) {
                std::this_thread::yield();
            } else {
                std::unique_lock<std::mutex> lock(s->wake_mutex);
                s->wake_cv.wait_for(lock, std::chrono::milliseconds(2), [&] {
                    return s->step_seq.load(std::memory_order_acquire) != seen || s->stopping.load(std::memory_order_acquire);
                });
            }
        }
        if (s->stopping.load(std::memory_order_acquire)) return;
        seen = s->step_seq.load(std::memory_order_acquire);
        if (s->job.shards[d].desc.seq_count != 0) {
            if (usable) {
                s->device_status[d] = submit_device(s, d);
            } else {
                s->device_status[d] = CF_ERR_CUDA;
                s->device_error[d] = "the device could not be made current";
            }
        }
        s->pending.fetch_sub(1u, std::memory_order_release);
    }
}

}  // namespace

extern "C" cf_b200_mg_scheduler *cf_b200_mg_create(const cf_b200_mg_config *c) {
    if (!c || c->struct_size != sizeof(cf_b200_mg_config) || c->abi_version != CF_B200_ABI_VERSION || c->device_count == 0 ||
        c->device_count > CF_B200_MG_MAX_DEVICES || !c->device_ordinals || c->max_rows == 0 || c->query_head_count == 0 ||
        c->head_dim == 0 || (c->query_type != CF_B200_F16 && c->query_type != CF_B200_F32) ||
        (static_cast<uint64_t>(c->query_head_count) * c->head_dim * 2u) % 16u != 0)
        return nullptr;
    for (uint32_t i = 0; i < c->device_count; ++i)
        for (uint32_t j = 0; j < i; ++j)
            if (c->device_ordinals[i] == c->device_ordinals[j] || c->device_ordinals[i] < 0) return nullptr;
    auto s = std::make_unique<cf_b200_mg_scheduler>();
    s->config = *c;
    s->ordinals.assign(c->device_ordinals, c->device_ordinals + c->device_count);
    s->config.device_ordinals = nullptr;
    s->streams.assign(c->device_count, nullptr);
    s->done.assign(c->device_count, nullptr);
    s->failed.assign(c->device_count, 0);
    DeviceGuard guard;
    bool ok = true, every_device_maps_the_root = true;
    for (uint32_t d = 0; d < c->device_count && ok; ++d) {
        ok = cudaSetDevice(s->ordinals[d]) == cudaSuccess &&
             cudaStreamCreateWithFlags(&s->streams[d], cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreateWithFlags(&s->done[d], cudaEventDisableTiming) == cudaSuccess;
        if (ok && d > 0) {   // a direct path between the root and this device, both ways, where the box has one
            int can = 0;
            bool mapped = false;
            if (cudaDeviceCanAccessPeer(&can, s->ordinals[d], s->ordinals[0]) == cudaSuccess && can) {
                const cudaError_t e = cudaDeviceEnablePeerAccess(s->ordinals[0], 0);
                if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) ok = false;
                mapped = ok;
                cudaGetLastError();
            }
            if (!mapped) every_device_maps_the_root = false;
        }
    }
    // direct output needs every device to have the root's memory mapped; CHROMOFOLD_B200_MG_COPIES=1 keeps the copy path
    const char *copies = std::getenv("CHROMOFOLD_B200_MG_COPIES");
    s->direct = ok && every_device_maps_the_root && !(copies && copies[0] == '1');
    s->q_full.assign(c->device_count, nullptr);
    s->d_rows.assign(c->device_count, nullptr);
    s->h_rows.assign(c->device_count, nullptr);
    s->rows_held.assign(c->device_count, 0u);
    for (uint32_t d = 0; d < c->device_count && ok && s->direct; ++d) {
        ok = cudaSetDevice(s->ordinals[d]) == cudaSuccess &&
             (d == 0 || cudaMalloc(&s->q_full[d], s->query_row_bytes() * c->max_rows) == cudaSuccess) &&
             cudaMalloc(&s->d_rows[d], sizeof(uint32_t) * c->max_rows) == cudaSuccess &&
             cudaMallocHost(&s->h_rows[d], sizeof(uint32_t) * c->max_rows) == cudaSuccess;
    }
    if (ok) ok = cudaSetDevice(s->ordinals[0]) == cudaSuccess;
    for (uint32_t d = 1; d < c->device_count && ok; ++d) {
        int can = 0;
        if (cudaDeviceCanAccessPeer(&can, s->ordinals[0], s->ordinals[d]) == cudaSuccess && can) {
            const cudaError_t e = cudaDeviceEnablePeerAccess(s->ordinals[d], 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) ok = false;
            cudaGetLastError();
        }
    }
    ok = ok && cudaEventCreateWithFlags(&s->ready, cudaEventDisableTiming) == cudaSuccess &&
         cudaMalloc(&s->staging_q, s->query_row_bytes() * c->max_rows) == cudaSuccess &&
         cudaMalloc(&s->staging_out, s->output_row_bytes() * c->max_rows) == cudaSuccess &&
         cudaMalloc(&s->d_perm, sizeof(uint32_t) * c->max_rows) == cudaSuccess &&
         cudaMallocHost(&s->h_perm, sizeof(uint32_t) * c->max_rows) == cudaSuccess;
    if (!ok) {
        s->release();
        return nullptr;
    }
    try {
        for (uint32_t d = 1; d < c->device_count; ++d) s->workers.emplace_back(worker_main, s.get(), d);
    } catch (...) {
        s->release();
        return nullptr;
    }
    return s.release();
}

extern "C" void cf_b200_mg_destroy(cf_b200_mg_scheduler *s) {
    if (!s) return;
    {
        DeviceGuard guard;
        for (size_t d = 0; d < s->ordinals.size(); ++d)
            if (cudaSetDevice(s->ordinals[d]) == cudaSuccess) cudaStreamSynchronize(s->streams[d]);
    }
    s->release();
    delete s;
}

extern "C" const char *cf_b200_mg_last_error(const cf_b200_mg_scheduler *s) { return s ? s->error.c_str() : "scheduler is null"; }

extern "C" cf_status cf_b200_mg_set_device_failed(cf_b200_mg_scheduler *s, int32_t ordinal, uint32_t failed) {
    if (!s) return CF_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(s->mutex);
    for (size_t d = 0; d < s->ordinals.size(); ++d)
        if (s->ordinals[d] == ordinal) {
            s->failed[d] = failed ? 1 : 0;
            return CF_OK;
        }
    return s->fail(CF_ERR_INVALID_ARGUMENT, "unknown device ordinal");
}

namespace {
// Indices of the devices that may take work.
std::vector<uint32_t> usable_devices(const cf_b200_mg_scheduler *s, uint32_t device_count) {
    std::vector<uint32_t> out;
    for (uint32_t d = 0; d < device_count; ++d)
        if (!s || d >= s->failed.size() || !s->failed[d]) out.push_back(d);
    return out;
}
}  // namespace

extern "C" cf_status cf_b200_mg_plan_sequences(const cf_b200_mg_scheduler *s, const uint64_t *lengths, uint32_t n, uint32_t device_count,
                                               uint32_t *out_device) {
    if ((!lengths && n) || (!out_device && n) || device_count == 0 || device_count > CF_B200_MG_MAX_DEVICES ||
        (s && device_count != s->ordinals.size()))
        return CF_ERR_INVALID_ARGUMENT;
    std::vector<uint32_t> devices;
    if (s) {
        std::lock_guard<std::mutex> lock(s->mutex);
        devices = usable_devices(s, device_count);
    } else {
        devices = usable_devices(nullptr, device_count);
    }
    if (devices.empty()) return CF_ERR_UNSUPPORTED;
    // longest processing time first: sequences by falling length (ties: lower index), each to the least loaded device
    // (ties: lower device index)
    std::vector<uint32_t> order(n);
    std::iota(order.begin(), order.end(), 0u);
    std::stable_sort(order.begin(), order.end(), [&](uint32_t a, uint32_t b) { return lengths[a] > lengths[b]; });
    std::vector<uint64_t> load(devices.size(), 0);
    for (uint32_t i : order) {
        size_t best = 0;
        for (size_t d = 1; d < devices.size(); ++d)
            if (load[d] < load[best]) best = d;
        out_device[i] = devices[best];
        load[best] += lengths[i];
    }
    return CF_OK;
}

extern "C" cf_status cf_b200_mg_plan_kv_heads(const cf_b200_mg_scheduler *s, uint32_t kv_heads, uint32_t device_count, uint32_t *out_begin,
                                              uint32_t *out_span) {
    if (kv_heads == 0 || device_count == 0 || device_count > CF_B200_MG_MAX_DEVICES || !out_begin || !out_span ||
        (s && device_count != s->ordinals.size()))
        return CF_ERR_INVALID_ARGUMENT;
    std::vector<uint32_t> devices;
    if (s) {
        std::lock_guard<std::mutex> lock(s->mutex);
        devices = usable_devices(s, device_count);
    } else {
        devices = usable_devices(nullptr, device_count);
    }
    if (devices.empty()) return CF_ERR_UNSUPPORTED;
    for (uint32_t d = 0; d < device_count; ++d) out_begin[d] = out_span[d] = 0;
    const uint32_t active = std::min<uint32_t>(static_cast<uint32_t>(devices.size()), kv_heads);
    const uint32_t base = kv_heads / active, extra = kv_heads % active;
    uint32_t begin = 0;
    for (uint32_t i = 0; i < active; ++i) {   // contiguous blocks, the first `extra` devices take one head more
        const uint32_t span = base + (i < extra ? 1u : 0u);
        out_begin[devices[i]] = begin;
        out_span[devices[i]] = span;
        begin += span;
    }
    return CF_OK;
}

extern "C" cf_status cf_b200_mg_execute_async(cf_b200_mg_scheduler *s, const cf_b200_mg_shard *shards, uint32_t shard_count,
                                              const void *root_queries, void *root_output, uint32_t row_count, uint32_t mode,
                                              void *root_stream_ptr) {
    if (!s) return CF_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(s->mutex);
    const uint32_t devices = static_cast<uint32_t>(s->ordinals.size());
    if (!shards || shard_count != devices || !root_queries || !root_output || row_count == 0 || row_count > s->config.max_rows ||
        (mode != CF_B200_MG_BY_SEQUENCE && mode != CF_B200_MG_BY_KV_HEAD))
        return s->fail(CF_ERR_INVALID_ARGUMENT, "bad arguments");
    uint32_t listed = 0;
    for (uint32_t d = 0; d < devices; ++d) {
        const cf_b200_sealed_attention_desc &desc = shards[d].desc;
        if (desc.seq_count == 0) continue;
        if (s->failed[d]) {
            ++s->counters.refused_batches;
            return s->fail(CF_ERR_UNSUPPORTED, "a shard names a device that is marked failed");
        }
        if (desc.query_head_count != s->config.query_head_count || desc.head_dim != s->config.head_dim ||
            desc.query_type != s->config.query_type || desc.output_type != CF_B200_F32 || !desc.queries || !desc.output ||
            desc.seq_count > s->config.max_rows)
            return s->fail(CF_ERR_INVALID_ARGUMENT, "a shard does not match the scheduler's row shape");
        for (uint32_t i = 0; shards[d].rows && i < desc.seq_count; ++i)
            if (shards[d].rows[i] >= row_count) return s->fail(CF_ERR_INVALID_ARGUMENT, "a shard lists a row outside the batch");
        if (!shards[d].rows && desc.seq_count > row_count) return s->fail(CF_ERR_INVALID_ARGUMENT, "a shard has more entries than rows");
        const cf_status valid = cf_b200_sealed_attention_validate(&desc);
        if (valid != CF_OK) return s->fail(valid, "a shard's descriptor is not valid");
        listed += desc.seq_count;
    }
    if (listed == 0) return s->fail(CF_ERR_INVALID_ARGUMENT, "no device has work");
    if (mode == CF_B200_MG_BY_SEQUENCE && listed > s->config.max_rows) return s->fail(CF_ERR_INVALID_ARGUMENT, "more entries than max_rows");

    DeviceGuard guard;
    cudaStream_t root_stream = static_cast<cudaStream_t>(root_stream_ptr);
    const size_t q_row = s->query_row_bytes(), o_row = s->output_row_bytes();
    const bool direct = s->direct && s->every_device_may_store(root_output);
    cudaError_t e = cudaSetDevice(s->ordinals[0]);
    if (e != cudaSuccess) return s->cuda_fail(e, "cudaSetDevice");
    StepJob &job = s->job;
    job.shards = shards;
    job.mode = mode;
    job.row_count = row_count;
    job.root_queries = root_queries;
    job.root_output = root_output;
    job.direct = direct;
    const uint32_t q_units = static_cast<uint32_t>(q_row / 16u), o_units = static_cast<uint32_t>(o_row / 16u);

    if (mode == CF_B200_MG_BY_SEQUENCE && !direct) {
        // query rows into device-major order on the root (one kernel), one copy per device out, one per device back,
        // output rows back into batch order (one kernel)
        uint32_t at = 0;
        bool changed = s->last_perm.size() != listed;
        for (uint32_t d = 0; d < devices; ++d) {
            job.first_row[d] = at;
            for (uint32_t i = 0; i < shards[d].desc.seq_count; ++i, ++at) {
                const uint32_t row = shards[d].rows ? shards[d].rows[i] : i;
                if (!changed && s->last_perm[at] != row) changed = true;
                s->h_perm[at] = row;
            }
        }
        if (changed) {   // a new placement: the row order goes to the root device (a few hundred bytes)
            e = cudaMemcpyAsync(s->d_perm, s->h_perm, sizeof(uint32_t) * listed, cudaMemcpyHostToDevice, root_stream);
            if (e != cudaSuccess) return s->cuda_fail(e, "row order upload");
            e = cudaStreamSynchronize(root_stream);   // h_perm is rewritten by the next call
            if (e != cudaSuccess) return s->cuda_fail(e, "row order upload");
            s->last_perm.assign(s->h_perm, s->h_perm + listed);
        }
        const uint32_t blocks = std::min<uint32_t>(1024u, (listed * q_units + 255u) / 256u);
        permute_rows_kernel<true><<<blocks, 256, 0, root_stream>>>(static_cast<const uint4 *>(root_queries),
                                                                   reinterpret_cast<uint4 *>(s->staging_q), s->d_perm, listed, q_units);
    } else if (mode == CF_B200_MG_BY_KV_HEAD) {
        for (uint32_t d = 0; d < devices; ++d)
            if (shards[d].desc.seq_count && (shards[d].rows || shards[d].desc.seq_count != row_count))
                return s->fail(CF_ERR_INVALID_ARGUMENT, "kv-head sharding serves every row on every device");
    }
    if ((e = cudaEventRecord(s->ready, root_stream)) != cudaSuccess) return s->cuda_fail(e, "cudaEventRecord");

    // every device's share is queued by its own thread (the root's by this one), then the root stream waits for all
    for (uint32_t d = 0; d < devices; ++d) s->device_status[d] = CF_OK;
    s->pending.store(static_cast<uint32_t>(s->workers.size()), std::memory_order_release);
    s->step_seq.fetch_add(1u, std::memory_order_release);
    if (!s->workers.empty()) s->wake_cv.notify_all();
    if (shards[0].desc.seq_count) s->device_status[0] = submit_device(s, 0);
    while (s->pending.load(std::memory_order_acquire) != 0u) std::this_thread::yield();
    for (uint32_t d = 0; d < devices; ++d) {
        if (shards[d].desc.seq_count == 0) continue;
        if (s->device_status[d] != CF_OK) return s->fail(s->device_status[d], s->device_error[d]);
        ++s->counters.attention_launches;
        if (d != 0) {
            const cf_b200_sealed_attention_desc &desc = shards[d].desc;
            const uint32_t span = desc.kv_head_span ? desc.kv_head_span : desc.kv_head_count - desc.kv_head_begin;
            s->counters.peer_copies += direct ? 1u : 2u;   // direct: the outputs cross as stores of the combine kernel
            s->counters.peer_bytes += direct ? q_row * row_count + (mode == CF_B200_MG_BY_SEQUENCE
                                                      ? o_row * desc.seq_count
                                                      : static_cast<size_t>(span) * (desc.query_head_count / desc.kv_head_count) *
                                                            desc.head_dim * 4u * row_count)
                                      : mode == CF_B200_MG_BY_SEQUENCE
                                          ? (q_row + o_row) * desc.seq_count
                                          : q_row * row_count + static_cast<size_t>(span) * (desc.query_head_count / desc.kv_head_count) *
                                                                    desc.head_dim * 4u * row_count;
        }
        if ((e = cudaStreamWaitEvent(root_stream, s->done[d], 0)) != cudaSuccess) return s->cuda_fail(e, "cudaStreamWaitEvent");
    }
    if (mode == CF_B200_MG_BY_SEQUENCE && !direct) {
        const uint32_t oblocks = std::min<uint32_t>(1024u, (listed * o_units + 255u) / 256u);
        permute_rows_kernel<false><<<oblocks, 256, 0, root_stream>>>(reinterpret_cast<const uint4 *>(s->staging_out),
                                                                     static_cast<uint4 *>(root_output), s->d_perm, listed, o_units);
        if ((e = cudaPeekAtLastError()) != cudaSuccess) return s->cuda_fail(e, "row permutation");
    }
    ++s->counters.steps;
    if (direct) ++s->counters.direct_steps;
    s->error.clear();
    return CF_OK;
}

extern "C" cf_status cf_b200_mg_get_counters(const cf_b200_mg_scheduler *s, cf_b200_mg_counters *out) {
    if (!s || !out) return CF_ERR_INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(s->mutex);
    *out = s->counters;
    return CF_OK;
}
