// delta_fetch.cu — cf_delta_fetch_async (include/chromofold/chromofold.h; src/cuda/delta_apply.cu:12-44): token-id
// look-up in a reference/delta cluster. A cluster is one base sequence plus, per member ("leaf"), a sorted list of
// (position, value) overrides: fetch(leaf, pos) = the leaf's override at pos if it has one, else base[pos], else -1
// past the end of the base.
//
// The look-up is a latency-bound gather: one thread per query (grid-stride past 2^28 queries), a binary search over
// the leaf's override positions, every read through the read-only path. No allocation, no synchronisation.

#include "chromofold_b200/compat_kv.h"

namespace {

__global__ void __launch_bounds__(256) delta_fetch_kernel(const int32_t *__restrict__ base, int nbase,
                                                          const int32_t *__restrict__ dpos, const int32_t *__restrict__ dval,
                                                          const int32_t *__restrict__ dstart, const int32_t *__restrict__ dlen,
                                                          const int32_t *__restrict__ leaf_in, const int32_t *__restrict__ pos_in,
                                                          int32_t *__restrict__ out, size_t count) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < count;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int leaf = __ldg(leaf_in + i), pos = __ldg(pos_in + i);
        int result = (pos >= 0 && pos < nbase) ? __ldg(base + pos) : -1;
        const int first = __ldg(dstart + leaf), n = __ldg(dlen + leaf);
        int lo = 0, hi = n;   // first override position >= pos
        while (lo < hi) {
            const int mid = (lo + hi) >> 1;
            if (__ldg(dpos + first + mid) < pos) lo = mid + 1;
            else hi = mid;
        }
        if (lo < n && __ldg(dpos + first + lo) == pos) result = __ldg(dval + first + lo);
        out[i] = result;
    }
}

}  // namespace

extern "C" cf_status cf_delta_fetch_async(const int32_t *base, int nbase, const int32_t *dpos, const int32_t *dval,
                                          const int32_t *dstart, const int32_t *dlen, const int32_t *device_leaf,
                                          const int32_t *device_pos, int32_t *out, size_t count, void *stream) {
    if (!base || !dstart || !dlen || !device_leaf || !device_pos || !out) return CF_ERR_INVALID_ARGUMENT;  // delta_apply.cu:36
    if (count == 0) return CF_OK;
    const size_t blocks = (count + 255) / 256;
    const unsigned grid = static_cast<unsigned>(blocks < (1u << 20) ? blocks : (1u << 20));
    delta_fetch_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(base, nbase, dpos, dval, dstart, dlen, device_leaf,
                                                                            device_pos, out, count);
    return cudaPeekAtLastError() == cudaSuccess ? CF_OK : CF_ERR_CUDA;
}
