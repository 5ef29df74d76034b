/* sealed_kv.h — C ABI of the B200 sealed-KV decode-attention path.
 *
 * These entry points sit beside the reference's symbols (compat_kv.h). They exist because the reference
 * descriptors cannot express the target workloads: its launch takes at most 4096 page descriptors of 104
 * bytes each by value (include/chromofold/kv_cuda.h:13,21-41), has fp32-only queries (:68-69), keeps LUTs
 * and scale vectors per page, and has no rANS page at all (src/cuda/rans.cu is a flat stream decoder).
 *
 * Conventions are the reference's (include/chromofold/chromofold.h:25-30,48-50; specs/00-constitution.md):
 *   - every function returns cf_status; CF_OK means "launch accepted", not "finished";
 *   - `stream` is a cudaStream_t passed as void*, NULL is the default stream;
 *   - a required pointer that is NULL gives CF_ERR_INVALID_ARGUMENT before any CUDA call;
 *   - versioned structs carry struct_size and abi_version and are rejected when they do not match;
 *   - the *_async query-path calls allocate nothing, never synchronise and copy nothing between host and
 *     device; the caller owns stream ordering;
 *   - there is no CPU or dense fallback: when no CUDA device is usable the calls fail with CF_ERR_CUDA.
 */
#ifndef CHROMOFOLD_B200_SEALED_KV_H
#define CHROMOFOLD_B200_SEALED_KV_H

#include <stddef.h>
#include <stdint.h>

#include "chromofold_b200/cf_status.h"
#include "chromofold_b200/sealed_page_format.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CF_B200_ABI_VERSION 1u

/* Scalar types of query / output / appended K,V tensors; values of the reference's cf_device_scalar_type
 * (include/chromofold/device_kv_dataplane.h:11-15). */
#define CF_B200_F16 1u
#define CF_B200_BF16 2u
#define CF_B200_F32 3u

/* Page directory entry: where the record of (page_id, kv_head) lies in the arena.
 *   bits  0..39 : byte offset / 16
 *   bits 40..55 : record length / 16
 *   bits 56..63 : 0 (reserved) */
#define CF_B200_DIR_ENTRY(offset_units, length_units) \
    (((uint64_t)(offset_units) & 0xFFFFFFFFFFull) | ((uint64_t)(length_units) << 40))
#define CF_B200_DIR_OFFSET_UNITS(e) ((e) & 0xFFFFFFFFFFull)
#define CF_B200_DIR_LENGTH_UNITS(e) (((e) >> 40) & 0xFFFFull)

/* --------------------------------------------------------------------------------------------------
 * Raw launch: decode-step attention of a batch of sequences over sealed pages. The caller owns all
 * memory. Replaces, for sealed pages, cf_kv_paged_attention_async (include/chromofold/kv_cuda.h:86,
 * src/cuda/paged_kv_attention.cu:301-327) and the per-item launches of cf_ms_cuda_execute_batch_async
 * (src/cuda/multisequence_cuda_resolver.cu:376-419) and cf_attention_execute_async
 * (src/cuda/production_attention.cu:170-211).
 *
 * Semantics (src/cuda/paged_kv_attention.cu:41-176, src/runtime/kv_reference.cpp:164-243):
 *   one query token per sequence at position sealed_tokens + tail_tokens; visible tokens are
 *   window_begin <= t <= query position with window_begin as in paged_kv_attention.cu:50-52;
 *   score = (sum_d q[d] * (sym-128) * k_scale) * softmax_scale; one online softmax over all pages and the
 *   tail; output = weighted / sum; query head h reads kv head h / (Hq / Hkv); a sequence with no visible
 *   token gets zeros (paged_kv_attention.cu:170-173).
 * All pointers are DEVICE pointers. */
typedef struct cf_b200_sealed_attention_desc {
    uint32_t struct_size;
    uint32_t abi_version;

    uint32_t kv_head_count;     /* kv heads present in page_dir and in the tails */
    uint32_t query_head_count;  /* Hq of the whole layer; Hq % kv_head_count == 0 */
    uint32_t head_dim;
    uint32_t page_tokens;
    uint32_t block_size;
    uint32_t kv_head_begin;     /* this launch serves kv heads [kv_head_begin, kv_head_begin+kv_head_span) */
    uint32_t kv_head_span;      /* and the query heads that map to them; 0 means all */
    uint32_t codebook_id;

    const uint8_t *arena;
    const uint64_t *page_dir;            /* [page_id * kv_head_count + kv_head] */
    const uint32_t *page_table;          /* [slot][page_table_stride] page ids */
    const uint32_t *seq_sealed_tokens;   /* [slot] */
    const uint32_t *seq_slots;           /* [seq_count] batch index -> slot; NULL = identity */
    uint32_t page_table_stride;
    uint32_t seq_count;

    const cf_b200_codebook_tables *k_tables;
    const cf_b200_codebook_tables *v_tables;

    const void *tail_k;                  /* [slot][kv_head_count][tail_capacity][head_dim] of tail_type, may be NULL */
    const void *tail_v;
    const uint32_t *tail_tokens;         /* [slot], NULL = no tails */

    const void *queries;                 /* [seq_count][query_head_count][head_dim] */
    void *output;                        /* same shape */
    uint32_t query_type;                 /* CF_B200_F16 or CF_B200_F32. At head_dim 128 / 96 / 64 / 32 an fp32 row is
                                          * contracted as binary16(q) + binary16(q - binary16(q)) (scores equal to the
                                          * fp32 product to 2^-22 relative), which holds finite |q| up to 65504; larger
                                          * components give NaN there. Other geometries compute in fp32 throughout. */
    uint32_t output_type;                /* CF_B200_F16 or CF_B200_F32 */
    float softmax_scale;
    uint32_t causal_window;              /* 0 = all history */

    void *workspace;                     /* split-KV partials; see cf_b200_sealed_attention_workspace_bytes */
    uint64_t workspace_bytes;
    uint32_t min_pages_per_unit;         /* pages per split-KV unit; 0 = the library chooses (4 to 35) on the device, from the
                                            pages the launch will read: the size whose rounds over the GPU's resident
                                            warps cost least, among those whose partials fit the workspace. A unit's
                                            weighted sum is kept by the tensor cores in fp32; its rounding drifts by
                                            about 1e-7 of the output's scale per page, so units of hundreds of pages
                                            are a few 1e-5 off where the library's own sizes stay below 4e-6 */
    uint32_t kernel;                     /* CF_B200_KERNEL_* */
    uint32_t *status;                    /* optional device word; a kernel ORs CF_B200_DEVSTAT_* into it */
    uint32_t tail_type;                  /* CF_B200_F16 (0 means F16 too) or CF_B200_F32: element type of the tails */
    uint32_t tail_capacity;              /* rows per (slot, kv head) in tail_k / tail_v; 0 = page_tokens */
    /* Optional [seq_count]: position of each batch entry's query token. NULL = sealed + tail tokens (a decode
     * step). A smaller position hides the tokens after it (paged_kv_attention.cu:67-69), so several entries may
     * name the same slot with different positions: that is multi-query (prefill) attention over one sequence. */
    const uint32_t *query_positions;
    /* Shared prefix: the caller states that the first shared_prefix_pages entries of the page-table row of EVERY
     * listed sequence name the same pages (one sealed copy referenced by all, src/multisequence_cache.cpp:235-292).
     * Such pages are then decoded once per 128 query rows instead of once per sequence, and the contraction with all
     * the rows that share them runs on the tensor cores. Entries that name the SAME slot with different
     * query_positions (multi-query / prefill attention) share all of that slot's sealed pages this way. It is a
     * hint: the plan kernel checks the rows and that every entry's query position lies at or after the last shared
     * token; if not, or the geometry is not the lanes kernel's, or causal_window is in use, every page is handled
     * per entry as if the field were 0 (a failed check also raises CF_B200_DEVSTAT_PREFIX_MISMATCH).
     * The workspace must have been sized with the field set (cf_b200_sealed_attention_workspace_bytes). */
    uint32_t shared_prefix_pages;
    uint32_t reserved0;
    /* Optional [seq_count], device memory: batch entry i reads row row_map[i] of `queries` and writes row row_map[i] of
     * `output` instead of row i. A call can then serve a subset of a larger batch in place — the multi-GPU scheduler
     * (sealed_kv_multigpu.h) gives every GPU the rows of its own sequences this way. NULL = entry i is row i. The rows
     * of one call must be distinct (two entries writing one output row would race). The shared-prefix hint is not
     * used together with a row map. */
    const uint32_t *row_map;
} cf_b200_sealed_attention_desc;

#define CF_B200_KERNEL_AUTO 0u     /* lane-per-block tensor-core kernel when the geometry allows, else generic */
#define CF_B200_KERNEL_GENERIC 1u  /* any geometry within the format limits */
#define CF_B200_KERNEL_LANES 2u    /* head_dim 128, page_tokens 16, block_size 64, group <= 16; else UNSUPPORTED */
/* Measurement only: the lanes kernel's page fetch and entropy decode without its attention — every symbol the launch
 * would decode is folded into a checksum that replaces the partials; the output of the call is meaningless. Use it
 * with CF_B200_STAGE_PLAN | CF_B200_STAGE_ATTENTION to time the decode floor of a workload. */
#define CF_B200_KERNEL_DECODE_PROBE 3u
/* Test only: the lanes kernel (and, with shared_prefix_pages set, the shared-prefix kernel) runs its page fetch and
 * its per-lane block decoders as in an attention call, and stores every symbol they yield instead of consuming it:
 * `output` is then a device byte buffer [reserved0 page ids][kv_head_count][2][page_tokens * head_dim] — the K stream
 * and the V stream of each record, in stream order, one byte per symbol — and reserved0 (otherwise 0) is the number
 * of page ids it covers; records of other page ids are refused with CF_B200_DEVSTAT_BAD_RECORD. Only pages some
 * listed sequence reaches are written. Stages: CF_B200_STAGE_PLAN | CF_B200_STAGE_ATTENTION. */
#define CF_B200_KERNEL_DECODE_DUMP 4u

#define CF_B200_DEVSTAT_BAD_RECORD 0x1u      /* version / codebook id / size mismatch in a record header */
#define CF_B200_DEVSTAT_WAIT_EXPIRED 0x2u    /* a bounded wait on a bulk copy ran out */
#define CF_B200_DEVSTAT_WORKSPACE 0x4u       /* workspace too small for the planned units */
#define CF_B200_DEVSTAT_NONFINITE 0x8u       /* the sealer met NaN or Inf; the page was not published */
#define CF_B200_DEVSTAT_ARENA_FULL 0x10u     /* the sealer found no room in the arena */
#define CF_B200_DEVSTAT_PREFIX_MISMATCH 0x20u /* shared_prefix_pages was set but the page-table rows differ */
#define CF_B200_DEVSTAT_TAIL_FULL 0x80u      /* an append found its slot's unsealed tail full; the row was not stored */
#define CF_B200_SHARED_CHUNKS_MAX 16u        /* a batch entry's shared-prefix result comes in at most this many partials */

/* Test hook for the bounded waits of the attention kernels: from the next launch on, the record of page id
 * skip_copy_page_id is armed on its barrier but never fetched, and every wait gives up after wait_polls polls (each
 * poll is bounded to about a microsecond). The warp whose wait runs out raises CF_B200_DEVSTAT_WAIT_EXPIRED and leaves
 * in an orderly way (copies still in flight are given a bounded chance to land, tensor memory is freed); the launch
 * ends normally with an incomplete result. (0, 0) switches the hook off and restores the default bound. Process-wide. */
cf_status cf_b200_test_wait_expiry(uint32_t skip_copy_page_id, uint32_t wait_polls);

/* Host-side structural validation; dereferences nothing on the device
 * (cf_kv_validate_paged_attention_desc, src/cuda/paged_kv_attention.cu:280-299). */
cf_status cf_b200_sealed_attention_validate(const cf_b200_sealed_attention_desc *desc);

/* Workspace needed so that a batch with at most total_pages sealed pages (summed over sequences) never
 * has to grow its units beyond min_pages_per_unit (or, with 0, beyond 16 pages, 4 for small batches). A smaller
 * workspace is legal: units grow to fit. */
cf_status cf_b200_sealed_attention_workspace_bytes(const cf_b200_sealed_attention_desc *desc,
                                                   uint64_t total_pages, uint64_t *out_bytes);

cf_status cf_b200_sealed_attention_async(const cf_b200_sealed_attention_desc *desc, void *stream);

/* The same launch cut into its three kernels, so that a profiler or a benchmark can put events between them:
 * plan (chunk layout, one block), attention (the kernel that reads the pages), combine (merge + tail + output).
 * `stages` is a mask; running all three in order equals cf_b200_sealed_attention_async. */
#define CF_B200_STAGE_PLAN 1u
#define CF_B200_STAGE_ATTENTION 2u
#define CF_B200_STAGE_COMBINE 4u
cf_status cf_b200_sealed_attention_stages_async(const cf_b200_sealed_attention_desc *desc, uint32_t stages,
                                                void *stream);

/* The same attention for callers that cannot allocate device memory (an engine that gave the whole heap to its
 * own arena, a plugin inside another framework's budget, a serving thread where allocator calls are banned).
 * This entry point has no counterpart in the reference. It takes the descriptor of
 * cf_b200_sealed_attention_async, ignores `workspace` / `workspace_bytes`, and uses a fixed array inside the
 * library image instead: CF_B200_STATIC_WORKSPACE_BYTES per GPU that loads the library, held until exit.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine.
 *   - A batch whose partials cannot fit (seq_count x local query heads x (head_dim + 2) floats, one chunk per
 *     sequence at least) is rejected with CF_ERR_UNSUPPORTED; cf_b200_sealed_attention_static_error() says why and
 *     how many bytes were needed. Larger contexts are fine: chunks grow to fit the array. A shared_prefix_pages hint
 *     needs CF_B200_SHARED_CHUNKS_MAX more partials per sequence and query head; when only those do not fit, the
 *     call is served without the hint (every page then handled per sequence) instead of refused.
 *   - The first call on a device looks up the array's device address; make that call outside any stream capture.
 *   - All calls on a device share the array. Calls that overlap on the GPU race; order them on one stream or with
 *     events. Nothing has to be cleared between calls: each call rewrites what it reads. */
#define CF_B200_STATIC_WORKSPACE_BYTES (8u << 20)
cf_status cf_b200_sealed_attention_static_async(const cf_b200_sealed_attention_desc *desc, void *stream);
const char *cf_b200_sealed_attention_static_error(void);

/* --------------------------------------------------------------------------------------------------
 * Codebooks. Built on the host from symbol histograms (set-up work, not query path).
 * Normalisation rule for rANS (M = 4096, every symbol codable):
 *   f_i = 1 + floor(h_i * 3840 / N), the left-over slots go to the largest remainders (ties: lower symbol).
 * Huffman: weights 2*h_i + 1, lengths limited to 12, canonical codes in (length, symbol) order.
 * The reference has no codebook builder in-tree (tools/export_rans.py:27-29 imports it from elsewhere). */
cf_status cf_b200_codebook_build(const uint64_t histogram[256], cf_b200_codebook_tables *out_tables);

/* --------------------------------------------------------------------------------------------------
 * Raw launch: seal full active pages on the GPU. Replaces cf_device_seal_full_page_async
 * (src/cuda/device_kv_seal_attention.cu:244-334: finite scan, quantise, pack, publish — six launches, a
 * host synchronisation and nine allocations per page) with one launch and no host round trip.
 *
 * For every job j: reads rows job_rows[j] .. job_rows[j] + job_tokens[j] of slot job_slots[j] from tail_k / tail_v
 * ([slot][kv_head_count][tail_capacity][head_dim] of tail_type), quantises each
 * (kv_head, K|V) stream with its own absmax/127 binary16 scale (round-half-even, clamp [-128,127],
 * src/runtime/kv_gpu_fixture.cpp:12-16), codes it with `coder` (a stream that would not shrink is stored
 * fixed-width), takes room in the arena with one atomic add on *arena_cursor_units, writes the record and
 * then the directory entry of (job_pages[j], kv_head). A page with a non-finite value is not published: its
 * directory entries stay 0 and CF_B200_DEVSTAT_NONFINITE is set (device_kv_seal_attention.cu:255-267). */
typedef struct cf_b200_seal_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t kv_head_count;
    uint32_t head_dim;
    uint32_t page_tokens;
    uint32_t block_size;
    uint32_t coder;               /* CF_B200_CODER_* */
    uint32_t codebook_id;
    const cf_b200_codebook_tables *k_tables;
    const cf_b200_codebook_tables *v_tables;
    const void *tail_k;
    const void *tail_v;
    const uint32_t *job_slots;    /* [job_count] */
    const uint32_t *job_pages;    /* [job_count] page ids to publish */
    const uint32_t *job_tokens;   /* [job_count] valid rows, NULL = page_tokens */
    const uint32_t *job_heads;    /* [job_count] kv head of each job; NULL = every job seals all kv heads */
    const uint32_t *job_rows;     /* [job_count] first tail row of the tile to seal; NULL = 0 */
    uint32_t job_count;
    uint32_t tail_type;           /* CF_B200_F16 (0 means F16 too) or CF_B200_F32 */
    uint32_t tail_capacity;       /* rows per (slot, kv head) in tail_k / tail_v; 0 = page_tokens */
    uint32_t reserved;
    uint8_t *arena;
    uint64_t arena_units;                     /* capacity in 16-byte units */
    unsigned long long *arena_cursor_units;   /* device counter, next free unit */
    uint64_t *page_dir;
    uint32_t *status;
} cf_b200_seal_desc;

cf_status cf_b200_seal_validate(const cf_b200_seal_desc *desc);
cf_status cf_b200_seal_pages_async(const cf_b200_seal_desc *desc, void *stream);

/* Raw launch: append one token to the unsealed tails of the listed slots (the reference's append step,
 * src/cuda/device_kv_dataplane.cu:150-190, as one launch for a whole decode batch). Row i
 * (k_rows / v_rows: [row_count][kv_head_count][head_dim] of row_type — the element types a model's KV rows come in,
 * cf_device_tensor_view: fp16, bf16, fp32 — device memory) is stored at position
 * tail_tokens[slots[i]] of that slot's tails ([slot][kv_head_count][tail_capacity][head_dim] of tail_type) and the
 * count is raised by one. A slot may be listed once per call. A full tail (count == tail_capacity) takes nothing and
 * raises CF_B200_DEVSTAT_TAIL_FULL: seal first (cf_b200_seal_pages_async), then the caller resets the count. */
typedef struct cf_b200_append_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t kv_head_count;
    uint32_t head_dim;
    uint32_t tail_capacity;
    uint32_t tail_type;       /* CF_B200_F16 (0 too) or CF_B200_F32 */
    void *tail_k;
    void *tail_v;
    uint32_t *tail_tokens;    /* [slot] */
    const uint32_t *slots;    /* [row_count], distinct */
    const void *k_rows;
    const void *v_rows;
    uint32_t row_type;        /* CF_B200_F16, CF_B200_BF16 or CF_B200_F32 */
    uint32_t row_count;
    uint32_t *status;         /* optional */
} cf_b200_append_desc;
cf_status cf_b200_append_rows_async(const cf_b200_append_desc *desc, void *stream);

/* Symbol histograms of quantised K and V streams of the same tails (for codebook calibration).
 * hist_k / hist_v: device uint64[256], accumulated into (not cleared). */
cf_status cf_b200_histogram_async(const cf_b200_seal_desc *desc, unsigned long long *hist_k,
                                  unsigned long long *hist_v, void *stream);

/* Decode records back to symbols on the GPU (no attention): k_symbols / v_symbols are device uint8
 * [job][kv_head_count][page_tokens*head_dim] in stream order. This is the bit-exactness probe: the same
 * decode routines the attention kernels use, with the codes written out instead of consumed. */
cf_status cf_b200_decode_pages_async(const cf_b200_sealed_attention_desc *desc, const uint32_t *page_ids,
                                     uint32_t page_count, uint8_t *k_symbols, uint8_t *v_symbols, void *stream);

/* --------------------------------------------------------------------------------------------------
 * Comparison kernel: the same attention over UNCOMPRESSED binary16 pages, same page table and split-KV
 * skeleton, only the read differs (the reference's fairness rule for its dense comparison,
 * tests/latency_bench.cu). pool_k / pool_v: binary16 [page_id][kv_head_count][page_tokens][head_dim]. */
typedef struct cf_b200_dense_attention_desc {
    uint32_t struct_size;
    uint32_t abi_version;
    uint32_t kv_head_count;
    uint32_t query_head_count;
    uint32_t head_dim;
    uint32_t page_tokens;
    const void *pool_k;
    const void *pool_v;
    const uint32_t *page_table;
    const uint32_t *seq_sealed_tokens;
    const uint32_t *seq_slots;
    uint32_t page_table_stride;
    uint32_t seq_count;
    const void *queries;     /* binary16 */
    void *output;            /* float */
    float softmax_scale;
    uint32_t causal_window;
    void *workspace;
    uint64_t workspace_bytes;
    uint32_t min_pages_per_unit;
    uint32_t reserved;
} cf_b200_dense_attention_desc;

cf_status cf_b200_dense_attention_async(const cf_b200_dense_attention_desc *desc, void *stream);

/* Build identification; also what a loader calls to check that the library carries device code. */
const char *cf_b200_build_info(void);

/* Diagnostics: how many attention calls of this process launched the shared-prefix kernel (a shared_prefix_pages hint
 * given by the caller, or worked out by one of the stores behind the reference's ABIs for forked sequences and
 * prefill batches). A launch whose hint the plan kernel then refuses raises CF_B200_DEVSTAT_PREFIX_MISMATCH. */
unsigned long long cf_b200_shared_prefix_launches(void);

#ifdef __cplusplus
}
#endif

#endif
