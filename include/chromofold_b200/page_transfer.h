/* page_transfer.h — moving sealed pages out of one arena and into another: the warm-start file and the
 * prefill -> decode hand-over of the reference (record + FNV-1a checksum of src/persistent_page_store.cpp:11-15,
 * PAGE_MANIFEST / PAGE_DATA of docs/m16-disaggregated-serving.md:14), for format-v1 records.
 *
 * A transfer image is three parts, all little-endian:
 *   cf_b200_transfer_header (64 bytes)
 *   manifest: record_count entries of cf_b200_transfer_entry (16 bytes), page-major, kv head minor
 *   payload:  the records, each at its entry's 16-byte offset, packed without gaps
 * The codebooks a record was sealed with are NOT in the image: the header names them by codebook_id, and the receiving
 * side must hold the same tables (cf_b200_codebook_build of the same histogram), as the attention kernels check.
 *
 * pack writes manifest and payload on the device from (arena, page directory, page ids); unpack verifies every
 * record against its checksum, takes room in the destination arena with the same atomic cursor the sealer uses,
 * copies, and publishes directory entries for the given destination page ids. A record whose checksum or size does
 * not match is not published (its directory entry stays 0) and CF_B200_DEVSTAT_CHECKSUM is raised. Both calls follow
 * the conventions of sealed_kv.h: device pointers, no allocation, no synchronisation. */
#ifndef CHROMOFOLD_B200_PAGE_TRANSFER_H
#define CHROMOFOLD_B200_PAGE_TRANSFER_H

#include <stdint.h>

#include "chromofold_b200/sealed_kv.h"

#ifdef __cplusplus
extern "C" {
#endif

#define CF_B200_TRANSFER_MAGIC 0x3147504643ull /* "CFPG1" */
#define CF_B200_DEVSTAT_CHECKSUM 0x40u         /* a transferred record failed its checksum or size check */

typedef struct cf_b200_transfer_header {
    uint64_t magic;
    uint32_t version;          /* 1 */
    uint32_t format_version;   /* CF_B200_FORMAT_VERSION of the records */
    uint32_t kv_head_count, head_dim, page_tokens, block_size, codebook_id, page_count;
    uint64_t payload_bytes;    /* sum of the record lengths */
    uint64_t manifest_checksum; /* FNV-1a over the manifest bytes */
    uint64_t reserved;
} cf_b200_transfer_header;

typedef struct cf_b200_transfer_entry {
    uint32_t offset_units;     /* record offset in the payload / 16 */
    uint32_t length_units;     /* record length / 16; 0 = the page had no record for this kv head */
    uint64_t checksum;         /* cf_b200_record_checksum of the record */
} cf_b200_transfer_entry;

/* manifest[page_count * kv_head_count], payload[payload_capacity_bytes], payload_cursor_units (one u64, zeroed by the
 * caller, holds the packed length / 16 afterwards). A record that does not fit raises CF_B200_DEVSTAT_ARENA_FULL. */
cf_status cf_b200_pages_pack_async(const uint8_t *arena, const uint64_t *page_dir, uint32_t kv_head_count,
                                   const uint32_t *page_ids, uint32_t page_count, cf_b200_transfer_entry *manifest,
                                   uint8_t *payload, uint64_t payload_capacity_bytes,
                                   unsigned long long *payload_cursor_units, uint32_t *status, void *stream);

/* The inverse: records go to `arena` (room taken from arena_cursor_units, the sealer's cursor) and page_dir entries
 * of dst_page_ids are written. */
cf_status cf_b200_pages_unpack_async(const cf_b200_transfer_entry *manifest, const uint8_t *payload, uint64_t payload_bytes,
                                     uint32_t kv_head_count, const uint32_t *dst_page_ids, uint32_t page_count,
                                     uint8_t *arena, uint64_t arena_units, unsigned long long *arena_cursor_units,
                                     uint64_t *page_dir, uint32_t *status, void *stream);

/* FNV-1a on the host with the reference's constants (basis 1469598103934665603 — the reference's, which is not the
 * standard 64-bit basis — and prime 1099511628211, src/persistent_page_store.cpp:14): the manifest checksum. */
uint64_t cf_b200_fnv1a(const void *bytes, uint64_t count);
/* The record checksum, on the host. FNV-1a is a serial recurrence, so a record (a multiple of 16 bytes) is hashed as
 * 32 interleaved lanes: h_l = FNV-1a over the bytes of the 16-byte units l, l + 32, l + 64, ... (the basis for a lane
 * without units), and the checksum is FNV-1a over h_0 .. h_31, 8 little-endian bytes each. */
uint64_t cf_b200_record_checksum(const void *record, uint64_t bytes);

#ifdef __cplusplus
}
#endif

#endif
