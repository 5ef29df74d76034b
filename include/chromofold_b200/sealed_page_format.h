/* sealed_page_format.h — byte layout of one sealed KV page record (format v1).
 *
 * A record holds the K and V codes of ONE (page, kv_head): page_tokens x head_dim
 * int8 codes each, entropy coded in independent fixed-count blocks. The conventions
 * come from the reference's block streams:
 *   - block-rANS stream  : src/cuda/rans.cu:11-26 (PROB_BITS 12, M 4096, L 2^23, byte
 *                          renormalisation, per block a start state and a byte offset),
 *                          tools/export_rans.py:13-17 (data | byte_off | state0 | tables)
 *   - block-Huffman stream: include/chromofold/detail/block_huffman_device.cuh:12-19
 *                          (u32 words, bits MSB-first, per block a bit offset, one LUT of
 *                          2^maxlen entries sym | len<<8)
 *   - fixed-width stream : src/runtime/kv_gpu_fixture.cpp:20-43 (8-bit symbols packed
 *                          MSB-first into u32 words)
 *   - symbol = code + zero_point, zero_point 128 for int8 (kv_gpu_fixture.cpp:54-62)
 * What the reference does not have (it keeps LUTs, offsets and fp32 scale vectors per
 * page, kv_cuda.h:21-41) and this format adds: coding tables live in a shared codebook,
 * one fp16 absmax scale per stream, and one contiguous 16-byte aligned record so a page
 * can be fetched with a single bulk copy.
 *
 * Record (all little-endian, every part 16-byte aligned):
 *   +0                     cf_b200_record_header (16 B)
 *   +16                    K part, k_part_units * 16 bytes
 *   +16 + 16*k_part_units  V part, v_part_units * 16 bytes
 *
 * Part layout by coder (nblocks = ceil(page_tokens*head_dim / block_size)):
 *   RANS    : u32 state0[nblocks] | u16 byte_off[nblocks] | pad to 4 | payload bytes | pad to 16
 *             byte_off is relative to the first payload byte.
 *   HUFFMAN : u16 bit_off[nblocks] | pad to 4 | payload u32 words (MSB-first) | pad to 16
 *             bit_off is relative to the first payload bit.
 *   FIXED8  : payload u32 words, symbol i in bits [31-8*(i%4)-7 .. 31-8*(i%4)] of word i/4
 *   RANS_SPLIT4    : u32 state0[nblocks] | u16 byte_off[nblocks] | pad to 4 | u32 lo[block_size/8][nblocks] | payload | pad to 16
 *   HUFFMAN_SPLIT4 : u16 bit_off[nblocks] | pad to 4 | u32 lo[block_size/8][nblocks] | payload u32 words | pad to 16
 *
 * The nibble-split coders store the LOW nibble of every symbol raw and entropy-code the HIGH nibbles two at a
 * time: pair symbol k of a block = hi(symbol 2k) << 4 | hi(symbol 2k+1), coded by the same block-rANS / block-
 * Huffman stream as above (block_size/2 pair symbols per block, tables built over pair symbols). One step of the
 * reference's recurrence (rans.cu:20-23) or one LUT hit then yields two codes, and at 5-7 bits of entropy per code
 * the low nibble is so close to uniform that storing it raw costs ~1.5 % (Laplace b = 12). The raw plane is the
 * reference's fixed-width idea (kv_gpu_fixture.cpp:20-43) at 4 bits, laid out for the decoder: lo[j][b] holds the
 * low nibbles of symbols 8j..8j+7 of block b — symbol 8j+i at bits 8i..8i+3 for i < 4, symbol 8j+4+i at bits
 * 8i+4..8i+7 — word-interleaved across blocks, so that 32 lanes decoding 32 blocks read 32 different banks.
 * Needs block_size % 8 == 0 and page_tokens*head_dim % 8 == 0.
 *
 * Symbol order inside a stream:
 *   K: flat index = token * head_dim + dim   (the reference order, kv_gpu_fixture.cpp:83)
 *   V: flat index = dim * page_tokens + token (token-minor). A decoding lane owns one
 *      block, so with this order it owns whole channels and the PV contraction over
 *      tokens needs no cross-lane transpose.
 * Tokens at index >= token_count (a page sealed before it was full) are coded as the
 * zero_point symbol and are masked out by the consumer.
 *
 * Limits of v1: page_tokens*head_dim <= 4096 (16-bit block offsets), head_dim <= 128,
 * block_size in [16, 1024].
 */
#ifndef CHROMOFOLD_B200_SEALED_PAGE_FORMAT_H
#define CHROMOFOLD_B200_SEALED_PAGE_FORMAT_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CF_B200_FORMAT_VERSION 1u
#define CF_B200_RECORD_ALIGN 16u
#define CF_B200_ZERO_POINT 128

#define CF_B200_CODER_FIXED8 0u
#define CF_B200_CODER_HUFFMAN 1u
#define CF_B200_CODER_RANS 2u
#define CF_B200_CODER_RANS_SPLIT4 3u
#define CF_B200_CODER_HUFFMAN_SPLIT4 4u
#define CF_B200_CODER_MAX 4u

/* rans.cu:11-13 */
#define CF_B200_RANS_PROB_BITS 12u
#define CF_B200_RANS_M (1u << CF_B200_RANS_PROB_BITS)
#define CF_B200_RANS_L (1u << 23)

/* Huffman codes are length-limited so one LUT hit resolves a symbol
 * (block_huffman_device.cuh:10-11). */
#define CF_B200_HUFF_MAXLEN 12u
#define CF_B200_HUFF_LUT_SIZE (1u << CF_B200_HUFF_MAXLEN)

#define CF_B200_MAX_STREAM_SYMBOLS 4096u

typedef struct cf_b200_record_header {
    uint16_t k_part_units;   /* K part length in 16-byte units */
    uint16_t v_part_units;   /* V part length in 16-byte units */
    uint8_t k_coder;         /* CF_B200_CODER_* */
    uint8_t v_coder;
    uint16_t token_count;    /* valid tokens, 1..page_tokens */
    uint16_t k_scale_f16;    /* IEEE binary16 bits; dequant = (sym - 128) * scale */
    uint16_t v_scale_f16;
    uint16_t codebook_id;
    uint8_t flags;
    uint8_t version;         /* CF_B200_FORMAT_VERSION */
} cf_b200_record_header;

/* Shared coding tables for one stream kind (K or V) of one codebook.
 *   rans_slot[slot] = sym | (freq[sym] << 8) | ((slot - cum[sym]) << 20)
 *     — the three table reads of rans.cu:20-22 folded into one word. Every symbol has
 *     freq >= 1 and freq <= 3841, so 12 bits hold it.
 *   rans_freq / rans_cum are the plain tables of rans.cu:17-18 (the sealer needs them).
 *   huff_lut[look] = sym | (len << 8), block_huffman_device.cuh:12-19.
 *   huff_code[sym] = code | (len << 16), the sealer's side of the same code.
 *   rans_enc[sym] = { rcp, cum | (4096 - freq) << 13 | (shift - 1) << 25 } with shift = ceil(log2 freq) and
 *     rcp = ceil(2^(31 + shift) / freq): the sealer's division-free step, floor(x / freq) = umulhi(x, rcp) >> (shift - 1)
 *     for x < 2^31 and x' = x + cum + floor(x / freq) * (4096 - freq). freq = 1: { 2^32 - 1, (cum + 4095) | 4095 << 13 }. */
typedef struct cf_b200_codebook_tables {
    uint32_t rans_slot[4096];
    uint16_t rans_freq[256];
    uint16_t rans_cum[256];
    uint16_t huff_lut[4096];
    uint32_t huff_code[256];
    uint32_t rans_enc[256][2];
} cf_b200_codebook_tables;

#ifdef __cplusplus
}
#endif

#endif
