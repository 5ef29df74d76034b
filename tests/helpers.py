"""Seeded synthetic inputs shared by the tests (shapes and distributions of the benchmark configurations)."""
import numpy as np

from oracle import binding as ob


def laplace_codes(rng, shape, b):
    """Discretised Laplace(b) clipped to int8, as the benchmark configurations name it."""
    return np.rint(rng.laplace(0.0, b, shape)).clip(-128, 127).astype(np.int8)


def geometric_codes(rng, shape, p):
    """Two-sided geometric P(k) ~ (1-p)^|k| clipped to int8."""
    mag = rng.geometric(p, shape) - 1
    sign = rng.integers(0, 2, shape) * 2 - 1
    return (mag * sign).clip(-128, 127).astype(np.int8)


def codes_to_values(codes, scale):
    """fp16 K/V values whose per-stream quantisation gives back `codes` (the stream must contain +-127 or be
    scaled so that absmax/127 rounds to `scale`)."""
    return (codes.astype(np.float32) * np.float32(scale)).astype(np.float16)


def hist_of(symbols):
    return np.bincount(np.asarray(symbols, np.uint8).ravel(), minlength=256).astype(np.uint64)


SPLIT_CODERS = (3, 4)   # CF_B200_CODER_RANS_SPLIT4, CF_B200_CODER_HUFFMAN_SPLIT4


def pair_hist_of(symbols):
    """Histogram of the pair symbols the nibble-split coders code: hi(s[2k]) << 4 | hi(s[2k+1])."""
    s = np.asarray(symbols, np.uint8).ravel()
    s = s[:s.size // 2 * 2]
    return np.bincount((s[0::2] & 0xF0) | (s[1::2] >> 4), minlength=256).astype(np.uint64)


def hist_for_coder(symbols, coder):
    """The histogram a codebook for `coder` is built from: pair symbols for the nibble-split coders."""
    return pair_hist_of(symbols) if coder in SPLIT_CODERS else hist_of(symbols)


class HostCache:
    """CPU-side sealed cache built with the oracle encoder: the reference point for GPU parity checks."""

    def __init__(self, hkv, head_dim, page_tokens, block, coder, kcb, vcb, codebook_id=0):
        self.hkv, self.d, self.t, self.block, self.coder = hkv, head_dim, page_tokens, block, coder
        self.kcb, self.vcb, self.codebook_id = kcb, vcb, codebook_id
        self.records = {}   # slot -> list of pages -> list of per-head records
        self.symbols = {}   # slot -> list of pages -> list of (ksym, vsym)
        self.tokens = {}    # slot -> list of token counts

    def seal_page(self, slot, k, v, token_count=None):
        """k, v: float32 [hkv][tokens][d] (values already rounded to binary16)."""
        tokens = k.shape[1] if token_count is None else token_count
        recs, syms = [], []
        for h in range(self.hkv):
            r = ob.seal_record(k[h, :tokens], v[h, :tokens], tokens, self.d, self.t, self.block, self.coder,
                               self.codebook_id, self.kcb, self.vcb)
            assert r is not None
            recs.append(r[0])
            syms.append((r[1], r[2]))
        self.records.setdefault(slot, []).append(recs)
        self.symbols.setdefault(slot, []).append(syms)
        self.tokens.setdefault(slot, []).append(tokens)

    def flat(self, slots, stride):
        """Arena bytes, directory offsets, page table and sealed lengths in the oracle's layout."""
        blobs, offsets, cursor = [], [0] * self.hkv, 0  # page id 0 unused
        table = np.zeros((len(slots), stride), np.uint32)
        sealed = np.zeros(len(slots), np.uint32)
        pid = 1
        for i, s in enumerate(slots):
            for p, page in enumerate(self.records.get(s, [])):
                table[i, p] = pid
                pid += 1
                for rec in page:
                    offsets.append(cursor)
                    blobs.append(rec)
                    cursor += rec.size
            sealed[i] = sum(self.tokens.get(s, []))
        arena = np.concatenate(blobs + [np.zeros(64, np.uint8)]) if blobs else np.zeros(64, np.uint8)
        return arena, np.array(offsets, np.uint64), table, sealed


def attention_close(actual, expected, rel=2e-3, abs_=1e-3):
    """The benchmark's bar: |a - e| <= abs + rel * |e| element-wise."""
    actual = np.asarray(actual, np.float64)
    expected = np.asarray(expected, np.float64)
    err = np.abs(actual - expected)
    return bool(np.all(err <= abs_ + rel * np.abs(expected))), float(err.max())


def oracle_from_layer(layer, q16, causal_window=0, slots=None, threads=None):
    """CPU oracle attention over the very records a SealedKvLayer holds on the GPU (arena, directory, page table and
    tails are copied back): restated reference decoders -> dequantise -> double online softmax."""
    kcb = ob.codebook_from_hist(np.ones(256, np.uint64))
    vcb = ob.codebook_from_hist(np.ones(256, np.uint64))
    for cb, host in ((kcb, layer.host_tables[0]), (vcb, layer.host_tables[1])):
        slot = np.ctypeslib.as_array(host.rans_slot)
        cb.slot2sym[:] = (slot & 0xFF).astype(np.int32).tolist()
        cb.freq[:] = np.ctypeslib.as_array(host.rans_freq).astype(np.int32).tolist()
        cb.cum[:] = np.ctypeslib.as_array(host.rans_cum).astype(np.int32).tolist()
        cb.lut[:] = np.ctypeslib.as_array(host.huff_lut).astype(np.int32).tolist()
    arena = layer.arena[:layer.sealed_bytes() + 64].cpu().numpy()
    offsets = (layer.page_dir.cpu().numpy().astype(np.uint64) & np.uint64(0xFFFFFFFFFF)) * np.uint64(16)
    sel = np.arange(layer.max_sequences) if slots is None else np.asarray(slots)
    table = layer.page_table.cpu().numpy().astype(np.uint32)[sel]
    sealed = layer.sealed_tokens.cpu().numpy().astype(np.uint32)[sel]
    tails = layer.tail_tokens.cpu().numpy().astype(np.uint32)[sel]
    tk = layer.tail_k.cpu().numpy()[sel]
    tv = layer.tail_v.cpu().numpy()[sel]
    return ob.sealed_decode_attention(arena, offsets, table, sealed, q16, layer.query_heads, layer.kv_heads, layer.head_dim,
                                      layer.page_tokens, layer.block_size, causal_window, 1.0 / np.sqrt(layer.head_dim),
                                      kcb, vcb, tail_k=tk, tail_v=tv, tail_count=tails, threads=threads)
