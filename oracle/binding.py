"""ctypes binding of the CPU oracle (liboracle.so) and of the reference's own sources built into
oracle/_ref. Test infrastructure: only tests, the smoke check and the benchmark's CPU-baseline leg import it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

CODER_FIXED8, CODER_HUFFMAN, CODER_RANS, CODER_RANS_SPLIT4, CODER_HUFFMAN_SPLIT4 = 0, 1, 2, 3, 4


def build(with_ref=None):
    """Compile liboracle.so; also oracle/_ref when the reference tree is present (or with_ref=True)."""
    targets = ["all"]
    # the reference tree: CF_REFERENCE_ROOT, or a checkout named `reference` beside this repository
    ref_root = os.environ.get("CF_REFERENCE_ROOT", os.path.abspath(os.path.join(HERE, "..", "..", "reference")))
    if with_ref is None:
        with_ref = os.path.isdir(os.path.join(ref_root, "src", "runtime"))
    if with_ref:
        targets.append("ref")
        # the reference's own test programs, linked against this repository's library (which must be built already)
        if os.path.exists(os.path.join(HERE, "..", "chromofold_b200", "libchromofold_b200.so")):
            targets += ["reftests", "benchmarks"]
    subprocess.run(["make", "-C", HERE, f"REF={ref_root}"] + targets, check=True, capture_output=True)


_lib = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            build(with_ref=False)
        _lib = C.CDLL(path)
        _lib.orc_half_to_float.restype = C.c_float
        _lib.orc_half_to_float.argtypes = [C.c_uint16]
        _lib.orc_float_to_half.restype = C.c_uint16
        _lib.orc_float_to_half.argtypes = [C.c_float]
        _lib.orc_rans_encode.restype = C.c_int64
        _lib.orc_huff_encode.restype = C.c_int64
        _lib.orc_seal_record.restype = C.c_uint32
        _lib.orc_seal_record_symbols.restype = C.c_uint32
        _lib.orc_hardware_threads.restype = C.c_uint
    return _lib


def ref_cpu():
    """The reference's CPU sources (None when oracle/_ref was not built)."""
    path = os.path.join(HERE, "_ref", "libcfref_cpu.so")
    return C.CDLL(path) if os.path.exists(path) else None


def ref_cuda():
    """The reference's CUDA sources for this path, compiled for sm_100a (None when not built)."""
    path = os.path.join(HERE, "_ref", "libcfref_cuda.so")
    return C.CDLL(path) if os.path.exists(path) else None


def ref_mscache():
    """The reference's host sequence cache (src/multisequence_cache.cpp) with the tensor-view validator it calls
    (None when not built)."""
    path = os.path.join(HERE, "_ref", "libcfref_mscache.so")
    return C.CDLL(path) if os.path.exists(path) else None


def ref_msbridge():
    """The reference's llama-server multisequence bridge (integrations/llama.cpp/multisequence/
    llama_server_multisequence_bridge.cpp over its host cache; None when not built)."""
    path = os.path.join(HERE, "_ref", "libcfref_msbridge.so")
    return C.CDLL(path) if os.path.exists(path) else None


def ref_device():
    """The reference's own decode runtime, seal engine, sequence resolver and dataplane (src/cuda/production_attention.cu,
    device_kv_seal_attention.cu, multisequence_cuda_resolver.cu, device_kv_dataplane.cu), compiled for sm_100a (None when
    not built)."""
    path = os.path.join(HERE, "_ref", "libcfref_device.so")
    return C.CDLL(path) if os.path.exists(path) else None


def ref_adapter():
    """The reference's llama KV adapter with everything under it (integrations/llama.cpp/chromofold_kv_adapter.cpp,
    src/runtime/compressed_kv_cache.cu, its quantiser and its paged-attention kernel), compiled for sm_100a (None when not
    built)."""
    path = os.path.join(HERE, "_ref", "libcfref_adapter.so")
    return C.CDLL(path) if os.path.exists(path) else None


def reference_test_programs():
    """{name: path} of the reference's own test programs built against this repository's library (oracle/_ref/reftests)."""
    folder = os.path.join(HERE, "_ref", "reftests")
    if not os.path.isdir(folder):
        return {}
    return {name: os.path.join(folder, name) for name in sorted(os.listdir(folder)) if os.access(os.path.join(folder, name), os.X_OK)}


def _p(a, t=None):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


class Codebook(C.Structure):
    _fields_ = [("freq", C.c_int32 * 256), ("cum", C.c_int32 * 256), ("slot2sym", C.c_int32 * 4096),
                ("hlen", C.c_uint8 * 256), ("hcode", C.c_uint32 * 256), ("lut", C.c_int32 * 4096)]

    def np(self, name):
        return np.ctypeslib.as_array(getattr(self, name)).copy()


def codebook_from_hist(hist):
    hist = np.ascontiguousarray(hist, np.uint64)
    assert hist.shape == (256,)
    cb = Codebook()
    lib().orc_codebook_build(_p(hist), C.byref(cb))
    return cb


def rans_encode(sym, block, cb):
    sym = np.ascontiguousarray(sym, np.uint8)
    n = sym.size
    nb = (n + block - 1) // block
    data = np.zeros(2 * n + 8, np.uint8)
    off = np.zeros(nb, np.int32)
    st = np.zeros(nb, np.uint32)
    used = lib().orc_rans_encode(_p(sym), C.c_int(n), C.c_int(block), cb.freq, cb.cum, _p(data), _p(off), _p(st))
    return data[:used].copy(), off, st


def rans_decode(data, off, st, cb, block, n):
    out = np.zeros(n, np.int32)
    padded = np.concatenate([np.ascontiguousarray(data, np.uint8), np.zeros(8, np.uint8)])
    lib().orc_rans_decode(_p(padded), _p(np.ascontiguousarray(off, np.int32)), _p(np.ascontiguousarray(st, np.uint32)),
                          cb.slot2sym, cb.freq, cb.cum, C.c_int(block), C.c_int(n), _p(out))
    return out


def huff_encode(sym, block, cb):
    sym = np.ascontiguousarray(sym, np.uint8)
    n = sym.size
    words = np.zeros((n * 12 + 31) // 32 + 2, np.uint32)
    off = np.zeros((n + block - 1) // block, np.int32)
    used = lib().orc_huff_encode(_p(sym), C.c_int(n), C.c_int(block), cb.hlen, cb.hcode, _p(words), _p(off))
    return words[:used].copy(), off


def huff_decode(words, off, cb, block, n):
    out = np.zeros(n, np.uint8)
    padded = np.concatenate([np.ascontiguousarray(words, np.uint32), np.zeros(2, np.uint32)])
    lib().orc_huff_decode(_p(padded), _p(np.ascontiguousarray(off, np.int32)), cb.lut, C.c_int(12), C.c_int(block),
                          C.c_int(n), _p(out))
    return out


def quantize_stream(x):
    x = np.ascontiguousarray(x, np.float32).ravel()
    codes = np.zeros(x.size, np.int8)
    scale = C.c_uint16(0)
    rc = lib().orc_quantize_stream(_p(x), C.c_uint32(x.size), C.byref(scale), _p(codes))
    return rc, scale.value, codes


def record_capacity(head_dim, page_tokens, block):
    n = head_dim * page_tokens
    nb = (n + block - 1) // block
    return 2 * (n + 6 * nb) + 128


def seal_record(k, v, token_count, head_dim, page_tokens, block, coder, codebook_id, kcb, vcb):
    """k, v: float32 [token_count][head_dim]. Returns (record bytes, k symbols, v symbols) or None if not finite."""
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    n = head_dim * page_tokens
    rec = np.zeros(record_capacity(head_dim, page_tokens, block), np.uint8)
    ks = np.zeros(n, np.uint8)
    vs = np.zeros(n, np.uint8)
    size = lib().orc_seal_record(_p(k), _p(v), C.c_uint32(token_count), C.c_uint32(head_dim), C.c_uint32(page_tokens),
                                 C.c_uint32(block), C.c_uint32(coder), C.c_uint32(codebook_id), C.byref(kcb),
                                 C.byref(vcb), _p(rec), _p(ks), _p(vs))
    if size == 0:
        return None
    return rec[:size].copy(), ks, vs


def seal_record_symbols(k_sym, v_sym, k_scale_bits, v_scale_bits, token_count, head_dim, page_tokens, block, coder,
                        codebook_id, kcb, vcb):
    k_sym = np.ascontiguousarray(k_sym, np.uint8)
    v_sym = np.ascontiguousarray(v_sym, np.uint8)
    rec = np.zeros(record_capacity(head_dim, page_tokens, block), np.uint8)
    size = lib().orc_seal_record_symbols(_p(k_sym), _p(v_sym), C.c_uint16(k_scale_bits), C.c_uint16(v_scale_bits),
                                         C.c_uint32(token_count), C.c_uint32(head_dim), C.c_uint32(page_tokens),
                                         C.c_uint32(block), C.c_uint32(coder), C.c_uint32(codebook_id), C.byref(kcb),
                                         C.byref(vcb), _p(rec))
    return rec[:size].copy()


def open_record(rec, head_dim, page_tokens, block, kcb, vcb):
    n = head_dim * page_tokens
    ks = np.zeros(n, np.uint8)
    vs = np.zeros(n, np.uint8)
    padded = np.concatenate([np.ascontiguousarray(rec, np.uint8), np.zeros(16, np.uint8)])
    rc = lib().orc_open_record(_p(padded), C.c_uint32(head_dim), C.c_uint32(page_tokens), C.c_uint32(block),
                               C.byref(kcb), C.byref(vcb), _p(ks), _p(vs))
    assert rc == 0
    return ks, vs


def dense_attention(keys, values, token_begin, queries, query_token_begin, causal_window, score_scale):
    """keys/values float32 [Hkv][T][D]; queries float32 [Q][Hq][D] -> (rc, out [Q][Hq][D])."""
    keys = np.ascontiguousarray(keys, np.float32)
    values = np.ascontiguousarray(values, np.float32)
    queries = np.ascontiguousarray(queries, np.float32)
    hkv, t, d = keys.shape
    nq, hq, _ = queries.shape
    out = np.zeros_like(queries)
    rc = lib().orc_dense_attention(_p(keys), _p(values), C.c_uint32(token_begin), C.c_uint32(t), _p(queries),
                                   C.c_uint32(nq), C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(d),
                                   C.c_uint32(query_token_begin), C.c_uint32(causal_window), C.c_float(score_scale),
                                   _p(out))
    return rc, out


def sealed_decode_attention(arena, dir_offset, page_table, seq_tokens, queries_f16, hq, hkv, head_dim, page_tokens,
                            block, causal_window, score_scale, kcb, vcb, tail_k=None, tail_v=None, tail_count=None,
                            threads=None):
    """Batch decode-step attention from sealed records on the CPU. queries_f16: uint16 bits [S][Hq][D]."""
    arena = np.ascontiguousarray(arena, np.uint8)
    dir_offset = np.ascontiguousarray(dir_offset, np.uint64)
    page_table = np.ascontiguousarray(page_table, np.uint32)
    seq_tokens = np.ascontiguousarray(seq_tokens, np.uint32)
    queries_f16 = np.asarray(queries_f16)
    if queries_f16.dtype != np.float16 and queries_f16.dtype != np.uint16:   # fp32 queries: the oracle's rows are binary16
        narrowed = queries_f16.astype(np.float16)
        if not np.array_equal(narrowed.astype(queries_f16.dtype), queries_f16):
            raise ValueError("the oracle takes binary16 queries; these values do not survive the narrowing")
        queries_f16 = narrowed
    q = np.ascontiguousarray(queries_f16).view(np.uint16)
    s = seq_tokens.size
    out = np.zeros((s, hq, head_dim), np.float32)
    if tail_count is not None:
        tail_k = np.ascontiguousarray(tail_k).view(np.uint16)
        tail_v = np.ascontiguousarray(tail_v).view(np.uint16)
        tail_count = np.ascontiguousarray(tail_count, np.uint32)
    if threads is None:
        threads = lib().orc_hardware_threads()
    rc = lib().orc_sealed_decode_attention(
        _p(arena), _p(dir_offset), _p(page_table), C.c_uint32(page_table.shape[1]), _p(seq_tokens), C.c_uint32(s),
        _p(tail_k), _p(tail_v), _p(tail_count), _p(q), C.c_uint32(hq), C.c_uint32(hkv), C.c_uint32(head_dim),
        C.c_uint32(page_tokens), C.c_uint32(block), C.c_uint32(causal_window), C.c_float(score_scale), C.byref(kcb),
        C.byref(vcb), C.c_uint32(threads), _p(out))
    assert rc == 0, rc
    return out
