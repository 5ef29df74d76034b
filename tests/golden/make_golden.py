"""Generate the golden vectors under tests/golden from the reference's own sources.

Run in a container that has the reference tree (it builds oracle/_ref first):

    python tests/golden/make_golden.py

Every array written here is an OUTPUT OF THE REFERENCE's code (src/runtime/kv_reference.cpp,
kv_gpu_fixture.cpp, kv_runtime.cpp, include/chromofold/detail/block_huffman_device.cuh) on seeded
synthetic inputs; the inputs are stored beside the outputs. The oracle is then checked against these files
wherever the reference tree is absent.
"""
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import binding as ob  # noqa: E402


def p(a):
    return a.ctypes.data_as(C.c_void_p)


def fixture_pages(ref, rng):
    out = {}
    for name, (tokens, dim, block, bits) in {
        "int8_16x128": (16, 128, 64, 8),
        "int4_16x128": (16, 128, 64, 4),
        "int8_9x32": (9, 32, 64, 8),
        "int4_70x64": (70, 64, 64, 4),
    }.items():
        n = tokens * dim
        k = rng.standard_normal(n).astype(np.float32)
        v = rng.standard_normal(n).astype(np.float32)
        words = (n * bits + 31) // 32
        nb = (n + block - 1) // block
        kw = np.zeros(words, np.uint32)
        vw = np.zeros(words, np.uint32)
        ko = np.zeros(nb, np.int32)
        vo = np.zeros(nb, np.int32)
        lut = np.zeros(1 << bits, np.int32)
        ksc = np.zeros(dim, np.float32)
        vsc = np.zeros(tokens, np.float32)
        dk = np.zeros(n, np.float32)
        dv = np.zeros(n, np.float32)
        res = C.c_uint64(0)
        rc = ref.ref_fixture_encode(p(k), p(v), C.c_uint32(3), C.c_uint32(tokens), C.c_uint32(dim), C.c_uint32(1),
                                    C.c_uint32(block), C.c_uint32(bits), p(kw), p(ko), p(vw), p(vo), p(lut), p(ksc),
                                    p(vsc), p(dk), p(dv), C.byref(res))
        assert rc == 0
        ksym = np.zeros(n, np.uint8)
        assert ref.ref_fixture_decode(p(kw), C.c_uint64(words), C.c_uint32(bits), C.c_uint64(n), p(ksym)) == 0
        vsym = np.zeros(n, np.uint8)
        assert ref.ref_fixture_decode(p(vw), C.c_uint64(words), C.c_uint32(bits), C.c_uint64(n), p(vsym)) == 0
        for key, val in dict(k=k, v=v, k_words=kw, v_words=vw, k_offsets=ko, v_offsets=vo, lut=lut, k_scales=ksc,
                             v_scales=vsc, dequantized_k=dk, dequantized_v=dv, k_symbols=ksym, v_symbols=vsym,
                             shape=np.array([tokens, dim, block, bits, res.value], np.int64)).items():
            out[f"{name}.{key}"] = val
    np.savez_compressed(os.path.join(HERE, "fixture_pages.npz"), **out)


def paged_attention(ref, rng):
    """The scenario of the reference's tests/kv_reference_test.cpp:119-173 and wider ones, on seeded inputs."""
    out = {}
    cases = {
        # name: (Hq, Hkv, D, page sizes, tail tokens, query count, query_token_begin, window)
        "gqa4x2_pages4_6_tail3_win7": (4, 2, 8, [4, 6], 3, 3, 10, 7),
        "gqa8x2_d64_full": (8, 2, 64, [16, 16, 16, 5], 2, 1, 54, 0),
        "mha_d128_window": (4, 4, 128, [16, 16], 0, 1, 31, 20),
        "gqa32x8_d128": (32, 8, 128, [16] * 3, 7, 1, 55, 0),
    }
    for name, (hq, hkv, d, sizes, tail, nq, qbegin, window) in cases.items():
        sealed = sum(sizes)
        k = rng.standard_normal((hkv, sealed, d)).astype(np.float32)
        v = rng.standard_normal((hkv, sealed, d)).astype(np.float32)
        tk = rng.standard_normal((hkv, max(tail, 1), d)).astype(np.float32)
        tv = rng.standard_normal((hkv, max(tail, 1), d)).astype(np.float32)
        q = rng.standard_normal((nq, hq, d)).astype(np.float32)
        scale = np.float32(1.0 / np.sqrt(d))
        dk = np.zeros_like(k)
        dv = np.zeros_like(v)
        res = np.zeros((nq, hq, d), np.float32)
        sz = np.array(sizes, np.uint32)
        rc = ref.ref_paged_attention_int4(p(k), p(v), C.c_uint32(sealed), p(sz), C.c_uint32(len(sizes)), p(tk), p(tv),
                                          C.c_uint32(tail), p(q), C.c_uint32(nq), C.c_uint32(hq), C.c_uint32(hkv),
                                          C.c_uint32(d), C.c_uint32(qbegin), C.c_uint32(window), C.c_float(scale),
                                          C.c_int(0), p(res), p(dk), p(dv))
        assert rc == 0, (name, rc)
        rev = np.zeros_like(res)
        rc = ref.ref_paged_attention_int4(p(k), p(v), C.c_uint32(sealed), p(sz), C.c_uint32(len(sizes)), p(tk), p(tv),
                                          C.c_uint32(tail), p(q), C.c_uint32(nq), C.c_uint32(hq), C.c_uint32(hkv),
                                          C.c_uint32(d), C.c_uint32(qbegin), C.c_uint32(window), C.c_float(scale),
                                          C.c_int(1), p(rev), None, None)
        assert rc == 0
        for key, val in dict(k=k, v=v, tail_k=tk[:, :tail], tail_v=tv[:, :tail], q=q, dequantized_k=dk,
                             dequantized_v=dv, output=res, output_reversed_pages=rev,
                             shape=np.array([hq, hkv, d, tail, nq, qbegin, window], np.int64),
                             page_sizes=sz).items():
            out[f"{name}.{key}"] = val
    np.savez_compressed(os.path.join(HERE, "paged_attention.npz"), **out)


class SoftmaxState(C.Structure):
    _fields_ = [("max_score", C.c_double), ("exp_sum", C.c_double), ("weighted_values", C.POINTER(C.c_double)),
                ("dim", C.c_uint32), ("initialized", C.c_uint32)]


def online_softmax(ref, rng):
    """cf_online_softmax_{init,accumulate,merge,finalize}: the split of tests/kv_runtime_test.cpp:122-158 and a
    seeded 3-way split at dim 128."""
    out = {}
    cases = {
        "extreme_scores": (np.array([-1000.0, -2.0, 3.0, 2.5, 900.0, 899.0]),
                           np.array([[1, 0, 0, 0], [0, 1, 0, 0], [0, 0, 1, 0], [0, 0, 0, 1], [1, 2, 3, 4],
                                     [4, 3, 2, 1]], np.float32), [3, 6]),
        "seeded_d128": (rng.standard_normal(40) * 6.0, rng.standard_normal((40, 128)).astype(np.float32),
                        [11, 12, 40]),
    }
    for name, (scores, values, cuts) in cases.items():
        dim = values.shape[1]
        merged_buf = (C.c_double * dim)()
        merged = SoftmaxState()
        assert ref.cf_online_softmax_init(C.byref(merged), merged_buf, C.c_uint32(dim)) == 0
        begin = 0
        partial_max, partial_sum, partial_w = [], [], []
        for end in cuts:
            buf = (C.c_double * dim)()
            st = SoftmaxState()
            assert ref.cf_online_softmax_init(C.byref(st), buf, C.c_uint32(dim)) == 0
            for i in range(begin, end):
                row = np.ascontiguousarray(values[i])
                assert ref.cf_online_softmax_accumulate(C.byref(st), C.c_double(scores[i]), p(row)) == 0
            partial_max.append(st.max_score)
            partial_sum.append(st.exp_sum)
            partial_w.append(np.array(buf[:]))
            assert ref.cf_online_softmax_merge(C.byref(merged), C.byref(st)) == 0
            begin = end
        final = np.zeros(dim, np.float32)
        assert ref.cf_online_softmax_finalize(C.byref(merged), p(final)) == 0
        for key, val in dict(scores=scores, values=values, cuts=np.array(cuts), partial_max=np.array(partial_max),
                             partial_sum=np.array(partial_sum), partial_weighted=np.array(partial_w),
                             merged_max=np.array(merged.max_score), merged_sum=np.array(merged.exp_sum),
                             merged_weighted=np.array(merged_buf[:]), output=final).items():
            out[f"{name}.{key}"] = val
    np.savez_compressed(os.path.join(HERE, "online_softmax.npz"), **out)


def huffman_decode(ref, rng):
    """Variable-length streams (written by the oracle's encoder) decoded by the reference's cf_bh_decode_at."""
    out = {}
    for name, b in {"laplace_b4": 4.0, "laplace_b12": 12.0, "laplace_b0p7": 0.7}.items():
        n = 2048
        sym = (np.rint(rng.laplace(0, b, n)).clip(-128, 127).astype(np.int64) + 128).astype(np.uint8)
        cb = ob.codebook_from_hist(np.bincount(sym, minlength=256))
        words, off = ob.huff_encode(sym, 64, cb)
        lut = cb.np("lut")
        dec = np.zeros(n, np.uint8)
        padded = np.concatenate([words, np.zeros(2, np.uint32)])
        for blk in range(n // 64):
            pos = int(off[blk])
            for j in range(64):
                sl = ref.ref_bh_decode_at(p(padded), p(lut), C.c_int(12), C.c_int(pos))
                dec[blk * 64 + j] = sl & 0xFF
                pos += sl >> 8
        assert np.array_equal(dec, sym)
        for key, val in dict(words=words, offsets=off, lut=lut, decoded_by_reference=dec).items():
            out[f"{name}.{key}"] = val
    np.savez_compressed(os.path.join(HERE, "huffman_decode.npz"), **out)


def delta_cluster():
    """A small reference/delta cluster frozen by the reference's own exporter (tools/export_delta.py, numpy only):
    base + sparse per-member overrides + the original sequences the fetch must reproduce."""
    import subprocess
    ref_root = os.environ.get("CF_REFERENCE_ROOT", os.path.abspath(os.path.join(HERE, "..", "..", "..", "reference")))
    subprocess.run([sys.executable, os.path.join(ref_root, "tools", "export_delta.py"), os.path.join(HERE, "delta_cluster.cfdc"),
                    "--members", "12", "--base", "600", "--divergence", "0.02", "--suffix", "24", "--vocab", "50000",
                    "--seed", "7"], check=True)


def main():
    ob.build(with_ref=True)
    ref = ob.ref_cpu()
    assert ref is not None
    rng = np.random.default_rng(20240611)
    fixture_pages(ref, rng)
    paged_attention(ref, rng)
    online_softmax(ref, rng)
    huffman_decode(ref, rng)
    delta_cluster()
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz") or f.endswith(".cfdc"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
