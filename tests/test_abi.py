"""The shared library loads without a GPU, exports every symbol its headers declare, and validates arguments
before touching CUDA (the reference's conformance rule, packaging/conformance.c:33-38)."""
import ctypes as C
import os
import re

import numpy as np

from helpers import hist_of, laplace_codes

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    text = open(os.path.join(ROOT, "include", "chromofold_b200", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return set(re.findall(r"\b(cf_[a-z0-9_]+)\s*\(", text))


def test_every_declared_symbol_is_exported(native):
    lib = native.lib()
    headers = [h for h in os.listdir(os.path.join(ROOT, "include", "chromofold_b200")) if h.endswith(".h")]
    seen = 0
    for h in headers:
        # one header's functions live in a library of their own (its names clash with another header's)
        where = native.ms_bridge_lib() if h in native.MS_BRIDGE_EXPORTS else lib
        for name in _declared(h):
            assert hasattr(where, name), f"{h}: {name} is declared but not exported"
            seen += 1
    assert seen >= 10
    assert b"sm_100a" in lib.cf_b200_build_info()


def test_struct_sizes_match_the_headers(native):
    # computed by hand from the header layouts; a mismatch means the ctypes mirror drifted
    assert C.sizeof(native.CodebookTables) == 4096 * 4 + 256 * 2 + 256 * 2 + 4096 * 2 + 256 * 4 + 256 * 8
    assert C.sizeof(native.SealedAttentionDesc) == 224
    assert C.sizeof(native.SealDesc) == 160
    assert C.sizeof(native.DenseAttentionDesc) == 120


def test_null_and_bad_arguments_are_rejected_before_cuda(native):
    lib = native.lib()
    assert lib.cf_b200_sealed_attention_validate(None) == native.CF_ERR_INVALID_ARGUMENT
    assert lib.cf_b200_sealed_attention_async(None, None) == native.CF_ERR_INVALID_ARGUMENT
    assert lib.cf_b200_seal_pages_async(None, None) == native.CF_ERR_INVALID_ARGUMENT
    assert lib.cf_b200_codebook_build(None, None) == native.CF_ERR_INVALID_ARGUMENT
    d = native.SealedAttentionDesc()
    d.struct_size, d.abi_version = C.sizeof(d), native.ABI_VERSION
    assert lib.cf_b200_sealed_attention_validate(C.byref(d)) == native.CF_ERR_INVALID_ARGUMENT   # zero geometry
    d.kv_head_count, d.query_head_count, d.head_dim, d.page_tokens, d.block_size = 8, 32, 128, 16, 64
    d.softmax_scale, d.seq_count = 0.088, 1
    for f in ("queries", "output", "workspace", "seq_sealed_tokens", "k_tables", "v_tables"):
        setattr(d, f, 0x1000)   # fake device pointers, never dereferenced (tests/paged_kv_cuda_seam.cu:12-13)
    d.workspace_bytes = 1 << 20
    d.query_type, d.output_type = native.F16, native.F32
    assert lib.cf_b200_sealed_attention_validate(C.byref(d)) == native.CF_OK
    d.query_head_count = 30                                  # GQA mismatch
    assert lib.cf_b200_sealed_attention_validate(C.byref(d)) == native.CF_ERR_INVALID_ARGUMENT
    d.query_head_count = 32
    d.softmax_scale = float("nan")
    assert lib.cf_b200_sealed_attention_validate(C.byref(d)) == native.CF_ERR_INVALID_ARGUMENT
    d.softmax_scale = 0.088
    d.head_dim = 256                                         # beyond CF_KV_MAX_HEAD_DIM
    assert lib.cf_b200_sealed_attention_validate(C.byref(d)) == native.CF_ERR_UNSUPPORTED
    d.head_dim = 128
    d.abi_version = 7
    assert lib.cf_b200_sealed_attention_validate(C.byref(d)) == native.CF_ERR_INVALID_ARGUMENT
    d.abi_version = native.ABI_VERSION
    d.tail_tokens = 0x1000                                   # tail count without tail rows
    assert lib.cf_b200_sealed_attention_validate(C.byref(d)) == native.CF_ERR_INVALID_ARGUMENT
    d.tail_tokens = None
    d.workspace_bytes = 64                                   # no room for a single partial
    assert lib.cf_b200_sealed_attention_validate(C.byref(d)) == native.CF_ERR_INVALID_ARGUMENT


def test_codebook_tables_match_oracle(native, oracle):
    """The library's codebook builder and the oracle's implement the same stated rule, independently."""
    rng = np.random.default_rng(3)
    hists = [hist_of(laplace_codes(rng, 50000, b).astype(np.int16) + 128) for b in (0.7, 4.0, 12.0, 60.0)]
    hists += [np.zeros(256, np.uint64), np.ones(256, np.uint64), hist_of(np.full(9, 128, np.uint8))]
    for hist in hists:
        cb = oracle.codebook_from_hist(hist)
        t = native.CodebookTables()
        assert native.lib().cf_b200_codebook_build(hist.ctypes.data_as(C.c_void_p), C.byref(t)) == 0
        assert np.array_equal(np.ctypeslib.as_array(t.rans_freq), cb.np("freq"))
        assert np.array_equal(np.ctypeslib.as_array(t.rans_cum), cb.np("cum"))
        slot = np.ctypeslib.as_array(t.rans_slot)
        assert np.array_equal(slot & 0xFF, cb.np("slot2sym"))
        s2s = cb.np("slot2sym")
        assert np.array_equal((slot >> 8) & 0xFFF, cb.np("freq")[s2s])
        assert np.array_equal(slot >> 20, np.arange(4096) - cb.np("cum")[s2s])
        assert np.array_equal(np.ctypeslib.as_array(t.huff_lut).astype(np.int32), cb.np("lut"))
        code = np.ctypeslib.as_array(t.huff_code)
        assert np.array_equal(code & 0xFFFF, cb.np("hcode")) and np.array_equal(code >> 16, cb.np("hlen"))
        # the sealer's reciprocals divide exactly: floor(x / f) for states at both ends of the range and around multiples of f
        enc = np.ctypeslib.as_array(t.rans_enc).astype(np.uint64)
        f, cum = cb.np("freq").astype(np.uint64), cb.np("cum").astype(np.uint64)
        assert np.array_equal((enc[:, 1] >> np.uint64(13)) & np.uint64(0xFFF), np.uint64(4096) - f)
        for x in (1 << 23, (1 << 31) - 1, 12345678, (1 << 27) + 5):
            xs = np.concatenate([np.full(256, x, np.uint64), (np.uint64(x) // f) * f, (np.uint64(x) // f) * f - np.uint64(1)])
            e = np.tile(enc, (3, 1))
            q = ((xs * e[:, 0]) >> np.uint64(32)) >> (e[:, 1] >> np.uint64(25))
            nxt = xs + (e[:, 1] & np.uint64(0x1FFF)) + q * ((e[:, 1] >> np.uint64(13)) & np.uint64(0xFFF))
            ff, cc = np.tile(f, 3), np.tile(cum, 3)
            assert np.array_equal(nxt, ((xs // ff) << np.uint64(12)) + xs % ff + cc)


def test_every_c_header_compiles_as_c11():
    """The boundary is a C ABI: every header under include/chromofold_b200 (the C++ convenience class apart) must be
    usable from plain C, as the reference requires of its own runtime headers (.github/workflows/m9-runtime.yml:34-48)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        import pytest
        pytest.skip("no C compiler here")
    include = os.path.join(ROOT, "include")
    for h in sorted(os.listdir(os.path.join(include, "chromofold_b200"))):
        if not h.endswith(".h"):
            continue
        done = subprocess.run([gcc, "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-I" + include, "-x", "c", "-"],
                              input=f'#include "chromofold_b200/{h}"\nint main(void) {{ return 0; }}\n', text=True,
                              capture_output=True)
        assert done.returncode == 0, f"{h}: {done.stderr[:400]}"
