"""Reference/delta cluster fetch (cf_delta_fetch_async): the oracle against the cluster the reference's exporter
froze (tests/golden/delta_cluster.cfdc), and the CUDA entry point against both."""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import delta

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "delta_cluster.cfdc")


def _all_queries(c):
    leaf = np.concatenate([np.full(c["lengths"][i], i, np.int32) for i in range(c["n"])])
    pos = np.concatenate([np.arange(c["lengths"][i], dtype=np.int32) for i in range(c["n"])])
    return leaf, pos


def test_oracle_reconstructs_every_original_token():
    c = delta.load_cfdc(GOLD)
    assert c["n"] == 12 and c["nbase"] == 600 and int(c["ostart"][-1]) == c["originals"].size
    leaf, pos = _all_queries(c)
    got = delta.fetch(c["base"], c["dpos"], c["dval"], c["dstart"], c["dlen"], leaf, pos)
    assert np.array_equal(got, c["originals"])
    # past the base and without an override: -1 (src/cuda/delta_apply.cu:18)
    far = delta.fetch(c["base"], c["dpos"], c["dval"], c["dstart"], c["dlen"], [0, 3], [c["nbase"] + 500, 10 ** 6])
    assert list(far) == [-1, -1]


def test_entry_point_rejects_null_pointers_before_cuda(native):
    lib = native.lib()
    lib.cf_delta_fetch_async.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 7 + [C.c_size_t, C.c_void_p]
    fake = 0x1000
    assert lib.cf_delta_fetch_async(None, 1, fake, fake, fake, fake, fake, fake, fake, 4, None) == 1
    assert lib.cf_delta_fetch_async(fake, 1, fake, fake, fake, fake, fake, fake, None, 4, None) == 1
    assert lib.cf_delta_fetch_async(fake, 1, None, None, fake, fake, fake, fake, fake, 0, None) == 0   # nothing to do


@pytest.mark.gpu
def test_cuda_fetch_matches_golden_and_oracle(native):
    import torch
    lib = native.lib()
    lib.cf_delta_fetch_async.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 7 + [C.c_size_t, C.c_void_p]
    c = delta.load_cfdc(GOLD)
    dev = {k: torch.from_numpy(c[k]).cuda() for k in ("base", "dpos", "dval", "dstart", "dlen")}
    leaf, pos = _all_queries(c)
    rng = np.random.default_rng(3)
    extra_leaf = rng.integers(0, c["n"], 5000).astype(np.int32)
    extra_pos = rng.integers(0, c["nbase"] + 200, 5000).astype(np.int32)   # some past every sequence's end
    leaf2, pos2 = np.concatenate([leaf, extra_leaf]), np.concatenate([pos, extra_pos])
    d_leaf, d_pos = torch.from_numpy(leaf2).cuda(), torch.from_numpy(pos2).cuda()
    out = torch.full((leaf2.size,), -7, dtype=torch.int32, device="cuda")
    rc = lib.cf_delta_fetch_async(dev["base"].data_ptr(), c["nbase"], dev["dpos"].data_ptr(), dev["dval"].data_ptr(),
                                  dev["dstart"].data_ptr(), dev["dlen"].data_ptr(), d_leaf.data_ptr(), d_pos.data_ptr(),
                                  out.data_ptr(), leaf2.size, None)
    assert rc == 0
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    assert np.array_equal(got[:leaf.size], c["originals"])
    assert np.array_equal(got[leaf.size:], delta.fetch(c["base"], c["dpos"], c["dval"], c["dstart"], c["dlen"], extra_leaf, extra_pos))
