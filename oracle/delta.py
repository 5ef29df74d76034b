"""CPU oracle (test infrastructure, never on the product path) for the reference/delta cluster fetch.

load_cfdc reads the reference's frozen cluster file (layout of tools/export_delta.py:13-17); fetch restates
cf_delta_fetch_kernel (src/cuda/delta_apply.cu:12-28): base[pos], or -1 past the base, overridden by the leaf's
delta at pos when a binary search over its sorted positions finds one. Pinned by tests/golden/delta_cluster.cfdc,
which the reference's own exporter wrote together with the original sequences the fetch must reproduce."""
import struct

import numpy as np


def load_cfdc(path):
    with open(path, "rb") as f:
        raw = f.read()
    assert raw[:4] == b"CFDC"
    version, n, nbase, ndelta, vocab, total = struct.unpack_from("<IIIIIQ", raw, 4)
    assert version == 1
    off = 4 + struct.calcsize("<IIIIIQ")
    out = {"n": n, "nbase": nbase, "vocab": vocab}
    for name, count in (("base", nbase), ("lengths", n), ("dstart", n), ("dlen", n), ("dpos", ndelta), ("dval", ndelta),
                        ("ostart", n + 1), ("originals", total)):
        out[name] = np.frombuffer(raw, dtype="<i4", count=count, offset=off).copy()
        off += 4 * count
    assert off == len(raw)
    return out


def fetch(base, dpos, dval, dstart, dlen, leaf, pos):
    leaf, pos = np.asarray(leaf), np.asarray(pos)
    out = np.empty(leaf.shape, np.int32)
    for i in range(leaf.size):
        p, first, n = int(pos[i]), int(dstart[leaf[i]]), int(dlen[leaf[i]])
        res = int(base[p]) if 0 <= p < len(base) else -1
        lo, hi = 0, n
        while lo < hi:
            mid = (lo + hi) >> 1
            if dpos[first + mid] < p:
                lo = mid + 1
            else:
                hi = mid
        if lo < n and dpos[first + lo] == p:
            res = int(dval[first + lo])
        out[i] = res
    return out
