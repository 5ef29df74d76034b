"""GPU test of the reference's device sequence resolver ABI (compat_ms.h): pages published as the reference's int4
descriptors, shared between sequences by reference, copy-on-write tails, one batched launch per layer for mixed
decode / prefill items with strided typed tensors, snapshots, removal and reclamation."""
import ctypes as C

import numpy as np
import pytest

from compat_types import MsBatchItem, MsConfig, MsCounters, MsPublication, PageDescriptor, TensorView

pytestmark = pytest.mark.gpu


def _int4_page(rng, tokens, hkv, d, block):
    """A page in the reference's device format (src/cuda/device_kv_seal_attention.cu:80-118): rows [token][kv head][dim],
    per flat block a scale absmax/7, q = rint(x/scale) clamped to [-8, 7], symbol q + 8, two nibbles per byte."""
    out = []
    for _ in range(2):
        x = rng.standard_normal(tokens * hkv * d).astype(np.float32)
        nb = (x.size + block - 1) // block
        scales = np.ones(nb, np.float32)
        sym = np.zeros(x.size, np.uint8)
        for b in range(nb):
            seg = x[b * block:(b + 1) * block]
            m = np.abs(seg).max()
            scales[b] = m / np.float32(7.0) if m > 0 else 1.0
            sym[b * block:(b + 1) * block] = (np.clip(np.rint(seg / scales[b]), -8, 7) + 8).astype(np.uint8)
        packed = (sym[0::2] & 0xF) | ((sym[1::2] & 0xF) << 4)
        deq = ((sym.astype(np.float32) - 8) * np.repeat(scales, block)[:x.size]).reshape(tokens, hkv, d)
        out.append((packed.astype(np.uint8), scales, deq))
    return out


def _expected(oracle, k, v, sealed, tile, q, positions, scale, group):
    dk, dv = k.copy(), v.copy()
    for h in range(k.shape[1]):
        for t0 in range(0, sealed, tile):
            n = min(tile, sealed - t0)
            for src, dst in ((k, dk), (v, dv)):
                rc, bits, codes = oracle.quantize_stream(np.ascontiguousarray(src[t0:t0 + n, h]))
                s = np.array([bits], np.uint16).view(np.float16)[0].astype(np.float32)
                dst[t0:t0 + n, h] = codes.reshape(n, -1).astype(np.float32) * s
    out = np.zeros(q.shape)
    for i, pos in enumerate(positions):
        for h in range(q.shape[1]):
            s = (dk[:pos + 1, h // group].astype(np.float64) @ q[i, h].astype(np.float64)) * scale
            w = np.exp(s - s.max())
            out[i, h] = (w[:, None] * dv[:pos + 1, h // group]).sum(0) / w.sum()
    return out


def test_resolver_publish_share_batch_reclaim(native, oracle):
    import torch
    lib = native.lib()
    lib.cf_ms_cuda_create.restype = C.c_void_p
    lib.cf_ms_cuda_last_error.restype = C.c_char_p
    layers, hkv, hq, d, page, block = 2, 2, 8, 64, 64, 32
    r = C.c_void_p(lib.cf_ms_cuda_create(C.byref(MsConfig(layers, hkv, hq, d, page, hq // hkv, 0))))
    rng = np.random.default_rng(21)
    A, B, Cc = C.c_int64(7), C.c_int64(8), C.c_int64(9)
    assert lib.cf_ms_cuda_sequence_create(r, A) == 0 and lib.cf_ms_cuda_sequence_create(r, Cc) == 0
    keep, history = [], {}

    def publish(seq, layer, begin, tokens):
        (kp, ks, kd), (vp, vs, vd) = _int4_page(rng, tokens, hkv, d, block)
        t = [torch.from_numpy(x).cuda() for x in (kp, vp, ks, vs)]
        keep.append(t)
        pub = MsPublication()
        pub.sequence_id, pub.layer = seq.value, layer
        pub.descriptor = PageDescriptor(t[0].data_ptr(), t[1].data_ptr(), t[2].data_ptr(), t[3].data_ptr(), begin, tokens, hkv, d,
                                        block, ks.size, kp.size, vp.size, kp.size + vp.size + 8 * ks.size, 1)
        pub.resident_bytes, pub.seal_generation = kp.size + vp.size + 8 * ks.size, 1
        rc = lib.cf_ms_cuda_publish_page_async(r, C.byref(pub), None)
        if rc == 0:
            hk, hv = history.setdefault((seq.value, layer), (np.zeros((0, hkv, d), np.float32), np.zeros((0, hkv, d), np.float32)))
            history[(seq.value, layer)] = (np.concatenate([hk, kd]), np.concatenate([hv, vd]))
        return rc

    for layer in range(layers):
        assert publish(A, layer, 0, page) == 0, lib.cf_ms_cuda_last_error(r)
        assert publish(A, layer, page, page) == 0
    assert publish(A, 0, 5, page) == -1 and b"continue" in lib.cf_ms_cuda_last_error(r)
    assert publish(Cc, 0, 0, 40) == 0                    # a short page is fine as the last one ...
    assert publish(Cc, 0, 40, page) == -1                # ... and nothing may follow it
    # B shares A's sealed pages by reference, then both get their own unsealed rows
    assert lib.cf_ms_cuda_copy_sequence_async(r, A, B, None) == 0
    tails = {}
    for seq, count in ((A, 5), (B, 11)):
        for layer in range(layers):
            tk = rng.standard_normal((count, hkv, d)).astype(np.float32)
            tv = rng.standard_normal((count, hkv, d)).astype(np.float32)
            dk, dv = torch.from_numpy(tk).cuda(), torch.from_numpy(tv).cuda()
            keep.append((dk, dv))
            assert lib.cf_ms_cuda_stage_active_async(r, seq, layer, 2 * page, C.c_void_p(dk.data_ptr()), C.c_void_p(dv.data_ptr()),
                                                     count, None) == 0, lib.cf_ms_cuda_last_error(r)
            tails[(seq.value, layer)] = (tk, tv)
    assert lib.cf_ms_cuda_audit(r) == 0
    n = MsCounters()
    lib.cf_ms_cuda_get_counters(r, C.byref(n))
    assert n.pages_registered == 5 and n.page_registration_failures == 2

    # a batch: decode items for A and B on both layers, a 3-token prefill item for B on layer 1, one item for Cc;
    # queries fp16 strided, outputs fp32 dense or fp16 strided
    scale = 1.0 / np.sqrt(d)
    spec = [(A, 0, 1, 2 * page + 5), (B, 0, 1, 2 * page + 11), (A, 1, 1, 2 * page + 5), (B, 1, 3, 2 * page + 8), (Cc, 0, 1, 40)]
    items = (MsBatchItem * len(spec))()
    checks = []
    for i, (seq, layer, nq, begin) in enumerate(spec):
        q = rng.standard_normal((nq, hq, d)).astype(np.float16)
        qd = torch.zeros((nq, hq, d + 8), dtype=torch.float16, device="cuda")
        qd[:, :, :d] = torch.from_numpy(q).cuda()
        half_out = i % 2 == 1
        od = torch.zeros((nq, hq, d + (8 if half_out else 0)), dtype=torch.float16 if half_out else torch.float32, device="cuda")
        w = 2 if half_out else 4
        keep.append((qd, od))
        items[i].sequence_id, items[i].layer = seq.value, layer
        items[i].query = TensorView(qd.data_ptr(), 1, nq, hq, d, hq * (d + 8) * 2, (d + 8) * 2, 2, 0)
        items[i].output, items[i].output_type = od.data_ptr(), 1 if half_out else 3
        items[i].output_token_stride_bytes = hq * od.shape[2] * w
        items[i].output_head_stride_bytes, items[i].output_element_stride_bytes = od.shape[2] * w, w
        items[i].query_token_begin, items[i].softmax_scale, items[i].causal_window = begin, scale, 0
        checks.append((seq.value, layer, q.astype(np.float32), [begin + j for j in range(nq)], od, half_out))
    assert lib.cf_ms_cuda_execute_batch_async(r, items, len(spec), None) == 0, lib.cf_ms_cuda_last_error(r)
    torch.cuda.synchronize()
    for seq, layer, q, pos, od, half_out in checks:
        src = 7 if seq == 8 else seq                      # B reads A's pages
        hk, hv = history[(src, layer)]
        sealed = hk.shape[0]
        if (seq, layer) in tails:
            hk = np.concatenate([hk, tails[(seq, layer)][0]])
            hv = np.concatenate([hv, tails[(seq, layer)][1]])
        want = _expected(oracle, hk, hv, sealed, 16, q, pos, scale, hq // hkv)
        got = od[:, :, :d].float().cpu().numpy()
        assert np.abs(got - want).max() <= (2e-3 if half_out else 2e-4), (seq, layer)
    lib.cf_ms_cuda_get_counters(r, C.byref(n))
    assert n.sequence_attention_launches == 2            # one launch per layer for five items
    assert n.decode_items == 4 and n.prefill_items == 1 and n.snapshots_acquired == 5 and n.in_flight_page_references == 9
    assert n.copy_on_write_tail_copies == 0

    # removal retires only what nobody shares; reclamation waits for the snapshots' events
    assert lib.cf_ms_cuda_sequence_remove_async(r, A, None) == 0
    lib.cf_ms_cuda_get_counters(r, C.byref(n))
    assert n.pages_retired == 0                          # B still references every page of A
    assert lib.cf_ms_cuda_reclaim_async(r, None) == 0
    lib.cf_ms_cuda_get_counters(r, C.byref(n))
    assert n.snapshots_released == 5 and n.in_flight_page_references == 0
    assert lib.cf_ms_cuda_cancel_sequence_async(r, B, None) == 0
    assert lib.cf_ms_cuda_execute_batch_async(r, C.byref(items[1]), 1, None) == -1      # cancelled: not dispatchable
    assert lib.cf_ms_cuda_sequence_remove_async(r, B, None) == 0
    assert lib.cf_ms_cuda_reclaim_async(r, None) == 0
    lib.cf_ms_cuda_get_counters(r, C.byref(n))
    assert n.pages_retired == 4 and n.pages_reclaimed == 4 and n.pending_reclamation_bytes == 0
    assert lib.cf_ms_cuda_audit(r) == 0 and n.dense_fallback_launches == 0
    lib.cf_ms_cuda_destroy(r, None)


def test_refused_seal_leaves_the_sequence_untouched_and_arena_slots_are_reused(native):
    """A tail with a NaN row: the seal call fails, the sequence keeps its rows and its token counts, nothing is
    published, the status bit is reported. Then churn: forty sequences are sealed, removed and reclaimed one after the
    other, and the arena does not grow past its first slots."""
    import torch
    lib = native.lib()
    lib.cf_ms_cuda_create.restype = C.c_void_p
    lib.cf_ms_cuda_last_error.restype = C.c_char_p
    hkv, hq, d, page = 2, 8, 128, 16
    r = C.c_void_p(lib.cf_ms_cuda_create(C.byref(MsConfig(1, hkv, hq, d, page, hq // hkv, 0))))
    rng = np.random.default_rng(33)

    def view(t):
        es = t.element_size()
        return TensorView(t.data_ptr(), 3, t.shape[0], t.shape[1], t.shape[2], t.stride(0) * es, t.stride(1) * es, es, 0)

    def rows(n, poison=False):
        x = rng.standard_normal((n, hkv, d)).astype(np.float32)
        if poison:
            x[3, 1, 7] = np.nan
        return torch.from_numpy(x).cuda()

    def stats():
        v = [C.c_uint64(0) for _ in range(4)]
        bits = C.c_uint32(0)
        assert lib.cf_b200_ms_arena_stats(r, *[C.byref(x) for x in v], C.byref(bits)) == 0
        return [int(x.value) for x in v] + [int(bits.value)]

    def tokens(seq):
        a, b = C.c_uint32(0), C.c_uint32(0)
        assert lib.cf_b200_ms_sequence_tokens(r, C.c_int64(seq), 0, C.byref(a), C.byref(b)) == 0
        return int(a.value), int(b.value)

    assert lib.cf_ms_cuda_sequence_create(r, C.c_int64(1)) == 0
    k, v = rows(16, poison=True), rows(16)
    assert lib.cf_b200_ms_append_active_async(r, C.c_int64(1), 0, 0, C.byref(view(k)), C.byref(view(v)), None) == 0
    n = MsCounters()
    lib.cf_ms_cuda_get_counters(r, C.byref(n))
    registered = n.pages_registered
    assert lib.cf_b200_ms_seal_active_async(r, C.c_int64(1), 0, None) == -1
    assert b"NaN" in lib.cf_ms_cuda_last_error(r)
    assert tokens(1) == (0, 16)                           # nothing sealed, the rows are still the active tail
    in_use, free, live, arena0, bits = stats()
    assert in_use == 0 and live == 0 and bits & native.DEVSTAT_NONFINITE
    lib.cf_ms_cuda_get_counters(r, C.byref(n))
    assert n.pages_registered == registered
    # the caller repairs the tail (drops it, appends clean rows) and seals
    assert lib.cf_b200_ms_truncate_async(r, C.c_int64(1), 0, None) == 0
    k = rows(16)
    assert lib.cf_b200_ms_append_active_async(r, C.c_int64(1), 0, 0, C.byref(view(k)), C.byref(view(v)), None) == 0
    assert lib.cf_b200_ms_seal_active_async(r, C.c_int64(1), 0, None) == 0, lib.cf_ms_cuda_last_error(r)
    assert tokens(1) == (16, 0)
    in_use, free, live, arena1, _ = stats()
    assert in_use == 1 and 0 < live <= hkv * (16 + 2 * 2048)
    for seq in range(100, 140):
        assert lib.cf_ms_cuda_sequence_create(r, C.c_int64(seq)) == 0
        k, v = rows(16), rows(16)
        assert lib.cf_b200_ms_append_active_async(r, C.c_int64(seq), 0, 0, C.byref(view(k)), C.byref(view(v)), None) == 0
        assert lib.cf_b200_ms_seal_active_async(r, C.c_int64(seq), 0, None) == 0
        assert lib.cf_ms_cuda_sequence_remove_async(r, C.c_int64(seq), None) == 0
        torch.cuda.synchronize()
        assert lib.cf_ms_cuda_reclaim_async(r, None) == 0
    in_use, free, live2, arena2, _ = stats()
    assert in_use == 1 and free <= 1 and arena2 == arena1 and live2 == live
    lib.cf_ms_cuda_get_counters(r, C.byref(n))
    assert n.pages_reclaimed == 40
    assert lib.cf_ms_cuda_audit(r) == 0
    lib.cf_ms_cuda_destroy(r, None)
