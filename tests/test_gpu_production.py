"""GPU test of the reference's batched decode runtime ABI (compat_production.h): items over int4 page descriptors and
fp32 tails, checked against fp64 softmax attention on the dequantised rows."""
import ctypes as C

import numpy as np
import pytest

from compat_types import AttentionBatchItem, AttentionCounters, AttentionRuntimeConfig, PageDescriptor, TensorView

pytestmark = pytest.mark.gpu

HQ, HKV, D, BLOCK, PAGE = 8, 2, 64, 32, 16


def _int4_page(rng, tokens, token_begin, keep):
    """One page the way the reference's seal engine writes it (src/cuda/device_kv_seal_attention.cu:80-134): one
    fp32 scale per `BLOCK` values = absmax / 7, nibble = clamp(round(x / scale), -7, 7) + 8, low nibble first."""
    import torch
    desc, dense = PageDescriptor(), []
    for name in ("key", "value"):
        x = rng.standard_normal((tokens, HKV, D)).astype(np.float32)
        blocks = x.reshape(-1, BLOCK)
        scale = (np.abs(blocks).max(axis=1) / 7.0).astype(np.float32)
        q = np.clip(np.rint(blocks / scale[:, None]), -7, 7).astype(np.int32)
        dense.append((q.astype(np.float32) * scale[:, None]).reshape(tokens, HKV, D))
        nib = (q + 8).astype(np.uint8).reshape(-1)
        payload = (nib[0::2] | (nib[1::2] << 4)).astype(np.uint8)
        p, s = torch.from_numpy(payload).cuda(), torch.from_numpy(scale).cuda()
        keep += [p, s]
        setattr(desc, name + "_payload", p.data_ptr())
        setattr(desc, name + "_scales", s.data_ptr())
        setattr(desc, name + "_payload_bytes", payload.size)
    desc.token_begin, desc.token_count, desc.kv_head_count, desc.head_dim = token_begin, tokens, HKV, D
    desc.block_size, desc.blocks_per_page = BLOCK, tokens * HKV * D // BLOCK
    return desc, dense[0], dense[1]


def _expect(k, v, q, qpos, window, scale):
    """k, v [tokens][HKV][D] from token 0; q [HQ][D] -> [HQ][D] in fp64."""
    first = 0 if window == 0 else max(0, qpos + 1 - window)
    out = np.zeros((HQ, D))
    for h in range(HQ):
        kv = h // (HQ // HKV)
        s = (k[first:qpos + 1, kv].astype(np.float64) @ q[h].astype(np.float64)) * scale
        w = np.exp(s - s.max())
        out[h] = (w[:, None] * v[first:qpos + 1, kv]).sum(0) / w.sum()
    return out


@pytest.mark.parametrize("mode", [1, 0], ids=["optimized", "reference"])
def test_batched_items_over_int4_descriptors(native, mode):
    import torch
    lib = native.lib()
    lib.cf_attention_runtime_create.restype = C.c_void_p
    lib.cf_attention_last_error.restype = C.c_char_p
    rng = np.random.default_rng(31 + mode)
    cfg = AttentionRuntimeConfig()
    cfg.layer_count, cfg.query_head_count, cfg.kv_head_count, cfg.head_dim = 2, HQ, HKV, D
    cfg.page_size, cfg.block_size, cfg.gqa_group_size, cfg.mode = PAGE, BLOCK, HQ // HKV, mode
    rt = C.c_void_p(lib.cf_attention_runtime_create(C.byref(cfg)))
    keep, items, expected, outputs = [], (AttentionBatchItem * 3)(), [], []
    # (pages, tail tokens, window, query dtype, output dtype)
    cases = [(5, 7, 0, torch.float32, torch.float32), (3, 0, 40, torch.float16, torch.float16), (0, 9, 0, torch.bfloat16, torch.float32)]
    scale = 1.0 / np.sqrt(D)
    for i, (pages, tail, window, qdt, odt) in enumerate(cases):
        descs = (PageDescriptor * max(pages, 1))()
        ks, vs = [], []
        for pg in range(pages):
            descs[pg], k, v = _int4_page(rng, PAGE, pg * PAGE, keep)
            ks.append(k)
            vs.append(v)
        tk = rng.standard_normal((tail, HKV, D)).astype(np.float32)
        tv = rng.standard_normal((tail, HKV, D)).astype(np.float32)
        ks.append(tk)
        vs.append(tv)
        k_all, v_all = np.concatenate(ks), np.concatenate(vs)
        qpos = pages * PAGE + tail - 1
        q = torch.from_numpy(rng.standard_normal((HQ, D)).astype(np.float32)).to(qdt).cuda()
        out = torch.zeros((HQ, D), dtype=odt, device="cuda")
        d_desc = torch.from_numpy(np.frombuffer(bytes(descs), dtype=np.uint8).copy()).cuda()
        d_tk, d_tv = torch.from_numpy(tk).cuda(), torch.from_numpy(tv).cuda()
        keep += [q, out, d_desc, d_tk, d_tv]
        it = items[i]
        it.sequence_id, it.layer = 100 + i, i % 2
        esz = q.element_size()
        it.query = TensorView(q.data_ptr(), {torch.float16: 1, torch.bfloat16: 2, torch.float32: 3}[qdt], 1, HQ, D,
                              HQ * D * esz, D * esz, esz, 0)
        it.output, it.output_type = out.data_ptr(), {torch.float16: 1, torch.float32: 3}[odt]
        osz = out.element_size()
        it.output_token_stride_bytes, it.output_head_stride_bytes, it.output_element_stride_bytes = HQ * D * osz, D * osz, osz
        it.query_token_begin, it.softmax_scale, it.causal_window = qpos, scale, window
        it.sealed_pages, it.sealed_page_count = (d_desc.data_ptr() if pages else None), pages
        it.active_keys, it.active_values = (d_tk.data_ptr() if tail else None), (d_tv.data_ptr() if tail else None)
        it.active_token_begin, it.active_token_count = pages * PAGE, tail
        expected.append(_expect(k_all, v_all, q.float().cpu().numpy(), qpos, window, scale))
        outputs.append(out)
    assert lib.cf_attention_execute_async(rt, items, 3, None) == 0, lib.cf_attention_last_error(rt)
    torch.cuda.synchronize()
    for out, exp in zip(outputs, expected):
        tol = 2e-3 if out.dtype == torch.float16 else 2e-5
        assert np.allclose(out.float().cpu().numpy(), exp, rtol=2e-3, atol=tol)
    assert lib.cf_attention_compare_async(rt, items, 3, C.c_float(1e-4), C.c_float(1e-5), None) == 0, lib.cf_attention_last_error(rt)
    assert lib.cf_attention_compare_async(rt, items, 3, C.c_float(1e-12), C.c_float(1e-12), None) in (0, -1)
    counters = AttentionCounters()
    assert lib.cf_attention_get_counters(rt, C.byref(counters)) == 0
    assert counters.decode_launches == 1 and counters.grouped_batches == 1 and counters.grouped_items == 3
    assert counters.kernel_launches_avoided == 2 and counters.descriptor_bytes_read == 8 * 88
    assert (counters.optimized_launches if mode == 1 else counters.reference_launches) >= 2
    assert counters.pool_misses >= 1 and counters.pool_hits >= 1 and counters.cuda_errors == 0
    # K + V nibbles of the pages inside each item's window, every kv head: item 0 all 5 pages, item 1 its 3 pages
    assert counters.compressed_payload_bytes_read >= (5 + 3) * PAGE * HKV * D
    # two items for the same (sequence, layer) are refused
    items[1].sequence_id, items[1].layer = items[0].sequence_id, items[0].layer
    assert lib.cf_attention_execute_async(rt, items, 3, None) == -1
    assert b"same sequence" in lib.cf_attention_last_error(rt)
    lib.cf_attention_runtime_destroy(rt, None)
