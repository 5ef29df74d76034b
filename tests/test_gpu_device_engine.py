"""GPU tests of the reference's device-resident ABIs served by this library (compat_device.h): the seal engine's state
machine with its ten host-side fault points, synchronous rejection of NaN pages, strided / typed queries and outputs,
and the append dataplane with fp16 / bf16 / fp32 strided views."""
import ctypes as C

import numpy as np
import pytest

from compat_types import DeviceKvConfig, DeviceKvCounters, DeviceSealConfig, DeviceSealCounters, TensorView

pytestmark = pytest.mark.gpu


def _expected(oracle, k, v, sealed, tile, q, positions, window, scale, group):
    """fp64 softmax over what the engine holds: sealed rows quantised tile by tile (int8, one fp16 scale per stream),
    unsealed rows as given. k, v: [tokens][Hkv][D]."""
    dk, dv = k.copy(), v.copy()
    for h in range(k.shape[1]):
        for t0 in range(0, sealed, tile):
            for src, dst in ((k, dk), (v, dv)):
                rc, bits, codes = oracle.quantize_stream(np.ascontiguousarray(src[t0:t0 + tile, h]))
                s = np.array([bits], np.uint16).view(np.float16)[0].astype(np.float32)
                dst[t0:t0 + tile, h] = codes.reshape(tile, -1).astype(np.float32) * s
    nq, hq, d = q.shape
    out = np.zeros((nq, hq, d))
    for i, pos in enumerate(positions):
        lo = 0 if window == 0 or pos + 1 <= window else pos + 1 - window
        for h in range(hq):
            kv = h // group
            s = (dk[lo:pos + 1, kv].astype(np.float64) @ q[i, h].astype(np.float64)) * scale
            w = np.exp(s - s.max())
            out[i, h] = (w[:, None] * dv[lo:pos + 1, kv]).sum(0) / w.sum()
    return out


def test_seal_engine_state_machine_faults_and_attention(native, oracle):
    import torch
    lib = native.lib()
    lib.cf_device_seal_create.restype = C.c_void_p
    lib.cf_device_seal_last_error.restype = C.c_char_p
    layers, hkv, hq, d, page = 2, 2, 8, 128, 64          # tiles of 16 tokens at head_dim 128: four records per page and head
    cfg = DeviceSealConfig(layers, hkv, hq, d, page, hq // hkv, 64, 0)
    e = C.c_void_p(lib.cf_device_seal_create(C.byref(cfg)))
    rng = np.random.default_rng(77)
    tokens = page * 2 + 9
    k = rng.standard_normal((tokens, hkv, d)).astype(np.float32)
    v = rng.standard_normal((tokens, hkv, d)).astype(np.float32)
    dk, dv = torch.from_numpy(k).cuda(), torch.from_numpy(v).cuda()
    state, n = C.c_uint32(0), DeviceSealCounters()

    def stage(layer, begin, count):
        return lib.cf_device_seal_stage_active_page(e, layer, begin, C.c_void_p(dk[begin:].data_ptr()),
                                                    C.c_void_p(dv[begin:].data_ptr()), count, None)

    assert stage(0, 0, 10) == 0
    lib.cf_device_seal_get_state(e, 0, C.byref(state))
    assert state.value == 0                                       # ACTIVE_FILLING
    assert lib.cf_device_seal_full_page_async(e, 0, None) == -1   # not full
    assert stage(0, 0, page) == 0
    lib.cf_device_seal_get_state(e, 0, C.byref(state))
    assert state.value == 1                                       # ACTIVE_FULL
    # every fault point aborts the seal, leaves the page staged and the generation where it was
    for fault in range(1, 11):
        if fault == 8:
            continue                                              # PAGE_TABLE_GROW is only reached when the table grows
        assert lib.cf_device_seal_set_fault(e, fault) == 0
        assert lib.cf_device_seal_full_page_async(e, 0, None) == -1, fault
        assert b"injected transactional seal failure" in lib.cf_device_seal_last_error(e)
        lib.cf_device_seal_get_state(e, 0, C.byref(state))
        assert state.value == 1
        lib.cf_device_seal_get_counters(e, C.byref(n))
        assert n.seal_successes == 0 and n.page_table_generation == 0 and n.descriptor_publications == 0
    assert n.seal_failures == 10 and n.seal_attempts == 10        # 9 injected + the "not full" attempt
    lib.cf_device_seal_set_fault(e, 0)
    assert lib.cf_device_seal_full_page_async(e, 0, None) == 0, lib.cf_device_seal_last_error(e)
    lib.cf_device_seal_get_state(e, 0, C.byref(state))
    lib.cf_device_seal_get_counters(e, C.byref(n))
    assert state.value == 0 and n.seal_successes == 1 and n.page_table_generation == 1
    assert 0 < n.payload_bytes_written < page * hkv * d * 2 * 2   # smaller than fp16
    # the successful seal and the six aborted attempts that got past quantisation (faults 4, 5, 6, 7, 9, 10), booked
    # where the reference books them (src/cuda/device_kv_seal_attention.cu:275)
    assert n.values_quantized == 7 * 2 * page * hkv * d
    assert stage(0, 5, 3) == -1                                    # must continue the sealed history
    assert stage(0, page, page) == 0 and lib.cf_device_seal_full_page_async(e, 0, None) == 0
    assert stage(0, 2 * page, 9) == 0

    # attention: fp16 strided query view, bf16 strided output
    nq, window, scale = 3, 100, 1.0 / np.sqrt(d)
    q = rng.standard_normal((nq, hq, d)).astype(np.float16)
    q_pad = torch.zeros((nq, hq, d + 8), dtype=torch.float16, device="cuda")
    q_pad[:, :, :d] = torch.from_numpy(q).cuda()
    view = TensorView(q_pad.data_ptr(), 1, nq, hq, d, hq * (d + 8) * 2, (d + 8) * 2, 2, 0)
    out = torch.zeros((nq, hq, d + 4), dtype=torch.bfloat16, device="cuda")
    pos = [tokens - nq + i for i in range(nq)]
    rc = lib.cf_device_seal_attention_async(e, 0, C.byref(view), C.c_void_p(out.data_ptr()), 2, C.c_uint64(hq * (d + 4) * 2),
                                            C.c_uint64((d + 4) * 2), C.c_uint64(2), pos[0], C.c_float(scale), window, None)
    assert rc == 0, lib.cf_device_seal_last_error(e)
    torch.cuda.synchronize()
    want = _expected(oracle, k, v, 2 * page, 16, q.astype(np.float32), pos, window, scale, hq // hkv)
    got = out[:, :, :d].float().cpu().numpy()
    assert np.abs(got - want).max() <= 2e-2                       # bf16 output: 8 mantissa bits
    # fp32 dense query and output: the tight bar
    qf = torch.from_numpy(q.astype(np.float32)).cuda()
    view = TensorView(qf.data_ptr(), 3, nq, hq, d, hq * d * 4, d * 4, 4, 0)
    outf = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda")
    assert lib.cf_device_seal_attention_async(e, 0, C.byref(view), C.c_void_p(outf.data_ptr()), 3, C.c_uint64(hq * d * 4),
                                              C.c_uint64(d * 4), C.c_uint64(4), pos[0], C.c_float(scale), window, None) == 0
    torch.cuda.synchronize()
    assert np.abs(outf.cpu().numpy() - want).max() <= 2e-4
    lib.cf_device_seal_get_counters(e, C.byref(n))
    assert n.compressed_attention_launches == 2 and n.query_conversion_launches == 1 and n.output_conversion_launches == 1
    assert n.sealed_pages_consumed == 4

    # a page with a NaN is rejected synchronously, nothing is published, the page stays staged (layer 1 untouched so far)
    bad = dk.clone()
    bad[17, 1, 5] = float("nan")
    assert lib.cf_device_seal_stage_active_page(e, 1, 0, C.c_void_p(bad.data_ptr()), C.c_void_p(dv.data_ptr()), page, None) == 0
    assert lib.cf_device_seal_full_page_async(e, 1, None) == -1
    assert b"NaN or Inf" in lib.cf_device_seal_last_error(e)
    lib.cf_device_seal_get_counters(e, C.byref(n))
    lib.cf_device_seal_get_state(e, 1, C.byref(state))
    assert n.invalid_pages_rejected == 1 and state.value == 1
    assert stage(1, 0, page) == 0 and lib.cf_device_seal_full_page_async(e, 1, None) == 0      # clean data seals fine
    assert lib.cf_device_seal_clear_async(e, None) == 0
    lib.cf_device_seal_get_state(e, 0, C.byref(state))
    assert state.value == 0
    lib.cf_device_seal_destroy(e, None)


@pytest.mark.parametrize("dtype", ["f16", "bf16", "f32"])
def test_dataplane_append_seal_attention(native, oracle, dtype):
    import torch
    lib = native.lib()
    lib.cf_device_kv_create.restype = C.c_void_p
    lib.cf_device_kv_last_error.restype = C.c_char_p
    layers, hkv, hq, d, page = 1, 2, 4, 64, 32
    p = C.c_void_p(lib.cf_device_kv_create(C.byref(DeviceKvConfig(layers, hkv, hq, d, page, hq // hkv, 0))))
    rng = np.random.default_rng(5)
    tdt = {"f16": torch.float16, "bf16": torch.bfloat16, "f32": torch.float32}[dtype]
    code = {"f16": 1, "bf16": 2, "f32": 3}[dtype]
    width = 2 if dtype != "f32" else 4
    tokens = 2 * page + 7
    # strided source: rows padded to d + 8 elements
    k_src = torch.from_numpy(rng.standard_normal((tokens, hkv, d + 8)).astype(np.float32)).cuda().to(tdt)
    v_src = torch.from_numpy(rng.standard_normal((tokens, hkv, d + 8)).astype(np.float32)).cuda().to(tdt)
    k = k_src[:, :, :d].float().cpu().numpy()
    v = v_src[:, :, :d].float().cpu().numpy()

    def view(t, begin, count):
        return TensorView(t[begin:].data_ptr(), code, count, hkv, d, hkv * (d + 8) * width, (d + 8) * width, width, 0)

    def append(begin, count):
        kv, vv = view(k_src, begin, count), view(v_src, begin, count)
        return lib.cf_device_kv_append_async(p, 0, begin, C.byref(kv), C.byref(vv), None)

    assert append(0, 20) == 0
    assert append(25, 4) == -1 and b"non-contiguous" in lib.cf_device_kv_last_error(p)
    assert append(20, 20) == -1 and b"page boundary" in lib.cf_device_kv_last_error(p)
    assert append(20, 12) == 0
    assert lib.cf_device_kv_seal_full_pages_async(p, None) == 0, lib.cf_device_kv_last_error(p)
    assert append(32, 32) == 0 and lib.cf_device_kv_seal_full_pages_async(p, None) == 0
    assert append(64, 7) == 0
    n = DeviceKvCounters()
    lib.cf_device_kv_get_counters(p, C.byref(n))
    assert n.device_append_calls == 4 and n.seal_successes == 2 and n.dense_fallback_launches == 0
    assert n.device_values_appended == 2 * tokens * hkv * d and 0 < n.compressed_bytes < 2 * page * hkv * d * 2 * 2
    assert {"f16": n.fp16_values_converted, "bf16": n.bf16_values_converted, "f32": n.fp32_values_copied}[dtype] == 2 * tokens * hkv * d
    nq, scale = 2, 1.0 / np.sqrt(d)
    q = rng.standard_normal((nq, hq, d)).astype(np.float32)
    dq = torch.from_numpy(q).cuda()
    out = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda")
    assert lib.cf_device_kv_attention_async(p, 0, C.c_void_p(dq.data_ptr()), C.c_void_p(out.data_ptr()), nq, tokens - nq,
                                            C.c_float(scale), 0, None) == 0, lib.cf_device_kv_last_error(p)
    torch.cuda.synchronize()
    want = _expected(oracle, k, v, 2 * page, 16, q, [tokens - 2, tokens - 1], 0, scale, hq // hkv)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-4
    assert lib.cf_device_kv_clear_async(p, None) == 0
    # a layer may start anywhere (src/cuda/device_kv_dataplane.cu:160-168): the same rows appended from position 1000 on
    # give the same answers at positions shifted by 1000; a gap after a seal is still refused
    def append_at(base, begin, count):
        kv, vv = view(k_src, begin, count), view(v_src, begin, count)
        return lib.cf_device_kv_append_async(p, 0, base + begin, C.byref(kv), C.byref(vv), None)
    assert append_at(1000, 0, 32) == 0 and lib.cf_device_kv_seal_full_pages_async(p, None) == 0
    assert append_at(1005, 32, 8) == -1 and b"non-contiguous" in lib.cf_device_kv_last_error(p)
    assert append_at(1000, 32, 32) == 0 and lib.cf_device_kv_seal_full_pages_async(p, None) == 0
    assert append_at(1000, 64, 7) == 0
    out2 = torch.zeros_like(out)
    assert lib.cf_device_kv_attention_async(p, 0, C.c_void_p(dq.data_ptr()), C.c_void_p(out2.data_ptr()), nq, 1000 + tokens - nq,
                                            C.c_float(scale), 0, None) == 0, lib.cf_device_kv_last_error(p)
    torch.cuda.synchronize()
    assert np.abs(out2.cpu().numpy() - want).max() <= 2e-4
    assert lib.cf_device_kv_attention_async(p, 0, C.c_void_p(dq.data_ptr()), C.c_void_p(out2.data_ptr()), nq, 10,
                                            C.c_float(scale), 0, None) == -1 and b"before" in lib.cf_device_kv_last_error(p)
    assert lib.cf_device_kv_clear_async(p, None) == 0
    assert append(0, 5) == 0                                       # usable after clear
    lib.cf_device_kv_destroy(p, None)


def test_prefill_through_the_dataplane_takes_the_shared_prefix_path(native, oracle):
    """A call with several query tokens (llama.cpp evaluating a prompt batch) over a sealed history: the engine passes
    the shared-prefix hint by itself; the answers equal the ones the same query tokens get one at a time."""
    import torch
    lib = native.lib()
    lib.cf_device_kv_create.restype = C.c_void_p
    lib.cf_device_kv_last_error.restype = C.c_char_p
    lib.cf_b200_shared_prefix_launches.restype = C.c_uint64
    layers, hkv, hq, d, page = 1, 2, 8, 128, 64
    p = C.c_void_p(lib.cf_device_kv_create(C.byref(DeviceKvConfig(layers, hkv, hq, d, page, hq // hkv, 0))))
    rng = np.random.default_rng(15)
    tokens = 4 * page + 9                                      # 16 sealed records of 16 tokens + a 9-token tail
    k = torch.from_numpy(rng.standard_normal((tokens, hkv, d)).astype(np.float32)).cuda()
    v = torch.from_numpy(rng.standard_normal((tokens, hkv, d)).astype(np.float32)).cuda()
    view = lambda t, begin, count: TensorView(t[begin:].data_ptr(), 3, count, hkv, d, hkv * d * 4, d * 4, 4, 0)
    for begin in range(0, tokens, page):
        count = min(page, tokens - begin)
        kv, vv = view(k, begin, count), view(v, begin, count)
        assert lib.cf_device_kv_append_async(p, 0, begin, C.byref(kv), C.byref(vv), None) == 0, lib.cf_device_kv_last_error(p)
        if count == page:
            assert lib.cf_device_kv_seal_full_pages_async(p, None) == 0
    nq, scale = 6, C.c_float(1.0 / np.sqrt(d))
    q = torch.from_numpy(rng.standard_normal((nq, hq, d)).astype(np.float32)).cuda()
    out = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda")
    before = lib.cf_b200_shared_prefix_launches()
    assert lib.cf_device_kv_attention_async(p, 0, C.c_void_p(q.data_ptr()), C.c_void_p(out.data_ptr()), nq, tokens - nq, scale, 0, None) == 0
    torch.cuda.synchronize()
    assert lib.cf_b200_shared_prefix_launches() == before + 1
    single = torch.zeros((nq, hq, d), dtype=torch.float32, device="cuda")
    for i in range(nq):
        assert lib.cf_device_kv_attention_async(p, 0, C.c_void_p(q[i:].data_ptr()), C.c_void_p(single[i:].data_ptr()), 1,
                                                tokens - nq + i, scale, 0, None) == 0
    torch.cuda.synchronize()
    assert lib.cf_b200_shared_prefix_launches() == before + 1
    assert float((out - single).abs().max()) <= 2e-5 and float(out.abs().max()) > 0
    want = _expected(oracle, k.cpu().numpy(), v.cpu().numpy(), 4 * page, 16, q.cpu().numpy(),
                     [tokens - nq + i for i in range(nq)], 0, 1.0 / np.sqrt(d), hq // hkv)
    assert np.abs(out.cpu().numpy() - want).max() <= 2e-4
    # a sliding window turns the hint off (the shared-prefix kernel serves whole histories only)
    assert lib.cf_device_kv_attention_async(p, 0, C.c_void_p(q.data_ptr()), C.c_void_p(out.data_ptr()), nq, tokens - nq, scale, 100, None) == 0
    assert lib.cf_b200_shared_prefix_launches() == before + 1
    lib.cf_device_kv_destroy(p, None)
