"""Transfer images of sealed pages (page_transfer.h): host checksum definition, and on the GPU a pack -> image ->
unpack round trip into another store with bit-identical attention, plus rejection of a tampered record."""
import ctypes as C

import numpy as np
import pytest


def _fnv(data, h=1469598103934665603):
    for b in data:
        h = ((h ^ b) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


def test_checksums_on_the_host_follow_their_definition(native):
    lib = native.lib()
    lib.cf_b200_fnv1a.restype = C.c_uint64
    lib.cf_b200_record_checksum.restype = C.c_uint64
    assert lib.cf_b200_fnv1a(b"", C.c_uint64(0)) == 1469598103934665603
    # the reference's basis (src/persistent_page_store.cpp:14), which is not the standard FNV-1a 64 one
    assert lib.cf_b200_fnv1a(b"a", C.c_uint64(1)) == _fnv(b"a") != 0xaf63dc4c8601ec8c
    assert lib.cf_b200_fnv1a(b"sealed pages", C.c_uint64(12)) == _fnv(b"sealed pages")
    rng = np.random.default_rng(5)
    for units in (1, 31, 32, 33, 257):
        rec = rng.integers(0, 256, 16 * units, dtype=np.uint8).tobytes()
        lanes = b"".join(_fnv(b"".join(rec[16 * u:16 * u + 16] for u in range(l, units, 32))).to_bytes(8, "little") for l in range(32))
        assert lib.cf_b200_record_checksum(rec, C.c_uint64(len(rec))) == _fnv(lanes)
    assert lib.cf_b200_pages_pack_async(None, None, 8, None, 1, None, None, C.c_uint64(0), None, None, None) == 1


@pytest.mark.gpu
def test_pages_travel_between_stores_and_tampering_is_caught(native, oracle):
    import torch
    from chromofold_b200.workloads import build_sealed_layer
    src, info = build_sealed_layer(np.array([1024, 48]), coder="rans", seed=95)
    image = src.export_pages(0)
    assert src.device_status() == 0
    header = native.TransferHeader.from_buffer_copy(image[:64])
    assert header.page_count == 64 and header.payload_bytes % 16 == 0
    assert len(image) == 64 + 16 * 64 * 8 + header.payload_bytes + 4 * 64
    # every manifest checksum equals the host definition applied to the record bytes
    lib = native.lib()
    lib.cf_b200_record_checksum.restype = C.c_uint64
    man = np.frombuffer(image[64:64 + 16 * 64 * 8], dtype=[("off", "<u4"), ("len", "<u4"), ("sum", "<u8")])
    body = image[64 + man.nbytes:64 + man.nbytes + header.payload_bytes]
    for e in man[:40]:
        rec = body[16 * int(e["off"]):16 * (int(e["off"]) + int(e["len"]))]
        assert lib.cf_b200_record_checksum(rec, C.c_uint64(len(rec))) == int(e["sum"])
    assert int(man["len"].sum()) * 16 == header.payload_bytes

    # a second store with the same codebooks (same histogram -> same tables)
    dst, _ = build_sealed_layer(np.array([0, 32]), coder="rans", seed=96, extra_pages_per_sequence=70, reserve_pages=80)
    dst.k_tables.copy_(src.k_tables)
    dst.v_tables.copy_(src.v_tables)
    dst.codebook_id = src.codebook_id
    assert dst.import_pages(0, image) == 64 and dst.device_status() == 0
    g = torch.Generator(device="cuda")
    g.manual_seed(97)
    q = torch.randn((1, 32, 128), generator=g, device="cuda").half()
    a = src.attention(q, slots=[0]).cpu().numpy()
    b = dst.attention(q, slots=[0]).cpu().numpy()
    assert np.array_equal(a, b)                                            # the same records, the same arithmetic
    assert int(dst.h_sealed[0]) == 1024

    # one flipped payload bit: that record is refused, the status word says so
    bad = bytearray(image)
    bad[64 + man.nbytes + 16 * int(man[5]["off"]) + 40] ^= 0x10
    dst2, _ = build_sealed_layer(np.array([0, 32]), coder="rans", seed=96, extra_pages_per_sequence=70, reserve_pages=80)
    dst2.k_tables.copy_(src.k_tables)
    dst2.v_tables.copy_(src.v_tables)
    dst2.import_pages(0, bytes(bad))
    assert dst2.device_status() & native.DEVSTAT_CHECKSUM
    # a damaged manifest or a wrong geometry never reaches the GPU
    bad = bytearray(image)
    bad[64 + 3] ^= 1
    with pytest.raises(ValueError):
        dst2.import_pages(1, bytes(bad))
    other, _ = build_sealed_layer(np.array([16]), kv_heads=4, query_heads=16, coder="rans", seed=98, extra_pages_per_sequence=70, reserve_pages=80)
    with pytest.raises(ValueError):
        other.import_pages(0, image)
