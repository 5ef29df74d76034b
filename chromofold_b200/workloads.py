"""Seeded synthetic workloads with the shapes, sizes and value distributions of the benchmark configurations.

No dataset is involved: codes are drawn on the GPU, turned into binary16 K/V values with a per-(page, kv head)
scale and sealed by the library's GPU sealer — the same append -> seal path a server takes.
"""
import numpy as np
import torch

from . import _native as N
from .cache import SealedKvLayer, swizzle_dense_tiles

CODERS = {"fixed8": N.CODER_FIXED8, "huffman": N.CODER_HUFFMAN, "rans": N.CODER_RANS,
          "rans4": N.CODER_RANS_SPLIT4, "huffman4": N.CODER_HUFFMAN_SPLIT4}   # the last two: nibble-split (sealed_page_format.h)


def uniform_contexts(batch, lo, hi, page_tokens, seed):
    """Context lengths uniform in [lo, hi], rounded down to whole pages (sealed pages only)."""
    rng = np.random.default_rng(seed)
    return (rng.integers(lo, hi + 1, batch) // page_tokens * page_tokens).astype(np.int64)


def laplace_codes(shape, b, gen, device):
    """Discretised Laplace(b) clipped to int8, drawn on the device (inverse CDF of a uniform)."""
    u = torch.rand(shape, generator=gen, device=device, dtype=torch.float32) - 0.5
    x = -b * torch.sign(u) * torch.log1p(-2.0 * u.abs().clamp(max=0.4999999))
    return torch.round(x).clamp_(-128, 127)


def geometric_codes(shape, p, gen, device):
    """Two-sided geometric P(k) ~ (1-p)^|k| clipped to int8."""
    u = torch.rand(shape, generator=gen, device=device, dtype=torch.float32).clamp_(min=1e-12)
    mag = torch.floor(torch.log(u) / np.log1p(-p))
    sign = torch.randint(0, 2, shape, generator=gen, device=device, dtype=torch.float32) * 2 - 1
    return (mag * sign).clamp_(-128, 127)


def tiles_from_codes(codes, lo, hi, gen):
    """codes float [n, hkv, T, D] -> binary16 values whose per-stream absmax quantisation returns the codes.
    One element per stream is pinned to +127 so that absmax/127 equals the drawn scale (U[lo, hi])."""
    n, hkv = codes.shape[:2]
    codes[:, :, 0, 0] = 127.0
    scale = (torch.rand((n, hkv, 1, 1), generator=gen, device=codes.device) * (hi - lo) + lo).half().float()
    return (codes * scale).half()


def entropy_bits(hist):
    hist = np.asarray(hist, np.float64)
    p = hist[hist > 0] / hist.sum()
    return float(-(p * np.log2(p)).sum())


def build_sealed_layer(contexts, *, query_heads=32, kv_heads=8, head_dim=128, page_tokens=16, block_size=64,
                       coder="rans", dist=("laplace", 12.0), seed=4, device="cuda:0", tiles_per_launch=2048,
                       extra_pages_per_sequence=2, keep_dense=False, reserve_pages=0):
    """Seal `contexts[i]` tokens for slot i. Returns (layer, info). With keep_dense=True the binary16 tiles are also
    kept as an uncompressed pool [page_id][kv_heads][page_tokens][head_dim] for the comparison kernel.
    `reserve_pages` more pages (directory entries and arena room) are set aside for pages sealed later."""
    with torch.cuda.device(device):   # the library launches on the current device
        return _build_sealed_layer(contexts, query_heads, kv_heads, head_dim, page_tokens, block_size, coder, dist, seed, device,
                                   tiles_per_launch, extra_pages_per_sequence, keep_dense, reserve_pages)


def _build_sealed_layer(contexts, query_heads, kv_heads, head_dim, page_tokens, block_size, coder, dist, seed, device,
                        tiles_per_launch, extra_pages_per_sequence, keep_dense, reserve_pages):
    contexts = np.asarray(contexts, np.int64)
    assert np.all(contexts % page_tokens == 0)
    pages = contexts // page_tokens
    total = int(pages.sum())
    stride = int(pages.max()) + extra_pages_per_sequence
    max_record = 16 + 2 * ((head_dim * page_tokens + 15) // 16 * 16)
    layer = SealedKvLayer(kv_heads=kv_heads, query_heads=query_heads, head_dim=head_dim, page_tokens=page_tokens,
                          block_size=block_size, coder=CODERS[coder], max_sequences=len(contexts),
                          max_pages_per_sequence=stride, max_pages=total + 2 + 2 * len(contexts) + reserve_pages,
                          arena_bytes=(total + 2 * len(contexts) + reserve_pages) * kv_heads * max_record + 4096, device=device)
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    draw = (lambda shape: laplace_codes(shape, dist[1], gen, device)) if dist[0] == "laplace" else (
        lambda shape: geometric_codes(shape, dist[1], gen, device))
    # jobs in page-major order so that a sequence's pages are appended in order
    job_slots = np.concatenate([np.nonzero(pages > p)[0] for p in range(int(pages.max()))]) if total else np.zeros(0, np.int64)
    dense_k = dense_v = None
    if keep_dense:
        dense_k = torch.zeros((layer.max_pages, kv_heads, page_tokens, head_dim), dtype=torch.float16, device=device)
        dense_v = torch.zeros_like(dense_k)
    hist_k = hist_v = None
    for begin in range(0, total, tiles_per_launch):
        slots = job_slots[begin:begin + tiles_per_launch]
        shape = (len(slots), kv_heads, page_tokens, head_dim)
        k_tiles = tiles_from_codes(draw(shape), 0.005, 0.02, gen)
        v_tiles = tiles_from_codes(draw(shape), 0.005, 0.02, gen)
        if hist_k is None:  # calibrate the shared codebooks on the first launch's tiles
            hk = torch.zeros(256, dtype=torch.int64, device=device)
            hv = torch.zeros_like(hk)
            d = layer._seal_desc(torch.arange(len(slots), dtype=torch.int32, device=device), None, None)
            d.tail_k, d.tail_v = k_tiles.data_ptr(), v_tiles.data_ptr()
            import ctypes as C
            N.check("histogram", layer.lib.cf_b200_histogram_async(C.byref(d), C.c_void_p(hk.data_ptr()),
                                                                    C.c_void_p(hv.data_ptr()),
                                                                    C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            hist_k, hist_v = hk.cpu().numpy().astype(np.uint64), hv.cpu().numpy().astype(np.uint64)
            layer.set_codebooks(hist_k, hist_v)
            if CODERS[coder] in (N.CODER_RANS_SPLIT4, N.CODER_HUFFMAN_SPLIT4):
                # the codebooks were built over pair symbols; the entropy reported per code is that of the plain symbols
                hk.zero_()
                hv.zero_()
                d.coder = N.CODER_RANS
                N.check("histogram", layer.lib.cf_b200_histogram_async(C.byref(d), C.c_void_p(hk.data_ptr()),
                                                                        C.c_void_p(hv.data_ptr()),
                                                                        C.c_void_p(torch.cuda.current_stream().cuda_stream)))
                hist_k, hist_v = hk.cpu().numpy().astype(np.uint64), hv.cpu().numpy().astype(np.uint64)
        first_id = layer.next_page_id
        layer.seal_tiles(slots, k_tiles, v_tiles)
        if keep_dense:
            dense_k[first_id:first_id + len(slots)] = swizzle_dense_tiles(k_tiles)
            dense_v[first_id:first_id + len(slots)] = swizzle_dense_tiles(v_tiles)
        torch.cuda.synchronize()
    status = layer.device_status()
    if status:
        raise RuntimeError(f"sealing raised device status {status:#x}")
    sealed_bytes = layer.sealed_bytes()
    tokens = int(contexts.sum())
    info = {
        "seq_tokens": tokens,
        "pages": total,
        "sealed_bytes": sealed_bytes,
        "bytes_per_seq_token": sealed_bytes / max(tokens, 1),
        "fp16_bytes_per_seq_token": 2 * 2 * kv_heads * head_dim,
        "h0_bits_k": entropy_bits(hist_k) if hist_k is not None else None,
        "h0_bits_v": entropy_bits(hist_v) if hist_v is not None else None,
        "dense_k": dense_k, "dense_v": dense_v,
    }
    return layer, info
