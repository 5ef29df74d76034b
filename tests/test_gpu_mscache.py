"""GPU test of the multi-sequence cache and llama-server runtime ABIs (compat_mscache.h): appended rows are sealed on
the GPU page by page, sequences share sealed pages after a copy, speculation rolls back, batches attend."""
import ctypes as C

import numpy as np
import pytest

from compat_types import (LlamaServerBatch, LlamaServerConfig, MsBatchItem, MultisequenceConfig, MultisequenceCounters,
                          TensorView)
from test_gpu_ms_resolver import _expected

pytestmark = pytest.mark.gpu

LAYERS, HKV, HQ, D, PAGE = 2, 2, 8, 128, 16


def _view(t, tokens):
    """A [tokens][HKV][D] view of a torch tensor (any scalar type, any strides)."""
    import torch
    code = {torch.float16: 1, torch.bfloat16: 2, torch.float32: 3}[t.dtype]
    es = t.element_size()
    return TensorView(t.data_ptr(), code, tokens, t.shape[1], t.shape[2], t.stride(0) * es, t.stride(1) * es, t.stride(2) * es, 0)


def _item(seq, layer, q, out, position):
    import torch
    it = MsBatchItem()
    it.sequence_id, it.layer = seq, layer
    it.query = _view(q, q.shape[0])
    it.output, it.output_type = out.data_ptr(), {torch.float16: 1, torch.float32: 3}[out.dtype]
    es = out.element_size()
    it.output_token_stride_bytes, it.output_head_stride_bytes, it.output_element_stride_bytes = out.stride(0) * es, out.stride(1) * es, es
    it.query_token_begin, it.softmax_scale, it.causal_window = position, 1.0 / np.sqrt(D), 0
    return it


def test_cache_appends_seal_share_speculate_and_attend(native, oracle):
    import torch
    lib = native.lib()
    lib.cf_multisequence_create.restype = C.c_void_p
    lib.cf_multisequence_last_error.restype = C.c_char_p
    lib.cf_sequence_speculation_begin.restype = C.c_uint64
    c = C.c_void_p(lib.cf_multisequence_create(C.byref(MultisequenceConfig(LAYERS, HKV, HQ, D, PAGE, HQ // HKV, 0, 1))))
    err = lambda: lib.cf_multisequence_last_error(c)
    i64 = C.c_int64
    rng = np.random.default_rng(90)
    assert lib.cf_sequence_create(c, i64(5)) == 0
    hist = {}   # (sequence, layer) -> [K rows, V rows] as fp32 numpy

    def append(seq, layer, tokens, dtype):
        k = torch.from_numpy(rng.standard_normal((tokens, HKV, D)).astype(np.float32) * 0.8).to(dtype).cuda()
        v = torch.from_numpy(rng.standard_normal((tokens, HKV, D)).astype(np.float32) * 0.8).to(dtype).cuda()
        begin = hist[(seq, layer)][0].shape[0] if (seq, layer) in hist else 0
        rc = lib.cf_sequence_append_async(c, i64(seq), layer, begin, C.byref(_view(k, tokens)), C.byref(_view(v, tokens)), None)
        if rc == 0:
            old = hist.get((seq, layer), [np.zeros((0, HKV, D), np.float32)] * 2)
            hist[(seq, layer)] = [np.concatenate([old[0], k.float().cpu().numpy()]), np.concatenate([old[1], v.float().cpu().numpy()])]
        return rc

    # 37 tokens per layer, in pieces that respect the page boundary: two sealed pages + 5 active rows
    for layer in range(LAYERS):
        for tokens, dtype in ((16, torch.float16), (9, torch.float32), (7, torch.bfloat16), (5, torch.float16)):
            assert append(5, layer, tokens, dtype) == 0, err()
    assert append(5, 0, 12, torch.float16) == -1 and b"boundary" in err()          # 5 + 12 > 16
    k_bad = torch.zeros((1, HKV, D), dtype=torch.float16, device="cuda")
    assert lib.cf_sequence_append_async(c, i64(5), 0, 99, C.byref(_view(k_bad, 1)), C.byref(_view(k_bad, 1)), None) == -1
    assert b"non-contiguous" in err()

    def attend(seq_layers, positions=None):
        qs, outs, items = [], [], (MsBatchItem * len(seq_layers))()
        for i, (seq, layer) in enumerate(seq_layers):
            q = torch.from_numpy(rng.standard_normal((1, HQ, D)).astype(np.float32)).cuda()
            out = torch.zeros((1, HQ, D), dtype=torch.float32, device="cuda")
            pos = hist[(seq, layer)][0].shape[0] - 1 if positions is None else positions[i]
            items[i] = _item(seq, layer, q, out, pos)
            qs.append(q)
            outs.append(out)
        assert lib.cf_multisequence_attention_async(c, items, len(seq_layers), None) == 0, err()
        torch.cuda.synchronize()
        for (seq, layer), q, out in zip(seq_layers, qs, outs):
            k, v = hist[(seq, layer)]
            sealed = k.shape[0] // PAGE * PAGE
            want = _expected(oracle, k, v, sealed, 16, q.cpu().numpy(), [k.shape[0] - 1], 1.0 / np.sqrt(D), HQ // HKV)
            assert np.allclose(out.cpu().numpy(), want, rtol=2e-3, atol=1e-3), (seq, layer)

    attend([(5, 0), (5, 1)])

    # copy shares the two sealed pages of each layer and copies the tails; the copy then diverges
    assert lib.cf_sequence_copy_async(c, i64(5), i64(6), 0, 1 << 30, None) == 0, err()
    for layer in range(LAYERS):
        hist[(6, layer)] = [a.copy() for a in hist[(5, layer)]]
    k = MultisequenceCounters()
    lib.cf_multisequence_get_counters(c, C.byref(k))
    assert k.shared_pages == 2 * LAYERS and k.shared_page_references == 4 * LAYERS and k.sequences_copied == 1
    assert append(6, 0, 11, torch.float32) == 0, err()                              # fills and seals page 3 of the copy only
    attend([(5, 0), (6, 0), (6, 1)])
    # a copy cut at a page boundary keeps whole pages; a cut inside a page is refused
    assert lib.cf_sequence_copy_async(c, i64(5), i64(7), 0, 32, None) == 0, err()
    for layer in range(LAYERS):
        hist[(7, layer)] = [a[:32].copy() for a in hist[(5, layer)]]
    attend([(7, 1)])
    # a range that cuts a page keeps the pages wholly inside it, nothing else (src/multisequence_cache.cpp:257-258)
    assert lib.cf_sequence_copy_async(c, i64(5), i64(8), 0, 20, None) == 0, err()
    for layer in range(LAYERS):
        hist[(8, layer)] = [a[:16].copy() for a in hist[(5, layer)]]
    attend([(8, 0)])
    # a range that starts later: page 1 and the five active rows, at their old positions 16..36
    assert lib.cf_sequence_copy_async(c, i64(5), i64(9), 10, 1 << 30, None) == 0, err()
    for layer in range(LAYERS):
        hist[(9, layer)] = [a[16:].copy() for a in hist[(5, layer)]]
    attend([(9, 0), (9, 1)], positions=[36, 36])
    bad_q = torch.zeros((1, HQ, D), dtype=torch.float32, device="cuda")
    early = (MsBatchItem * 1)(_item(9, 0, bad_q, bad_q.clone(), 12))
    assert lib.cf_multisequence_attention_async(c, early, 1, None) == -1 and b"before" in err()
    assert append(9, 0, 2, torch.float16) == -1              # hist-based begin 21 is not the logical 37
    # context shift: the whole sequence moves (only its offset changes), part of it cannot, a cut through a page is an error
    assert lib.cf_sequence_shift_async(c, i64(9), 0, 1 << 30, -16, None) == 0, err()
    attend([(9, 0), (9, 1)], positions=[20, 20])
    assert lib.cf_sequence_shift_async(c, i64(9), 0, 1 << 30, -1, None) == -1 and b"negative" in err()
    assert lib.cf_sequence_shift_async(c, i64(5), 16, 1 << 30, -8, None) == -1 and b"gap" in err()
    assert lib.cf_sequence_shift_async(c, i64(5), 8, 24, 0, None) == -1 and b"align" in err()
    assert lib.cf_sequence_shift_async(c, i64(5), 16, 32, 0, None) == 0 and lib.cf_sequence_shift_async(c, i64(5), 500, 600, 7, None) == 0
    assert append(9, 0, 2, torch.float16) == 0, err()         # after the shift the next position is 21 = its row count
    attend([(9, 0)], positions=[22])

    # speculation: three provisional tokens, one accepted; then a rollback of two more
    spec = lib.cf_sequence_speculation_begin(c, i64(5))
    base = {layer: [a.copy() for a in hist[(5, layer)]] for layer in range(LAYERS)}
    for layer in range(LAYERS):
        assert append(5, layer, 3, torch.float16) == 0, err()
    assert lib.cf_sequence_speculation_commit(c, i64(5), C.c_uint64(spec), 4, None) == -1
    assert lib.cf_sequence_speculation_commit(c, i64(5), C.c_uint64(spec), 1, None) == 0, err()
    for layer in range(LAYERS):
        hist[(5, layer)] = [a[:base[layer][0].shape[0] + 1] for a in hist[(5, layer)]]
    attend([(5, 0), (5, 1)])
    spec = lib.cf_sequence_speculation_begin(c, i64(5))
    keep = {layer: [a.copy() for a in hist[(5, layer)]] for layer in range(LAYERS)}
    for layer in range(LAYERS):
        assert append(5, layer, 2, torch.float16) == 0, err()
    assert lib.cf_sequence_speculation_rollback(c, i64(5), C.c_uint64(spec), None) == 0, err()
    for layer in range(LAYERS):
        hist[(5, layer)] = keep[layer]
    attend([(5, 0), (5, 1), (6, 0)])

    # suffix removal at a page boundary; removal inside a page is refused; whole removal and reclamation
    assert lib.cf_sequence_remove_async(c, i64(6), i64(20), i64(1 << 40), None) == -1 and b"immutable page" in err()
    assert lib.cf_sequence_remove_async(c, i64(6), i64(32), i64(1 << 40), None) == 0, err()
    for layer in range(LAYERS):
        hist[(6, layer)] = [a[:32] for a in hist[(6, layer)]]
    attend([(6, 0), (6, 1)])
    assert lib.cf_sequence_remove_async(c, i64(6), i64(4), i64(10), None) == -1                # not a suffix
    for seq in (5, 6, 7, 8, 9):
        assert lib.cf_sequence_remove_async(c, i64(seq), i64(-1), i64(-1), None) == 0, err()
    torch.cuda.synchronize()
    assert lib.cf_multisequence_reclaim_async(c, None) == 0 and lib.cf_multisequence_audit(c) == 0
    lib.cf_multisequence_get_counters(c, C.byref(k))
    assert k.active_sequences == 0 and k.pages_pending_reclamation == 0 and k.pages_reclaimed == 2 * LAYERS + 1
    assert k.invariant_failures == 0 and k.dense_fallback_launches == 0 and k.unsupported_operations == 4
    assert k.speculative_transactions_committed == 1 and k.speculative_transactions_rolled_back == 1
    lib.cf_multisequence_destroy(c, None)


def test_server_runtime_appends_whole_prompts_and_runs_interleaved_batches(native, oracle):
    import torch
    lib = native.lib()
    lib.cf_llama_server_runtime_create.restype = C.c_void_p
    lib.cf_llama_server_last_error.restype = C.c_char_p
    cfg = LlamaServerConfig(LAYERS, HQ, HKV, D, PAGE, 64, 4096, HQ // HKV, 0, 1, None, b"76f46ad2", b"0" * 64)
    s = C.c_void_p(lib.cf_llama_server_runtime_create(C.byref(cfg)))
    err = lambda: lib.cf_llama_server_last_error(s)
    rng = np.random.default_rng(91)
    i64 = C.c_int64
    rows = {}
    for seq, tokens in ((21, 45), (22, 16)):
        assert lib.cf_llama_server_slot_create(s, i64(seq)) == 0, err()
        for layer in range(LAYERS):
            k = torch.from_numpy(rng.standard_normal((tokens, HKV, D)).astype(np.float32) * 0.8).cuda()
            v = torch.from_numpy(rng.standard_normal((tokens, HKV, D)).astype(np.float32) * 0.8).cuda()
            # a prompt of 45 tokens crosses two page boundaries: the runtime cuts it page by page
            assert lib.cf_llama_server_append_layer_async(s, i64(seq), layer, 0, C.c_void_p(k.data_ptr()),
                                                          C.c_void_p(v.data_ptr()), tokens, None) == 0, err()
            rows[(seq, layer)] = (k.cpu().numpy(), v.cpu().numpy())
    keys = [(21, 0), (22, 1), (21, 1)]
    items = (MsBatchItem * len(keys))()
    keep = []
    for i, (seq, layer) in enumerate(keys):
        q = torch.from_numpy(rng.standard_normal((1, HQ, D)).astype(np.float32)).half().cuda()
        out = torch.zeros((1, HQ, D), dtype=torch.float32, device="cuda")
        items[i] = _item(seq, layer, q, out, rows[(seq, layer)][0].shape[0] - 1)
        keep.append((q, out))
    batch = LlamaServerBatch(None, 0, C.cast(items, C.c_void_p), len(keys))
    assert lib.cf_llama_server_execute_batch_async(s, C.byref(batch), None) == 0, err()
    torch.cuda.synchronize()
    for (seq, layer), (q, out) in zip(keys, keep):
        k, v = rows[(seq, layer)]
        sealed = k.shape[0] // PAGE * PAGE
        want = _expected(oracle, k, v, sealed, 16, q.float().cpu().numpy(), [k.shape[0] - 1], 1.0 / np.sqrt(D), HQ // HKV)
        assert np.allclose(out.cpu().numpy(), want, rtol=2e-3, atol=1e-3), (seq, layer)
    assert lib.cf_llama_server_shutdown_async(s, None) == 0, err()
    lib.cf_llama_server_runtime_destroy(s, None)


def test_forked_sequences_and_prefill_items_take_the_shared_prefix_path(native, oracle):
    """Sequences forked from one prompt share its sealed pages; a batch over them (and a prefill item, whose query tokens
    all see the item's sealed history) is served by the shared-prefix kernel without the caller saying anything: the
    resolver works the hint out from its own page references. The answers must equal the ones the same items get one by
    one (batches of fewer than four rows never take that path) and the oracle's."""
    import torch
    lib = native.lib()
    lib.cf_multisequence_create.restype = C.c_void_p
    lib.cf_multisequence_last_error.restype = C.c_char_p
    c = C.c_void_p(lib.cf_multisequence_create(C.byref(MultisequenceConfig(1, HKV, HQ, D, PAGE, HQ // HKV, 0, 1))))
    err = lambda: lib.cf_multisequence_last_error(c)
    i64 = C.c_int64
    rng = np.random.default_rng(91)
    rows = {}

    def append(seq, tokens):
        begin = rows[seq][0].shape[0] if seq in rows else 0
        done = 0
        while done < tokens:                                   # page by page: an append never crosses a page boundary
            n = min(tokens - done, PAGE - (begin + done) % PAGE)
            k = torch.from_numpy(rng.standard_normal((n, HKV, D)).astype(np.float32) * 0.8).cuda()
            v = torch.from_numpy(rng.standard_normal((n, HKV, D)).astype(np.float32) * 0.8).cuda()
            assert lib.cf_sequence_append_async(c, i64(seq), 0, begin + done, C.byref(_view(k, n)), C.byref(_view(v, n)), None) == 0, err()
            old = rows.get(seq, [np.zeros((0, HKV, D), np.float32)] * 2)
            rows[seq] = [np.concatenate([old[0], k.cpu().numpy()]), np.concatenate([old[1], v.cpu().numpy()])]
            done += n

    assert lib.cf_sequence_create(c, i64(1)) == 0
    append(1, 20 * PAGE)                                       # a 320-token prompt: 20 sealed pages
    forks = list(range(2, 10))
    for seq in forks:
        assert lib.cf_sequence_copy_async(c, i64(1), i64(seq), 0, 1 << 30, None) == 0, err()
        rows[seq] = [a.copy() for a in rows[1]]
        append(seq, 3 + seq)                                   # private continuations of different lengths, some sealing a page
    qs = {s: torch.from_numpy(rng.standard_normal((1, HQ, D)).astype(np.float32)).cuda() for s in forks}

    def run(seqs):
        outs = {s: torch.zeros((1, HQ, D), dtype=torch.float32, device="cuda") for s in seqs}
        items = (MsBatchItem * len(seqs))()
        for i, s in enumerate(seqs):
            items[i] = _item(s, 0, qs[s], outs[s], rows[s][0].shape[0] - 1)
        assert lib.cf_multisequence_attention_async(c, items, len(seqs), None) == 0, err()
        torch.cuda.synchronize()
        return {s: outs[s].cpu().numpy() for s in seqs}

    lib.cf_b200_shared_prefix_launches.restype = C.c_uint64
    before = lib.cf_b200_shared_prefix_launches()
    together = run(forks)                                      # 8 rows sharing 20 pages: the shared-prefix path
    assert lib.cf_b200_shared_prefix_launches() == before + 1
    for s in forks:
        alone = run([s])[s]                                    # one row: the per-sequence path
        assert lib.cf_b200_shared_prefix_launches() == before + 1
        assert np.abs(together[s] - alone).max() <= 2e-5, s
        k, v = rows[s]
        want = _expected(oracle, k, v, k.shape[0] // PAGE * PAGE, 16, qs[s].cpu().numpy(), [k.shape[0] - 1], 1.0 / np.sqrt(D), HQ // HKV)
        assert np.allclose(together[s], want, rtol=2e-3, atol=1e-3), s

    # prefill: six query tokens of sequence 1 in one item, at the last six positions of a 5-token tail after the prompt
    append(1, 5)
    n = rows[1][0].shape[0]
    q = torch.from_numpy(rng.standard_normal((5, HQ, D)).astype(np.float32)).cuda()
    out = torch.zeros((5, HQ, D), dtype=torch.float32, device="cuda")
    items = (MsBatchItem * 1)()
    items[0] = _item(1, 0, q, out, n - 5)
    assert lib.cf_multisequence_attention_async(c, items, 1, None) == 0, err()
    torch.cuda.synchronize()
    assert lib.cf_b200_shared_prefix_launches() == before + 2  # five query tokens over 20 sealed pages
    k, v = rows[1]
    want = _expected(oracle, k, v, 20 * PAGE, 16, q.cpu().numpy(), list(range(n - 5, n)), 1.0 / np.sqrt(D), HQ // HKV)
    assert np.allclose(out.cpu().numpy(), want, rtol=2e-3, atol=1e-3)
    assert lib.cf_multisequence_audit(c) == 0
    lib.cf_multisequence_destroy(c, None)
