"""Host-side mirror of the reference's single-layer compressed cache for the sealed-KV path.

The reference's CompressedKvCache (src/runtime/compressed_kv_cache.cu:66-178) keeps an appendable active tail,
seals full pages and hands an attention view to the kernel. This class keeps the same life cycle —
append -> seal_full_pages -> attention — for a batch of sequence slots, but every buffer lives on the GPU and
sealing and attention are the library's CUDA entry points (include/chromofold_b200/sealed_kv.h). PyTorch is
used for device memory and streams only.
"""
import ctypes as C

import numpy as np
import torch

from . import _native as N


def _ptr(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _stream_ptr():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _on_own_device(method):
    """Runs a method with the layer's GPU as the current CUDA device: the library launches on the current device, and a
    kernel must only ever be given memory of the GPU it runs on."""
    import functools

    @functools.wraps(method)
    def wrapper(self, *args, **kw):
        with torch.cuda.device(self.device):
            return method(self, *args, **kw)
    return wrapper


class SealedKvLayer:
    """One layer of sealed KV pages for up to `max_sequences` sequence slots on one GPU."""

    def __init__(self, *, kv_heads, query_heads, head_dim=128, page_tokens=16, block_size=64, coder=N.CODER_RANS,
                 max_sequences, max_pages_per_sequence, max_pages, arena_bytes, workspace_bytes=None,
                 codebook_id=0, device="cuda:0"):
        if not torch.cuda.is_available():
            raise RuntimeError("chromofold_b200 needs a CUDA device; there is no CPU path")
        self.lib = N.lib()
        self.device = torch.device(device)
        self.kv_heads, self.query_heads, self.head_dim = kv_heads, query_heads, head_dim
        self.page_tokens, self.block_size, self.coder, self.codebook_id = page_tokens, block_size, coder, codebook_id
        self.max_sequences, self.max_pages_per_sequence, self.max_pages = max_sequences, max_pages_per_sequence, max_pages
        dev = self.device
        self.arena_units = arena_bytes // 16
        self.arena = torch.zeros(self.arena_units * 16 + 64, dtype=torch.uint8, device=dev)
        self.page_dir = torch.zeros(max_pages * kv_heads, dtype=torch.int64, device=dev)
        self.page_table = torch.zeros((max_sequences, max_pages_per_sequence), dtype=torch.int32, device=dev)
        self.sealed_tokens = torch.zeros(max_sequences, dtype=torch.int32, device=dev)
        self.tail_tokens = torch.zeros(max_sequences, dtype=torch.int32, device=dev)
        self.tail_k = torch.zeros((max_sequences, kv_heads, page_tokens, head_dim), dtype=torch.float16, device=dev)
        self.tail_v = torch.zeros_like(self.tail_k)
        self.cursor = torch.zeros(1, dtype=torch.int64, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.k_tables = torch.zeros(C.sizeof(N.CodebookTables), dtype=torch.uint8, device=dev)
        self.v_tables = torch.zeros_like(self.k_tables)
        if workspace_bytes is None:
            d = self._attention_desc(None, None, max_sequences, None)
            d.shared_prefix_pages = 1   # also set room aside for the partials of a shared prefix
            need = C.c_uint64(0)
            N.check("workspace_bytes", self.lib.cf_b200_sealed_attention_workspace_bytes(
                C.byref(d), C.c_uint64(max_sequences * max_pages_per_sequence), C.byref(need)))
            workspace_bytes = need.value
        self.workspace = torch.zeros(workspace_bytes + 256, dtype=torch.uint8, device=dev)
        # host bookkeeping (authoritative for page ids and lengths)
        self.h_page_table = np.zeros((max_sequences, max_pages_per_sequence), np.int32)
        self.h_sealed = np.zeros(max_sequences, np.int64)
        self.h_tail = np.zeros(max_sequences, np.int64)
        self.next_page_id = 1  # page id 0 stays unpublished so a zeroed table entry is detectable
        self.host_tables = (N.CodebookTables(), N.CodebookTables())
        self._codebooks_set = False

    # -- codebooks ---------------------------------------------------------------------------------
    @_on_own_device
    def set_codebooks(self, hist_k, hist_v):
        for hist, host, dev in ((hist_k, self.host_tables[0], self.k_tables), (hist_v, self.host_tables[1], self.v_tables)):
            h = np.ascontiguousarray(hist, np.uint64)
            N.check("codebook_build", self.lib.cf_b200_codebook_build(h.ctypes.data_as(C.c_void_p), C.byref(host)))
            dev.copy_(torch.frombuffer(bytearray(bytes(host)), dtype=torch.uint8))
        self._codebooks_set = True

    def _need_codebooks(self):
        """An entropy coder codes against the layer's tables; all-zero tables would give records that decode to
        something else than what was sealed."""
        if self.coder != N.CODER_FIXED8 and not self._codebooks_set:
            raise RuntimeError("set_codebooks() must be called before pages are sealed with an entropy coder")

    @_on_own_device
    def histograms(self, slots=None):
        """Symbol histograms of the quantised streams of the current tails (GPU)."""
        slots = self._slots_tensor(slots)
        hk = torch.zeros(256, dtype=torch.int64, device=self.device)
        hv = torch.zeros_like(hk)
        d = self._seal_desc(slots, None, self.tail_tokens[slots.long()].contiguous())
        N.check("histogram", self.lib.cf_b200_histogram_async(C.byref(d), _ptr(hk), _ptr(hv), _stream_ptr()))
        return hk.cpu().numpy().astype(np.uint64), hv.cpu().numpy().astype(np.uint64)

    # -- append / seal -------------------------------------------------------------------------------
    @_on_own_device
    def append(self, slots, k, v):
        """Append one token per listed slot. k, v: float16 device tensors [len(slots), kv_heads, head_dim]."""
        slots = np.asarray(slots, np.int64)
        if np.any(self.h_tail[slots] >= self.page_tokens):
            raise ValueError("active tail is full: seal_full_pages() first")
        key = slots.tobytes()     # the device copy of a slot list is kept: a decode loop appends to the same slots every step
        if getattr(self, "_append_key", None) != key:
            self._append_key, self._append_slots = key, torch.as_tensor(slots.astype(np.int32), device=self.device)
        if k.dtype not in (torch.float16, torch.float32, torch.bfloat16):
            k, v = k.float(), v.float()
        k, v = k.contiguous(), v.to(k.dtype).contiguous()
        d = N.AppendDesc()
        d.struct_size, d.abi_version = C.sizeof(N.AppendDesc), N.ABI_VERSION
        d.kv_head_count, d.head_dim, d.tail_capacity, d.tail_type = self.kv_heads, self.head_dim, self.page_tokens, N.F16
        d.tail_k, d.tail_v, d.tail_tokens = self.tail_k.data_ptr(), self.tail_v.data_ptr(), self.tail_tokens.data_ptr()
        d.slots, d.k_rows, d.v_rows = self._append_slots.data_ptr(), k.data_ptr(), v.data_ptr()
        d.row_type = {torch.float16: N.F16, torch.bfloat16: N.BF16, torch.float32: N.F32}[k.dtype]
        d.row_count, d.status = slots.size, self.status.data_ptr()
        N.check("append_rows", self.lib.cf_b200_append_rows_async(C.byref(d), _stream_ptr()))
        self.h_tail[slots] += 1

    @_on_own_device
    def fill_tails(self, slots, k, v, tokens):
        """Set whole tails at once. k, v: float16 [len(slots), kv_heads, page_tokens, head_dim]."""
        slots = np.asarray(slots, np.int64)
        idx = torch.as_tensor(slots, device=self.device)
        self.tail_k[idx] = k.to(torch.float16)
        self.tail_v[idx] = v.to(torch.float16)
        self.h_tail[slots] = tokens
        self.tail_tokens[idx] = int(tokens)

    @_on_own_device
    def seal_full_pages(self, slots=None, force=False):
        """Seal the tails that hold page_tokens rows (all non-empty tails with force=True, the reference's flush)."""
        cand = np.arange(self.max_sequences) if slots is None else np.asarray(slots, np.int64)
        full = cand[(self.h_tail[cand] >= self.page_tokens) | (force & (self.h_tail[cand] > 0))]
        if full.size == 0:
            return 0
        if np.any(self.h_sealed[full] % self.page_tokens):
            raise ValueError("a sequence with a partly filled sealed page cannot grow")
        page_index = self.h_sealed[full] // self.page_tokens
        if np.any(page_index >= self.max_pages_per_sequence) or self.next_page_id + full.size > self.max_pages:
            raise ValueError("page table or page directory is full")
        ids = np.arange(self.next_page_id, self.next_page_id + full.size, dtype=np.int32)
        self.next_page_id += full.size
        rows = self.h_tail[full].astype(np.int32)
        d_slots = torch.as_tensor(full.astype(np.int32), device=self.device)
        d_ids = torch.as_tensor(ids, device=self.device)
        d_rows = torch.as_tensor(rows, device=self.device)
        d = self._seal_desc(d_slots, d_ids, d_rows)
        self._need_codebooks()
        N.check("seal_pages", self.lib.cf_b200_seal_pages_async(C.byref(d), _stream_ptr()))
        self.h_page_table[full, page_index] = ids
        self.page_table[d_slots.long(), torch.as_tensor(page_index, device=self.device)] = d_ids
        self.h_sealed[full] += rows
        self.h_tail[full] = 0
        self.sealed_tokens[d_slots.long()] += d_rows
        self.tail_tokens[d_slots.long()] = 0
        return int(full.size)

    @_on_own_device
    def seal_tiles(self, slots, k_tiles, v_tiles):
        """Append one full page to every listed slot straight from tile tensors (bulk loading).
        k_tiles, v_tiles: float16 device tensors [len(slots), kv_heads, page_tokens, head_dim]; a slot may appear
        several times, its pages are appended in list order."""
        slots = np.asarray(slots, np.int64)
        n = slots.size
        if self.next_page_id + n > self.max_pages:
            raise ValueError("page directory is full")
        ids = np.arange(self.next_page_id, self.next_page_id + n, dtype=np.int32)
        self.next_page_id += n
        order = np.zeros(n, np.int64)      # position of each job among the jobs of its slot
        seen = {}
        for j, s in enumerate(slots):
            order[j] = seen.get(int(s), 0)
            seen[int(s)] = order[j] + 1
        page_index = self.h_sealed[slots] // self.page_tokens + order
        if np.any(self.h_sealed[slots] % self.page_tokens) or np.any(page_index >= self.max_pages_per_sequence):
            raise ValueError("slot cannot take another full page")
        d_tiles = torch.arange(n, dtype=torch.int32, device=self.device)
        d_ids = torch.as_tensor(ids, device=self.device)
        d = self._seal_desc(d_tiles, d_ids, None)
        d.tail_k, d.tail_v = k_tiles.data_ptr(), v_tiles.data_ptr()
        self._need_codebooks()
        N.check("seal_pages", self.lib.cf_b200_seal_pages_async(C.byref(d), _stream_ptr()))
        self.h_page_table[slots, page_index] = ids
        self.page_table[torch.as_tensor(slots, device=self.device), torch.as_tensor(page_index, device=self.device)] = d_ids
        for s, c in seen.items():
            self.h_sealed[s] += c * self.page_tokens
        self.sealed_tokens.copy_(torch.as_tensor(self.h_sealed.astype(np.int32)))

    @_on_own_device
    def copy_sequence(self, src, dst):
        """Give slot `dst` the history of slot `src` without copying a sealed byte: the sealed pages are shared by page
        id (the reference's shared-page semantics, src/multisequence_cache.cpp:235-292); the unsealed tail is copied."""
        n = int((self.h_sealed[src] + self.page_tokens - 1) // self.page_tokens)
        self.h_page_table[dst, :n] = self.h_page_table[src, :n]
        self.page_table[dst, :n] = self.page_table[src, :n]
        self.h_sealed[dst], self.h_tail[dst] = self.h_sealed[src], self.h_tail[src]
        self.sealed_tokens[dst] = int(self.h_sealed[src])
        self.tail_tokens[dst] = int(self.h_tail[src])
        self.tail_k[dst] = self.tail_k[src]
        self.tail_v[dst] = self.tail_v[src]

    # -- import of records sealed elsewhere ------------------------------------------------------------
    @_on_own_device
    def import_records(self, slot, records, tokens_per_page=None):
        """Append already sealed pages to `slot`. records[p][h] is the record (bytes-like) of page p, kv head h."""
        blobs, entries = [], []
        cursor = int(self.cursor.item())
        for page in records:
            for rec in page:
                rec = np.frombuffer(bytes(rec), np.uint8)
                assert rec.size % 16 == 0
                entries.append(cursor | ((rec.size // 16) << 40))
                blobs.append(rec)
                cursor += rec.size // 16
        if cursor > self.arena_units:
            raise ValueError("arena is full")
        blob = np.concatenate(blobs)
        start = int(self.cursor.item()) * 16
        self.arena[start:start + blob.size] = torch.from_numpy(blob).to(self.device)
        self.cursor.fill_(cursor)
        n = len(records)
        ids = np.arange(self.next_page_id, self.next_page_id + n, dtype=np.int32)
        self.next_page_id += n
        first = int(self.h_sealed[slot] // self.page_tokens)
        e = torch.from_numpy(np.array(entries, np.int64)).to(self.device)
        self.page_dir[int(ids[0]) * self.kv_heads:(int(ids[-1]) + 1) * self.kv_heads] = e
        self.h_page_table[slot, first:first + n] = ids
        self.page_table[slot, first:first + n] = torch.from_numpy(ids).to(self.device)
        added = n * self.page_tokens if tokens_per_page is None else int(np.sum(tokens_per_page))
        self.h_sealed[slot] += added
        self.sealed_tokens[slot] += added

    # -- transfer images (warm-start file / hand-over to another GPU) -------------------------------------
    @_on_own_device
    def export_pages(self, slot):
        """The sealed pages of `slot` as one transfer image (bytes): header, manifest, packed records
        (include/chromofold_b200/page_transfer.h). Packed and checksummed on the GPU."""
        n = int((self.h_sealed[slot] + self.page_tokens - 1) // self.page_tokens)
        ids = torch.as_tensor(self.h_page_table[slot, :n].astype(np.int32), device=self.device)
        manifest = torch.zeros(n * self.kv_heads * 16, dtype=torch.uint8, device=self.device)
        capacity = n * self.kv_heads * (16 + 2 * ((self.head_dim * self.page_tokens + 15) // 16 * 16))
        payload = torch.zeros(capacity + 16, dtype=torch.uint8, device=self.device)
        cursor = torch.zeros(1, dtype=torch.int64, device=self.device)
        N.check("pages_pack", self.lib.cf_b200_pages_pack_async(
            C.c_void_p(self.arena.data_ptr()), C.c_void_p(self.page_dir.data_ptr()), C.c_uint32(self.kv_heads),
            C.c_void_p(ids.data_ptr()), C.c_uint32(n), C.c_void_p(manifest.data_ptr()), C.c_void_p(payload.data_ptr()),
            C.c_uint64(capacity), C.c_void_p(cursor.data_ptr()), C.c_void_p(self.status.data_ptr()), _stream_ptr()))
        used = int(cursor.item()) * 16
        man = manifest.cpu().numpy().tobytes()
        header = N.TransferHeader()
        header.magic, header.version, header.format_version = N.TRANSFER_MAGIC, 1, N.FORMAT_VERSION
        header.kv_head_count, header.head_dim, header.page_tokens = self.kv_heads, self.head_dim, self.page_tokens
        header.block_size, header.codebook_id, header.page_count = self.block_size, self.codebook_id, n
        header.payload_bytes = used
        self.lib.cf_b200_fnv1a.restype = C.c_uint64
        header.manifest_checksum = self.lib.cf_b200_fnv1a(man, C.c_uint64(len(man)))
        tokens = np.minimum(self.page_tokens, self.h_sealed[slot] - np.arange(n) * self.page_tokens).astype(np.uint32)
        return bytes(header) + man + payload[:used].cpu().numpy().tobytes() + tokens.tobytes()

    @_on_own_device
    def import_pages(self, slot, image):
        """Append the pages of a transfer image to `slot`. The image must match this layer's geometry and codebook
        id; every record is verified against its checksum on the GPU (a bad one is not published and raises
        CF_B200_DEVSTAT_CHECKSUM in the status word). Returns the number of pages."""
        header = N.TransferHeader.from_buffer_copy(image[:C.sizeof(N.TransferHeader)])
        if header.magic != N.TRANSFER_MAGIC or header.version != 1 or header.format_version != N.FORMAT_VERSION:
            raise ValueError("not a transfer image of this format version")
        if (header.kv_head_count, header.head_dim, header.page_tokens, header.block_size, header.codebook_id) != (
                self.kv_heads, self.head_dim, self.page_tokens, self.block_size, self.codebook_id):
            raise ValueError("transfer image geometry or codebook id does not match this layer")
        n, hs = header.page_count, C.sizeof(N.TransferHeader)
        man = image[hs:hs + 16 * n * self.kv_heads]
        self.lib.cf_b200_fnv1a.restype = C.c_uint64
        if self.lib.cf_b200_fnv1a(man, C.c_uint64(len(man))) != header.manifest_checksum:
            raise ValueError("transfer image manifest is corrupt")
        body = image[hs + len(man):hs + len(man) + header.payload_bytes]
        tokens = np.frombuffer(image[hs + len(man) + header.payload_bytes:], np.uint32)
        if len(body) != header.payload_bytes or tokens.size != n or self.h_sealed[slot] % self.page_tokens:
            raise ValueError("transfer image is truncated, or the sequence ends in a short page")
        first = int(self.h_sealed[slot] // self.page_tokens)
        if first + n > self.max_pages_per_sequence or self.next_page_id + n > self.max_pages:
            raise ValueError("page table or page directory is full")
        ids = np.arange(self.next_page_id, self.next_page_id + n, dtype=np.int32)
        self.next_page_id += n
        d_ids = torch.as_tensor(ids, device=self.device)
        d_man = torch.frombuffer(bytearray(man), dtype=torch.uint8).to(self.device)
        d_body = torch.zeros(len(body) + 16, dtype=torch.uint8, device=self.device)
        d_body[:len(body)] = torch.frombuffer(bytearray(body), dtype=torch.uint8).to(self.device)
        N.check("pages_unpack", self.lib.cf_b200_pages_unpack_async(
            C.c_void_p(d_man.data_ptr()), C.c_void_p(d_body.data_ptr()), C.c_uint64(len(body)), C.c_uint32(self.kv_heads),
            C.c_void_p(d_ids.data_ptr()), C.c_uint32(n), C.c_void_p(self.arena.data_ptr()), C.c_uint64(self.arena_units),
            C.c_void_p(self.cursor.data_ptr()), C.c_void_p(self.page_dir.data_ptr()), C.c_void_p(self.status.data_ptr()),
            _stream_ptr()))
        torch.cuda.current_stream().synchronize()   # the staging tensors above go away with this frame
        self.h_page_table[slot, first:first + n] = ids
        self.page_table[slot, first:first + n] = d_ids
        self.h_sealed[slot] += int(tokens.sum())
        self.sealed_tokens[slot] += int(tokens.sum())
        return n

    # -- attention -----------------------------------------------------------------------------------
    @_on_own_device
    def attention(self, queries, slots=None, out=None, *, softmax_scale=None, causal_window=0, kernel=N.KERNEL_AUTO,
                  kv_head_begin=0, kv_head_span=0, min_pages_per_unit=0, stages=N.STAGE_ALL, shared_prefix_pages=0,
                  query_positions=None, row_map=None):
        """Decode-step attention: queries [n, query_heads, head_dim] (float16 or float32) -> float32 output.
        shared_prefix_pages = P states that the first P pages of every listed sequence are the same pages (as after
        copy_sequence): they are then decoded once for all the sequences instead of once per sequence.
        query_positions (int32 device tensor [n]) gives every entry's query-token position instead of "right after
        everything cached"; entries naming the same slot at different positions are multi-query (prefill) attention.
        row_map (int32 device tensor [n], with `slots` and `out` given): entry i reads row row_map[i] of `queries` and
        writes row row_map[i] of `out`, so a call can serve a subset of a larger batch in place."""
        n = queries.shape[0] if row_map is None else int(row_map.numel())
        if out is None:
            out = torch.zeros((n, self.query_heads, self.head_dim), dtype=torch.float32, device=self.device)
        d = self._attention_desc(queries, out, n, slots)
        d.softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / float(np.sqrt(self.head_dim))
        d.causal_window = causal_window
        d.kernel = kernel
        d.kv_head_begin, d.kv_head_span = kv_head_begin, kv_head_span
        d.min_pages_per_unit = min_pages_per_unit
        d.shared_prefix_pages = shared_prefix_pages
        if query_positions is not None:
            d.query_positions = query_positions.data_ptr()
        if row_map is not None:
            d.row_map = row_map.data_ptr()
        N.check("sealed_attention", self.lib.cf_b200_sealed_attention_stages_async(C.byref(d), C.c_uint32(stages),
                                                                                      _stream_ptr()))
        return out

    @_on_own_device
    def attention_no_alloc(self, queries, slots=None, out=None, *, softmax_scale=None, causal_window=0,
                           kernel=N.KERNEL_AUTO, shared_prefix_pages=0):
        """The same decode-step attention through the entry point that uses the library's built-in workspace
        (for callers that cannot allocate device memory). `out` must be given by such a caller; it is created here
        only as a convenience for tests."""
        n = queries.shape[0]
        if out is None:
            out = torch.zeros((n, self.query_heads, self.head_dim), dtype=torch.float32, device=self.device)
        d = self._attention_desc(queries, out, n, slots)
        d.workspace, d.workspace_bytes = None, 0
        d.softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / float(np.sqrt(self.head_dim))
        d.causal_window = causal_window
        d.kernel = kernel
        d.shared_prefix_pages = shared_prefix_pages
        status = self.lib.cf_b200_sealed_attention_static_async(C.byref(d), _stream_ptr())
        if status != N.CF_OK:
            raise N.CfError(self.lib.cf_b200_sealed_attention_static_error().decode(), status)
        return out

    @_on_own_device
    def dump_lane_decoders(self, queries, slots=None, *, shared_prefix_pages=0, query_positions=None):
        """Test aid (CF_B200_KERNEL_DECODE_DUMP): run the plan and the attention kernels of a call on `queries`, with the
        lane-per-block decoders of the attention kernels storing every symbol they decode instead of consuming it.
        Returns uint8 [page ids][kv_heads][2 (K, V)][page_tokens*head_dim]; pages the call does not reach stay 0xFF."""
        n = queries.shape[0]
        page_ids = self.page_dir.numel() // self.kv_heads
        dump = torch.full((page_ids, self.kv_heads, 2, self.page_tokens * self.head_dim), 0xFF, dtype=torch.uint8,
                          device=self.device)
        d = self._attention_desc(queries, dump, n, slots)
        d.softmax_scale = 1.0
        d.kernel, d.reserved0 = N.KERNEL_DECODE_DUMP, page_ids
        d.shared_prefix_pages = shared_prefix_pages
        if query_positions is not None:
            d.query_positions = query_positions.data_ptr()
        N.check("decode dump", self.lib.cf_b200_sealed_attention_stages_async(
            C.byref(d), C.c_uint32(N.STAGE_PLAN | N.STAGE_ATTENTION), _stream_ptr()))
        return dump

    @_on_own_device
    def decode_pages(self, page_ids):
        """Decode whole records to symbols on the GPU: returns (k, v) uint8 [pages, kv_heads, page_tokens*head_dim]."""
        ids = torch.as_tensor(np.asarray(page_ids, np.int32), device=self.device)
        n = self.page_tokens * self.head_dim
        ks = torch.zeros((ids.numel(), self.kv_heads, n), dtype=torch.uint8, device=self.device)
        vs = torch.zeros_like(ks)
        d = self._attention_desc(None, None, 1, None)
        N.check("decode_pages", self.lib.cf_b200_decode_pages_async(C.byref(d), _ptr(ids), C.c_uint32(ids.numel()),
                                                                      _ptr(ks), _ptr(vs), _stream_ptr()))
        return ks, vs

    @_on_own_device
    def record_bytes(self, page_id, kv_head):
        """Copy one record back to the host (for byte-exactness checks and statistics)."""
        e = int(self.page_dir[page_id * self.kv_heads + kv_head].item())
        off, units = e & 0xFFFFFFFFFF, (e >> 40) & 0xFFFF
        return self.arena[off * 16:(off + units) * 16].cpu().numpy()

    @_on_own_device
    def sealed_bytes(self):
        return int(self.cursor.item()) * 16

    @_on_own_device
    def device_status(self):
        return int(self.status.item())

    # -- descriptors ---------------------------------------------------------------------------------
    def _slots_tensor(self, slots):
        if slots is None:
            slots = np.arange(self.max_sequences)
        if isinstance(slots, torch.Tensor):
            return slots.to(device=self.device, dtype=torch.int32)
        return torch.as_tensor(np.asarray(slots, np.int32), device=self.device)

    def _attention_desc(self, queries, out, n, slots):
        d = N.SealedAttentionDesc()
        d.struct_size, d.abi_version = C.sizeof(N.SealedAttentionDesc), N.ABI_VERSION
        d.kv_head_count, d.query_head_count, d.head_dim = self.kv_heads, self.query_heads, self.head_dim
        d.page_tokens, d.block_size, d.codebook_id = self.page_tokens, self.block_size, self.codebook_id
        d.arena, d.page_dir = self.arena.data_ptr(), self.page_dir.data_ptr()
        d.page_table, d.seq_sealed_tokens = self.page_table.data_ptr(), self.sealed_tokens.data_ptr()
        if slots is not None:
            self._slots_keepalive = self._slots_tensor(slots)
            d.seq_slots = self._slots_keepalive.data_ptr()
        d.page_table_stride, d.seq_count = self.max_pages_per_sequence, n
        d.k_tables, d.v_tables = self.k_tables.data_ptr(), self.v_tables.data_ptr()
        d.tail_k, d.tail_v, d.tail_tokens = self.tail_k.data_ptr(), self.tail_v.data_ptr(), self.tail_tokens.data_ptr()
        if queries is not None:
            d.queries = queries.data_ptr()
            d.query_type = N.F16 if queries.dtype == torch.float16 else N.F32
            d.output = out.data_ptr()
            d.output_type = N.F16 if out.dtype == torch.float16 else N.F32
        ws = self.workspace.data_ptr() if hasattr(self, "workspace") else 0
        aligned = (ws + 255) // 256 * 256
        d.workspace = aligned
        d.workspace_bytes = (self.workspace.numel() - (aligned - ws)) if hasattr(self, "workspace") else 0
        d.status = self.status.data_ptr()
        return d

    def _seal_desc(self, d_slots, d_ids, d_rows):
        d = N.SealDesc()
        d.struct_size, d.abi_version = C.sizeof(N.SealDesc), N.ABI_VERSION
        d.kv_head_count, d.head_dim, d.page_tokens, d.block_size = self.kv_heads, self.head_dim, self.page_tokens, self.block_size
        d.coder, d.codebook_id = self.coder, self.codebook_id
        d.k_tables, d.v_tables = self.k_tables.data_ptr(), self.v_tables.data_ptr()
        d.tail_k, d.tail_v = self.tail_k.data_ptr(), self.tail_v.data_ptr()
        self._seal_keepalive = (d_slots, d_ids, d_rows)
        d.job_slots = d_slots.data_ptr()
        d.job_pages = d_ids.data_ptr() if d_ids is not None else None
        d.job_tokens = d_rows.data_ptr() if d_rows is not None else None
        d.job_count = d_slots.numel()
        d.arena, d.arena_units = self.arena.data_ptr(), self.arena_units
        d.arena_cursor_units, d.page_dir, d.status = self.cursor.data_ptr(), self.page_dir.data_ptr(), self.status.data_ptr()
        return d


def swizzle_dense_tiles(tiles):
    """Binary16 tiles [..., 16 tokens, 128 channels] -> the chunk-swizzled row layout the dense comparison kernel reads:
    inside a token row, 16-byte chunk c is stored at position c ^ f(token),
    f(token) = (((token ^ (token >> 2)) & 1) << 2) | ((token >> 1) & 1)."""
    tok = torch.arange(16, device=tiles.device)
    f = (((tok ^ (tok >> 2)) & 1) << 2) | ((tok >> 1) & 1)
    src = torch.arange(16, device=tiles.device)[None, :] ^ f[:, None]          # [token][physical chunk] -> logical chunk
    v = tiles.reshape(*tiles.shape[:-2], 16, 16, 8)
    return v[..., tok[:, None], src, :].reshape(tiles.shape).contiguous()


def dense_attention(layer, pool_k, pool_v, queries, out, *, softmax_scale=None, causal_window=0, slots=None):
    """The comparison kernel: attention over uncompressed binary16 pages addressed by `layer`'s page table.
    pool_k / pool_v: swizzled tiles [page_id][kv_heads][16][128] (see swizzle_dense_tiles)."""
    with torch.cuda.device(layer.device):
        return _dense_attention(layer, pool_k, pool_v, queries, out, softmax_scale, causal_window, slots)


def _dense_attention(layer, pool_k, pool_v, queries, out, softmax_scale, causal_window, slots):
    d = N.DenseAttentionDesc()
    d.struct_size, d.abi_version = C.sizeof(N.DenseAttentionDesc), N.ABI_VERSION
    d.kv_head_count, d.query_head_count, d.head_dim, d.page_tokens = layer.kv_heads, layer.query_heads, layer.head_dim, layer.page_tokens
    d.pool_k, d.pool_v = pool_k.data_ptr(), pool_v.data_ptr()
    d.page_table, d.seq_sealed_tokens = layer.page_table.data_ptr(), layer.sealed_tokens.data_ptr()
    if slots is not None:
        layer._slots_keepalive = layer._slots_tensor(slots)
        d.seq_slots = layer._slots_keepalive.data_ptr()
    d.page_table_stride, d.seq_count = layer.max_pages_per_sequence, queries.shape[0]
    d.queries, d.output = queries.data_ptr(), out.data_ptr()
    d.softmax_scale = softmax_scale if softmax_scale is not None else 1.0 / float(np.sqrt(layer.head_dim))
    d.causal_window = causal_window
    ws = layer.workspace.data_ptr()
    aligned = (ws + 255) // 256 * 256
    d.workspace, d.workspace_bytes = aligned, layer.workspace.numel() - (aligned - ws)
    N.check("dense_attention", layer.lib.cf_b200_dense_attention_async(C.byref(d), _stream_ptr()))
    return out
