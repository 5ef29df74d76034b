"""ctypes view of libchromofold_b200.so (the C ABI declared under include/chromofold_b200/).

There is no fallback: if the shared library is missing or does not load, importing the symbols raises.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libchromofold_b200.so")

CF_OK, CF_ERR_INVALID_ARGUMENT, CF_ERR_UNSUPPORTED, CF_ERR_CUDA = 0, 1, 2, 3
ABI_VERSION = 1
F16, BF16, F32 = 1, 2, 3
CODER_FIXED8, CODER_HUFFMAN, CODER_RANS, CODER_RANS_SPLIT4, CODER_HUFFMAN_SPLIT4 = 0, 1, 2, 3, 4
KERNEL_AUTO, KERNEL_GENERIC, KERNEL_LANES, KERNEL_DECODE_PROBE, KERNEL_DECODE_DUMP = 0, 1, 2, 3, 4
STATIC_WORKSPACE_BYTES = 8 << 20
STAGE_PLAN, STAGE_ATTENTION, STAGE_COMBINE, STAGE_ALL = 1, 2, 4, 7
DEVSTAT_BAD_RECORD, DEVSTAT_WAIT_EXPIRED, DEVSTAT_WORKSPACE, DEVSTAT_NONFINITE, DEVSTAT_ARENA_FULL = 1, 2, 4, 8, 16
DEVSTAT_TAIL_FULL = 0x80

_u32, _u64, _vp, _f32 = C.c_uint32, C.c_uint64, C.c_void_p, C.c_float


class CodebookTables(C.Structure):
    _fields_ = [("rans_slot", _u32 * 4096), ("rans_freq", C.c_uint16 * 256), ("rans_cum", C.c_uint16 * 256),
                ("huff_lut", C.c_uint16 * 4096), ("huff_code", _u32 * 256), ("rans_enc", _u32 * 2 * 256)]


class SealedAttentionDesc(C.Structure):
    _fields_ = [
        ("struct_size", _u32), ("abi_version", _u32),
        ("kv_head_count", _u32), ("query_head_count", _u32), ("head_dim", _u32), ("page_tokens", _u32),
        ("block_size", _u32), ("kv_head_begin", _u32), ("kv_head_span", _u32), ("codebook_id", _u32),
        ("arena", _vp), ("page_dir", _vp), ("page_table", _vp), ("seq_sealed_tokens", _vp), ("seq_slots", _vp),
        ("page_table_stride", _u32), ("seq_count", _u32),
        ("k_tables", _vp), ("v_tables", _vp),
        ("tail_k", _vp), ("tail_v", _vp), ("tail_tokens", _vp),
        ("queries", _vp), ("output", _vp), ("query_type", _u32), ("output_type", _u32),
        ("softmax_scale", _f32), ("causal_window", _u32),
        ("workspace", _vp), ("workspace_bytes", _u64), ("min_pages_per_unit", _u32), ("kernel", _u32),
        ("status", _vp), ("tail_type", _u32), ("tail_capacity", _u32), ("query_positions", _vp),
        ("shared_prefix_pages", _u32), ("reserved0", _u32), ("row_map", _vp),
    ]


class SealDesc(C.Structure):
    _fields_ = [
        ("struct_size", _u32), ("abi_version", _u32),
        ("kv_head_count", _u32), ("head_dim", _u32), ("page_tokens", _u32), ("block_size", _u32),
        ("coder", _u32), ("codebook_id", _u32),
        ("k_tables", _vp), ("v_tables", _vp), ("tail_k", _vp), ("tail_v", _vp),
        ("job_slots", _vp), ("job_pages", _vp), ("job_tokens", _vp), ("job_heads", _vp), ("job_rows", _vp),
        ("job_count", _u32), ("tail_type", _u32), ("tail_capacity", _u32), ("reserved", _u32),
        ("arena", _vp), ("arena_units", _u64), ("arena_cursor_units", _vp), ("page_dir", _vp), ("status", _vp),
    ]


class AppendDesc(C.Structure):
    _fields_ = [
        ("struct_size", _u32), ("abi_version", _u32),
        ("kv_head_count", _u32), ("head_dim", _u32), ("tail_capacity", _u32), ("tail_type", _u32),
        ("tail_k", _vp), ("tail_v", _vp), ("tail_tokens", _vp), ("slots", _vp), ("k_rows", _vp), ("v_rows", _vp),
        ("row_type", _u32), ("row_count", _u32), ("status", _vp),
    ]


class DenseAttentionDesc(C.Structure):
    _fields_ = [
        ("struct_size", _u32), ("abi_version", _u32),
        ("kv_head_count", _u32), ("query_head_count", _u32), ("head_dim", _u32), ("page_tokens", _u32),
        ("pool_k", _vp), ("pool_v", _vp), ("page_table", _vp), ("seq_sealed_tokens", _vp), ("seq_slots", _vp),
        ("page_table_stride", _u32), ("seq_count", _u32),
        ("queries", _vp), ("output", _vp), ("softmax_scale", _f32), ("causal_window", _u32),
        ("workspace", _vp), ("workspace_bytes", _u64), ("min_pages_per_unit", _u32), ("reserved", _u32),
    ]


# Every symbol the headers under include/chromofold_b200 declare; the symbol test walks this list.
EXPORTS = {
    "sealed_kv.h": [
        "cf_b200_sealed_attention_validate", "cf_b200_sealed_attention_workspace_bytes",
        "cf_b200_sealed_attention_async", "cf_b200_sealed_attention_stages_async", "cf_b200_codebook_build",
        "cf_b200_seal_validate", "cf_b200_seal_pages_async", "cf_b200_append_rows_async", "cf_b200_histogram_async", "cf_b200_decode_pages_async",
        "cf_b200_dense_attention_async", "cf_b200_build_info", "cf_b200_sealed_attention_static_async",
        "cf_b200_sealed_attention_static_error", "cf_b200_shared_prefix_launches", "cf_b200_test_wait_expiry",
    ],
    "compat_kv.h": [
        "cf_kv_validate_page", "cf_kv_validate_layout", "cf_kv_page_resident_bytes", "cf_kv_cache_memory_stats",
        "cf_online_softmax_init", "cf_online_softmax_accumulate", "cf_online_softmax_merge", "cf_online_softmax_finalize",
        "cf_kv_validate_paged_attention_desc", "cf_kv_paged_attention_async", "cf_rans_decode_async",
        "cf_kv_attn_fused_async", "cf_kv_attn_dense_async", "cf_delta_fetch_async",
    ],
    "compat_device.h": [
        "cf_device_tensor_validate", "cf_device_kv_create", "cf_device_kv_destroy", "cf_device_kv_append_async",
        "cf_device_kv_seal_full_pages_async", "cf_device_kv_attention_async", "cf_device_kv_clear_async",
        "cf_device_kv_get_counters", "cf_device_kv_last_error", "cf_device_seal_create", "cf_device_seal_destroy",
        "cf_device_seal_stage_active_page", "cf_device_seal_full_page_async", "cf_device_seal_attention_async",
        "cf_device_seal_clear_async", "cf_device_seal_set_fault", "cf_device_seal_get_state",
        "cf_device_seal_get_counters", "cf_device_seal_last_error",
    ],
    "compat_ms.h": [
        "cf_ms_cuda_create", "cf_ms_cuda_destroy", "cf_ms_cuda_sequence_create", "cf_ms_cuda_sequence_remove_async",
        "cf_ms_cuda_publish_page_async", "cf_ms_cuda_stage_active_async", "cf_ms_cuda_copy_sequence_async",
        "cf_ms_cuda_shift_sequence", "cf_ms_cuda_execute_batch_async", "cf_ms_cuda_cancel_sequence_async",
        "cf_ms_cuda_reclaim_async", "cf_ms_cuda_audit", "cf_ms_cuda_get_counters", "cf_ms_cuda_last_error",
        "cf_b200_ms_append_active_async", "cf_b200_ms_seal_active_async", "cf_b200_ms_truncate_async",
        "cf_b200_ms_drop_prefix_async",
        "cf_b200_ms_sequence_tokens", "cf_b200_ms_page_sharing", "cf_b200_ms_arena_stats",
    ],
    "compat_mscache.h": [
        "cf_multisequence_create", "cf_multisequence_destroy", "cf_sequence_create", "cf_sequence_copy_async",
        "cf_sequence_remove_async", "cf_sequence_shift_async", "cf_sequence_append_async",
        "cf_multisequence_attention_async", "cf_sequence_speculation_begin", "cf_sequence_speculation_commit",
        "cf_sequence_speculation_rollback", "cf_multisequence_reclaim_async", "cf_multisequence_audit",
        "cf_multisequence_get_counters", "cf_multisequence_last_error",
        "cf_llama_server_runtime_create", "cf_llama_server_runtime_destroy", "cf_llama_server_slot_create",
        "cf_llama_server_slot_reset_async", "cf_llama_server_cancel_async", "cf_llama_server_sequence_copy_async",
        "cf_llama_server_sequence_remove_async", "cf_llama_server_sequence_shift_async",
        "cf_llama_server_append_layer_async", "cf_llama_server_execute_batch_async", "cf_llama_server_shutdown_async",
        "cf_llama_server_get_stats", "cf_llama_server_last_error",
    ],
    "sealed_kv_multigpu.h": [
        "cf_b200_mg_create", "cf_b200_mg_destroy", "cf_b200_mg_last_error", "cf_b200_mg_set_device_failed",
        "cf_b200_mg_plan_sequences", "cf_b200_mg_plan_kv_heads", "cf_b200_mg_execute_async", "cf_b200_mg_get_counters",
    ],
    "page_transfer.h": ["cf_b200_pages_pack_async", "cf_b200_pages_unpack_async", "cf_b200_fnv1a",
                        "cf_b200_record_checksum"],
    "compat_multigpu.h": [
        "cf_multigpu_cuda_create", "cf_multigpu_cuda_destroy", "cf_multigpu_cuda_validate_topology",
        "cf_multigpu_cuda_execute_async", "cf_multigpu_cuda_migrate_sequence_async",
        "cf_multigpu_cuda_inject_device_failure", "cf_multigpu_cuda_shutdown", "cf_multigpu_cuda_get_counters",
        "cf_multigpu_cuda_last_error",
    ],
    "compat_production.h": [
        "cf_attention_runtime_create", "cf_attention_runtime_destroy", "cf_attention_execute_async",
        "cf_attention_compare_async", "cf_attention_invalidate_graphs", "cf_attention_get_counters",
        "cf_attention_last_error",
    ],
    "compat_bridges.h": [
        "cf_llama_runtime_options_validate", "cf_llama_runtime_create", "cf_llama_runtime_destroy", "cf_llama_runtime_append",
        "cf_llama_runtime_record_compressed_launch", "cf_llama_runtime_record_dense_fallback",
        "cf_llama_runtime_record_cuda_error", "cf_llama_runtime_snapshot_get", "cf_llama_runtime_write_json",
        "cf_llama_runtime_last_error",
        "cf_llama_graph_options_validate", "cf_llama_model_topology_validate", "cf_llama_graph_create",
        "cf_llama_graph_destroy", "cf_llama_graph_append_device", "cf_llama_graph_record_attention",
        "cf_llama_graph_record_dense_dispatch", "cf_llama_graph_get_counters", "cf_llama_graph_write_evidence",
        "cf_llama_graph_last_error",
        "cf_llama_device_seal_bridge_create", "cf_llama_device_seal_bridge_destroy", "cf_llama_device_seal_bridge_stage",
        "cf_llama_device_seal_bridge_seal", "cf_llama_device_seal_bridge_attention", "cf_llama_device_seal_bridge_evidence",
        "cf_llama_device_seal_bridge_last_error",
        "cf_llama_device_graph_create", "cf_llama_device_graph_destroy", "cf_llama_device_graph_append_async",
        "cf_llama_device_graph_attention_async", "cf_llama_device_graph_get_counters", "cf_llama_device_graph_last_error",
        "cf_llama_server_cuda_bridge_create", "cf_llama_server_cuda_bridge_destroy", "cf_llama_server_cuda_slot_create",
        "cf_llama_server_cuda_slot_copy_async", "cf_llama_server_cuda_slot_cancel_async",
        "cf_llama_server_cuda_slot_reset_async", "cf_llama_server_cuda_dispatch_batch_async",
        "cf_llama_server_cuda_shutdown_audit", "cf_llama_server_cuda_last_error",
    ],
    "compat_adapter.h": [
        "cf_llama_kv_options_validate", "cf_llama_kv_create", "cf_llama_kv_destroy", "cf_llama_kv_append",
        "cf_llama_kv_attention", "cf_llama_kv_attention_host", "cf_llama_kv_flush", "cf_llama_kv_seq_rm",
        "cf_llama_kv_seq_cp", "cf_llama_kv_seq_shift", "cf_llama_kv_clear", "cf_llama_kv_get_stats",
        "cf_llama_kv_last_error", "cf_b200_llama_kv_reference_page", "cf_b200_llama_kv_reserved_bytes",
    ],
}

class MgConfig(C.Structure):   # cf_b200_mg_config
    _fields_ = [("struct_size", _u32), ("abi_version", _u32), ("device_count", _u32), ("device_ordinals", _vp),
                ("max_rows", _u32), ("query_head_count", _u32), ("head_dim", _u32), ("query_type", _u32)]


class MgShard(C.Structure):    # cf_b200_mg_shard
    _fields_ = [("desc", SealedAttentionDesc), ("rows", _vp)]


class MgCounters(C.Structure):
    _fields_ = [("steps", _u64), ("attention_launches", _u64), ("peer_copies", _u64), ("peer_bytes", _u64),
                ("refused_batches", _u64), ("direct_steps", _u64)]


MG_BY_SEQUENCE, MG_BY_KV_HEAD = 1, 2


# ---- the reference's llama-server runtime ABI (include/chromofold_b200/compat_mscache.h, compat_device.h) ----
class TensorView(C.Structure):       # cf_device_tensor_view
    _fields_ = [("data", _vp), ("scalar_type", _u32), ("token_count", _u32), ("head_count", _u32), ("head_dim", _u32),
                ("token_stride_bytes", _u64), ("head_stride_bytes", _u64), ("element_stride_bytes", _u64),
                ("device_ordinal", C.c_int32)]


class SequenceAttentionItem(C.Structure):   # cf_sequence_attention_item == cf_ms_batch_item
    _fields_ = [("sequence_id", C.c_int64), ("layer", _u32), ("query", TensorView), ("output", _vp), ("output_type", _u32),
                ("output_token_stride_bytes", _u64), ("output_head_stride_bytes", _u64), ("output_element_stride_bytes", _u64),
                ("query_token_begin", _u32), ("softmax_scale", _f32), ("causal_window", _u32)]


class LlamaServerConfig(C.Structure):
    _fields_ = [(n, _u32) for n in ("layer_count", "query_head_count", "kv_head_count", "head_dim", "page_size",
                                    "block_size", "context_window", "gqa_group_size", "cuda_device", "strict_mode")] + [
        ("evidence_path", C.c_char_p), ("llama_commit", C.c_char_p), ("model_sha256", C.c_char_p)]


class LlamaServerBatch(C.Structure):
    _fields_ = [("tokens", _vp), ("token_item_count", _u32), ("attention_items", _vp), ("attention_item_count", _u32)]


class TransferHeader(C.Structure):
    _fields_ = [("magic", _u64), ("version", _u32), ("format_version", _u32), ("kv_head_count", _u32), ("head_dim", _u32),
                ("page_tokens", _u32), ("block_size", _u32), ("codebook_id", _u32), ("page_count", _u32),
                ("payload_bytes", _u64), ("manifest_checksum", _u64), ("reserved", _u64)]


FORMAT_VERSION = 1   # CF_B200_FORMAT_VERSION of include/chromofold_b200/sealed_page_format.h
TRANSFER_MAGIC = 0x3147504643
DEVSTAT_CHECKSUM = 0x40

# Exported by libchromofold_b200_llama_ms.so (its names clash with compat_mscache.h's llama-server runtime)
MS_BRIDGE_EXPORTS = {
    "compat_llama_ms_bridge.h": [
        "cf_llama_server_multisequence_create", "cf_llama_server_multisequence_destroy", "cf_llama_server_slot_create",
        "cf_llama_server_slot_reset_async", "cf_llama_server_sequence_copy_async", "cf_llama_server_sequence_remove_async",
        "cf_llama_server_context_shift_async", "cf_llama_server_cancel_sequence_async",
        "cf_llama_server_batch_attention_async", "cf_llama_server_audit", "cf_llama_server_multisequence_last_error",
    ],
}
MS_BRIDGE_LIB_PATH = os.path.join(os.path.dirname(LIB_PATH), "libchromofold_b200_llama_ms.so")

_lib = None
_ms_bridge_lib = None


def ms_bridge_lib():
    """The llama-server multi-sequence bridge library (built beside the main one, linked against it)."""
    global _ms_bridge_lib
    if _ms_bridge_lib is None:
        lib()   # the bridge needs the main library's symbols
        if not os.path.exists(MS_BRIDGE_LIB_PATH):
            raise RuntimeError(f"{MS_BRIDGE_LIB_PATH} is missing: build it with `python -m chromofold_b200.build`")
        _ms_bridge_lib = C.CDLL(MS_BRIDGE_LIB_PATH)
    return _ms_bridge_lib


def lib():
    """The loaded shared library. Raises if it was not built (run `python -m chromofold_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m chromofold_b200.build`; "
                               "this package has no CPU or PyTorch fallback")
        _lib = C.CDLL(LIB_PATH)
        _lib.cf_b200_build_info.restype = C.c_char_p
        for name in ("cf_b200_sealed_attention_validate", "cf_b200_sealed_attention_workspace_bytes",
                     "cf_b200_sealed_attention_async", "cf_b200_sealed_attention_stages_async",
                     "cf_b200_codebook_build", "cf_b200_seal_validate",
                     "cf_b200_seal_pages_async", "cf_b200_append_rows_async", "cf_b200_histogram_async", "cf_b200_decode_pages_async",
                     "cf_b200_dense_attention_async", "cf_b200_sealed_attention_static_async"):
            getattr(_lib, name).restype = C.c_int
        _lib.cf_b200_sealed_attention_static_error.restype = C.c_char_p
        _lib.cf_b200_mg_create.restype = C.c_void_p
        _lib.cf_b200_mg_last_error.restype = C.c_char_p
        _lib.cf_b200_mg_last_error.argtypes = [C.c_void_p]
        _lib.cf_b200_mg_destroy.argtypes = [C.c_void_p]
    return _lib


class CfError(RuntimeError):
    def __init__(self, what, status):
        names = {1: "CF_ERR_INVALID_ARGUMENT", 2: "CF_ERR_UNSUPPORTED", 3: "CF_ERR_CUDA"}
        super().__init__(f"{what}: {names.get(status, status)}")
        self.status = status


def check(what, status):
    if status != CF_OK:
        raise CfError(what, status)
