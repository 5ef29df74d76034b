"""ctypes mirrors of the reference structs this library is layout-compatible with (include/chromofold_b200/compat_*.h)."""
import ctypes as C

_u32, _u64, _vp, _f32 = C.c_uint32, C.c_uint64, C.c_void_p, C.c_float


class SoftmaxState(C.Structure):
    _fields_ = [("max_score", C.c_double), ("exp_sum", C.c_double), ("weighted_values", C.POINTER(C.c_double)),
                ("dim", _u32), ("initialized", _u32)]


class PageView(C.Structure):
    _fields_ = [(n, _u32) for n in ("struct_size", "abi_version", "flags", "layer", "kv_head", "token_begin", "token_count",
                                    "head_dim", "block_size", "zero_point")] + [
        ("k_words", _vp), ("k_word_count", _u64), ("k_block_offsets", _vp), ("k_block_count", _u64),
        ("k_lut", _vp), ("k_lut_count", _u64), ("k_scales", _vp), ("k_scale_count", _u64),
        ("v_words", _vp), ("v_word_count", _u64), ("v_block_offsets", _vp), ("v_block_count", _u64),
        ("v_lut", _vp), ("v_lut_count", _u64), ("v_scales", _vp), ("v_scale_count", _u64)]


class CacheLayout(C.Structure):
    _fields_ = [(n, _u32) for n in ("struct_size", "abi_version", "layer_count", "kv_head_count", "head_dim",
                                    "page_capacity_tokens", "active_token_begin", "active_token_count",
                                    "active_element_bytes", "reserved")] + [
        ("pages", C.POINTER(PageView)), ("page_count", _u64), ("active_k_bytes", _u64), ("active_v_bytes", _u64)]


class MemoryStats(C.Structure):
    _fields_ = [(n, _u64) for n in ("sealed_payload_bytes", "sealed_descriptor_bytes", "active_payload_bytes",
                                    "total_resident_bytes", "sealed_tokens", "active_tokens", "page_count")]


class DevicePage(C.Structure):
    _fields_ = [(n, _vp) for n in ("k_words", "k_block_offsets", "k_lut", "k_scales", "v_words", "v_block_offsets",
                                   "v_lut", "v_scales")] + [
        (n, _u32) for n in ("token_begin", "token_count", "head_dim", "block_size", "k_max_code_length",
                            "v_max_code_length", "zero_point", "kv_head", "fixed_code_length")]


class PagedAttentionDesc(C.Structure):
    _fields_ = [("struct_size", _u32), ("abi_version", _u32), ("pages", _vp), ("page_count", _u32),
                ("kv_head_count", _u32), ("query_head_count", _u32), ("gqa_group_size", _u32), ("active_k", _vp),
                ("active_v", _vp), ("active_token_begin", _u32), ("active_token_count", _u32), ("queries", _vp),
                ("output", _vp), ("query_token_begin", _u32), ("query_count", _u32), ("head_dim", _u32),
                ("causal_window", _u32), ("softmax_scale", _f32)]


class LlamaKvOptions(C.Structure):
    _fields_ = [(n, _u32) for n in ("struct_size", "backend", "layer_count", "kv_head_count", "query_head_count",
                                    "head_dim", "page_size", "gqa_group_size", "kv_bits")]


class LlamaKvStats(C.Structure):
    _fields_ = [(n, _u64) for n in ("appended_tokens", "sealed_tokens", "sealed_pages", "active_tokens",
                                    "dense_active_bytes", "compressed_bytes", "descriptor_bytes")]


class TensorView(C.Structure):
    _fields_ = [("data", _vp), ("scalar_type", _u32), ("token_count", _u32), ("head_count", _u32), ("head_dim", _u32),
                ("token_stride_bytes", _u64), ("head_stride_bytes", _u64), ("element_stride_bytes", _u64),
                ("device_ordinal", C.c_int32)]


class DeviceKvConfig(C.Structure):
    _fields_ = [(n, _u32) for n in ("layer_count", "kv_head_count", "query_head_count", "head_dim", "page_size",
                                    "gqa_group_size", "use_async_allocator")]


class DeviceKvCounters(C.Structure):
    _fields_ = [(n, _u64) for n in (
        "device_append_calls", "device_values_appended", "fp16_values_converted", "bf16_values_converted",
        "fp32_values_copied", "quantization_launches", "huffman_pack_launches", "seal_attempts", "seal_successes",
        "seal_failures", "descriptor_publications", "compressed_attention_launches", "sealed_values_consumed",
        "active_values_consumed", "query_conversion_launches", "output_conversion_launches", "dense_fallback_launches",
        "cuda_errors", "active_bytes", "compressed_bytes", "descriptor_bytes", "workspace_bytes", "retired_pending_bytes",
        "peak_owned_bytes")]


class DeviceSealConfig(C.Structure):
    _fields_ = [(n, _u32) for n in ("layer_count", "kv_head_count", "query_head_count", "head_dim", "page_size",
                                    "gqa_group_size", "block_size", "use_async_allocator")]


class DeviceSealCounters(C.Structure):
    _fields_ = [(n, _u64) for n in (
        "seal_attempts", "seal_successes", "seal_failures", "finite_validation_launches", "values_scanned", "nan_values",
        "inf_values", "invalid_pages_rejected", "quantization_launches", "values_quantized", "saturation_count",
        "packing_launches", "symbols_packed", "payload_bytes_written", "descriptor_validations",
        "descriptor_publications", "page_table_reallocations", "page_table_generation", "compressed_attention_launches",
        "sealed_pages_consumed", "sealed_values_consumed", "active_values_consumed", "query_conversion_launches",
        "output_conversion_launches", "cuda_errors", "compressed_bytes", "descriptor_bytes", "workspace_bytes",
        "peak_owned_bytes")]


class PageDescriptor(C.Structure):
    _fields_ = [("key_payload", _vp), ("value_payload", _vp), ("key_scales", _vp), ("value_scales", _vp)] + [
        (n, _u32) for n in ("token_begin", "token_count", "kv_head_count", "head_dim", "block_size", "blocks_per_page")] + [
        (n, _u64) for n in ("key_payload_bytes", "value_payload_bytes", "resident_bytes", "generation")]


class MsConfig(C.Structure):
    _fields_ = [(n, _u32) for n in ("layer_count", "kv_head_count", "query_head_count", "head_dim", "page_size",
                                    "gqa_group_size", "use_async_allocator")]


class MsPublication(C.Structure):
    _fields_ = [("sequence_id", C.c_int64), ("layer", _u32), ("descriptor", PageDescriptor), ("resident_bytes", _u64),
                ("seal_generation", _u64)]


class MsBatchItem(C.Structure):
    _fields_ = [("sequence_id", C.c_int64), ("layer", _u32), ("query", TensorView), ("output", _vp), ("output_type", _u32),
                ("output_token_stride_bytes", _u64), ("output_head_stride_bytes", _u64), ("output_element_stride_bytes", _u64),
                ("query_token_begin", _u32), ("softmax_scale", _f32), ("causal_window", _u32)]


class MsCounters(C.Structure):
    _fields_ = [(n, _u64) for n in (
        "pages_registered", "page_registration_failures", "descriptor_tables_built", "descriptor_table_rebuilds",
        "snapshots_acquired", "snapshots_released", "in_flight_page_references", "snapshot_release_events",
        "stale_snapshot_rejections", "server_batches_received", "compressed_batches_executed",
        "sequence_attention_launches", "prefill_items", "decode_items", "tokens_per_batch_peak",
        "copy_on_write_tail_copies", "cancellation_requests", "pages_retired", "pages_reclaimed",
        "pending_reclamation_bytes", "pending_reclamation_bytes_peak", "cross_sequence_contamination",
        "dense_fallback_launches", "cuda_errors")]


assert C.sizeof(PageDescriptor) == 88 and C.sizeof(MsPublication) == 120 and C.sizeof(MsBatchItem) == 128
assert C.sizeof(TensorView) == 56 and C.sizeof(DeviceSealCounters) == 29 * 8 and C.sizeof(DeviceKvCounters) == 24 * 8
assert C.sizeof(PageView) == 168 and C.sizeof(CacheLayout) == 72 and C.sizeof(DevicePage) == 104
assert C.sizeof(PagedAttentionDesc) == 96 and C.sizeof(SoftmaxState) == 32


class AttentionTuning(C.Structure):
    _fields_ = [(n, _u32) for n in ("threads_per_block", "warps_per_block", "heads_per_block", "pages_per_work_unit",
                                    "vector_width", "enable_cuda_graphs", "enable_async_sealing")]


class AttentionRuntimeConfig(C.Structure):
    _fields_ = [(n, _u32) for n in ("layer_count", "query_head_count", "kv_head_count", "head_dim", "page_size",
                                    "block_size", "gqa_group_size", "cuda_device", "use_async_allocator", "mode")] + [
        ("tuning", AttentionTuning)]


class AttentionBatchItem(C.Structure):
    _fields_ = [("sequence_id", C.c_int64), ("layer", _u32), ("query", TensorView), ("output", _vp), ("output_type", _u32),
                ("output_token_stride_bytes", _u64), ("output_head_stride_bytes", _u64),
                ("output_element_stride_bytes", _u64), ("query_token_begin", _u32), ("softmax_scale", C.c_float),
                ("causal_window", _u32), ("sealed_pages", _vp), ("sealed_page_count", _u32), ("active_keys", _vp),
                ("active_values", _vp), ("active_token_begin", _u32), ("active_token_count", _u32)]


ATTENTION_COUNTER_NAMES = (
    "reference_launches", "optimized_launches", "decode_launches", "prefill_launches", "grouped_batches", "grouped_items",
    "kernel_launches_avoided", "graph_captures", "graph_replays", "graph_invalidations", "graph_replay_failures",
    "async_seal_submissions", "async_seal_overlaps", "descriptor_bytes_read", "compressed_payload_bytes_read",
    "scale_bytes_read", "allocation_count", "pool_hits", "pool_misses", "peak_reserved_bytes", "peak_live_bytes",
    "numerical_failures", "cross_sequence_contamination", "dense_fallback_launches", "cuda_errors")


class AttentionCounters(C.Structure):
    _fields_ = [(n, _u64) for n in ATTENTION_COUNTER_NAMES]


class MultisequenceConfig(C.Structure):
    _fields_ = [(n, _u32) for n in ("layer_count", "kv_head_count", "query_head_count", "head_dim", "page_size",
                                    "gqa_group_size", "use_async_allocator", "enable_invariant_auditor")]


MULTISEQUENCE_COUNTER_NAMES = (
    "sequences_created", "sequences_copied", "sequences_removed", "sequences_shifted", "active_sequences",
    "active_sequences_peak", "shared_pages", "shared_page_references", "page_ref_increments", "page_ref_decrements",
    "pages_reclaimed", "pages_pending_reclamation", "pending_reclamation_bytes", "pending_reclamation_bytes_peak",
    "speculative_transactions_started", "speculative_transactions_committed", "speculative_transactions_rolled_back",
    "batches_dispatched", "sequences_per_batch_peak", "invariant_audits", "invariant_failures", "unsupported_operations",
    "dense_fallback_launches")


class MultisequenceCounters(C.Structure):
    _fields_ = [(n, _u64) for n in MULTISEQUENCE_COUNTER_NAMES]


class LlamaServerConfig(C.Structure):
    _fields_ = [(n, _u32) for n in ("layer_count", "query_head_count", "kv_head_count", "head_dim", "page_size",
                                    "block_size", "context_window", "gqa_group_size", "cuda_device", "strict_mode")] + [
        ("evidence_path", C.c_char_p), ("llama_commit", C.c_char_p), ("model_sha256", C.c_char_p)]


class LlamaServerBatch(C.Structure):
    _fields_ = [("tokens", _vp), ("token_item_count", _u32), ("attention_items", _vp), ("attention_item_count", _u32)]


class LlamaServerStats(C.Structure):
    _fields_ = [(n, _u64) for n in ("http_requests", "interleaved_batches", "slot_reuses", "cancelled_requests",
                                    "context_shifts", "speculative_rollbacks", "dense_nodes_scheduled", "shutdown_audits",
                                    "shutdown_failures")]


class MultigpuDeviceConfig(C.Structure):
    _fields_ = [("device_ordinal", C.c_int32), ("memory_budget_bytes", _u64), ("peer_group", _u32)]


class MultigpuRuntimeConfig(C.Structure):
    _fields_ = [("devices", _vp)] + [(n, _u32) for n in ("device_count", "layer_count", "tensor_parallel_size",
                                                          "allow_host_staging", "require_peer_access", "collective")]


class MultigpuPageView(C.Structure):
    _fields_ = [("key_payload", _vp), ("value_payload", _vp), ("key_scales", _vp), ("value_scales", _vp),
                ("key_payload_bytes", _u64), ("value_payload_bytes", _u64)] + [
        (n, _u32) for n in ("key_codec", "value_codec", "token_count", "kv_head_count", "head_dim", "block_size")] + [
        ("source_device", C.c_int32), ("generation", _u64)]


class MultigpuShard(C.Structure):
    _fields_ = [("sequence_id", _u64), ("layer", _u32), ("query_head_begin", _u32), ("query_head_count", _u32),
                ("execution_device", C.c_int32), ("query", _vp), ("output", _vp), ("query_type", _u32),
                ("output_type", _u32), ("head_dim", _u32), ("page_count", _u32), ("pages", _vp)]


class MultigpuCounters(C.Structure):
    _fields_ = [(n, _u64) for n in (
        "batches_submitted", "shards_dispatched", "p2p_copy_calls", "p2p_bytes", "host_staged_copy_calls",
        "host_staged_bytes", "collective_calls", "collective_bytes", "mixed_codec_pages_consumed", "remote_pages_loaded",
        "migrations_completed", "device_failures_detected", "fail_closed_rejections", "cross_device_contamination",
        "dense_fallback_launches", "cuda_errors", "transfer_errors", "page_refs_at_shutdown", "snapshot_refs_at_shutdown")]


# ---- llama.cpp-side bridges (include/chromofold_b200/compat_bridges.h, compat_llama_ms_bridge.h) ----
class LlamaTensorView(C.Structure):
    _fields_ = [("data", _vp), ("token_stride_bytes", _u64), ("head_stride_bytes", _u64), ("element_stride_bytes", _u64),
                ("token_count", _u32), ("head_count", _u32), ("head_dim", _u32), ("scalar_type", _u32)]


class LlamaRuntimeOptions(C.Structure):
    _fields_ = [("struct_size", _u32), ("kv", LlamaKvOptions), ("causal_window", _u32), ("require_cuda", _u32),
                ("allow_dense_fallback", _u32), ("emit_stats", _u32)]


class LlamaRuntimeCounters(C.Structure):
    _fields_ = [(n, _u64) for n in ("append_calls", "appended_values", "compressed_attention_launches",
                                    "sealed_values_consumed", "active_values_consumed", "dense_fallback_launches",
                                    "rejected_operations", "cuda_errors")]


class LlamaRuntimeSnapshot(C.Structure):
    _fields_ = [("kv", LlamaKvStats), ("counters", LlamaRuntimeCounters), ("backend_selected", _u32), ("initialized", _u32),
                ("dense_fallback_allowed", _u32), ("evidence_complete", _u32)]


class LlamaModelTopology(C.Structure):
    _fields_ = [(n, _u32) for n in ("struct_size", "layer_count", "query_head_count", "kv_head_count", "head_dim",
                                    "context_size", "uniform_kv_geometry", "causal", "recurrent")]


class LlamaGraphOptions(C.Structure):
    _fields_ = [("struct_size", _u32), ("backend", _u32), ("page_size", _u32), ("window", _u32), ("emit_stats", _u32),
                ("evidence_path", C.c_char_p)]


class LlamaGraphCounters(C.Structure):
    _fields_ = [(n, _u64) for n in ("graph_append_calls", "graph_attention_dispatches", "graph_dense_dispatches",
                                    "query_layout_conversions", "output_layout_conversions", "unsupported_graphs")]


class LlamaDeviceSealOptions(C.Structure):
    _fields_ = [("struct_size", _u32), ("seal", DeviceSealConfig), ("require_cuda", _u32), ("allow_dense_fallback", _u32)]


class LlamaDeviceGraphOptions(C.Structure):
    _fields_ = [("struct_size", _u32), ("kv", DeviceKvConfig), ("causal", _u32), ("linear_sequence_only", _u32),
                ("dense_fallback_forbidden", _u32)]


class LlamaServerMultisequenceConfig(C.Structure):
    _fields_ = [("cache", MultisequenceConfig), ("strict_no_fallback", _u32), ("enable_prefix_sharing", _u32),
                ("enable_speculative_transactions", _u32)]
