"""ctypes binding of libmacllm_b200.so (the C ABI declared in include/macllm_b200.h).

The library is built in-tree by build.py.  Importing this module never falls back to a CPU
implementation: if the shared library is missing it raises, and GPU entry points return a
negative status with a message when no CUDA device is usable.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libmacllm_b200.so"

MK_OK, MK_KV_EXHAUSTED = 0, 1
TYPE_F32, TYPE_F16, TYPE_Q8_0, TYPE_Q4_K, TYPE_Q6_K = 0, 1, 8, 12, 14
TYPE_Q4_0, TYPE_Q5_0, TYPE_Q5_1, TYPE_Q2_K, TYPE_Q3_K, TYPE_Q5_K, TYPE_BF16 = 2, 6, 7, 10, 11, 13, 30
PATH_AUTO, PATH_GEMV, PATH_TENSOR, PATH_HALF, PATH_STREAM = 0, 1, 2, 3, 4
FWD_WANT_LOGITS, FWD_WANT_TOKENS = 1, 2


class MkError(RuntimeError):
    pass


class KvExhausted(MkError):
    pass


class LoadConfig(C.Structure):
    _fields_ = [("device_ordinal", C.c_int32), ("block_tokens", C.c_int32), ("slab_blocks", C.c_int32),
                ("kv_capacity_tokens", C.c_int64), ("prefix_capacity_tokens", C.c_int64), ("kv_dtype", C.c_int32),
                ("max_batch_tokens", C.c_int32), ("max_batch_lanes", C.c_int32), ("matmul_path", C.c_int32),
                ("ep_rank", C.c_int32), ("ep_size", C.c_int32), ("ep_mode", C.c_int32)]


class GgufSummary(C.Structure):
    _fields_ = [("architecture", C.c_char * 32), ("n_layers", C.c_int32), ("hidden_size", C.c_int32), ("q_heads", C.c_int32),
                ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("rotary_dim", C.c_int32), ("ffn_size", C.c_int32),
                ("vocab_size", C.c_int32), ("max_context", C.c_int32), ("experts", C.c_int32), ("experts_used", C.c_int32),
                ("expert_ffn_size", C.c_int32), ("tied_embeddings", C.c_int32), ("sliding_layers", C.c_int32),
                ("nope_layers", C.c_int32), ("qk_norm", C.c_int32), ("tensors_in_file", C.c_int64), ("matrices", C.c_int64),
                ("vectors", C.c_int64), ("matrix_bytes", C.c_int64)]


class RuntimeSpec(C.Structure):
    _fields_ = [("vocab_size", C.c_int32), ("max_context", C.c_int32), ("n_layers", C.c_int32), ("hidden_size", C.c_int32),
                ("n_stop_tokens", C.c_int32), ("stop_token_ids", C.c_uint32 * 8), ("weight_bytes", C.c_int64),
                ("weight_bytes_per_token", C.c_int64), ("kv_bytes_per_token", C.c_int64)]


class KvCapacity(C.Structure):
    _fields_ = [("block_tokens", C.c_int64), ("total_blocks", C.c_int64), ("free_blocks", C.c_int64),
                ("retired_blocks", C.c_int64)]


class PoolStats(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("allocated_blocks", "free_blocks", "live_blocks", "reserved_blocks", "retired_blocks",
                                         "shared_blocks", "live_references", "slabs", "submitted_epoch", "completed_epoch")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


class PrefixDiagnostics(C.Structure):
    _fields_ = [(n, C.c_int64) for n in ("entries", "cached_blocks", "capacity_blocks", "hits", "misses", "matched_tokens",
                                         "insertions", "evictions")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


class Lane(C.Structure):
    _fields_ = [("session", C.c_void_p), ("input_ids", C.POINTER(C.c_uint32)), ("n_tokens", C.c_int32), ("start_pos", C.c_int32)]


class EngineConfig(C.Structure):
    _fields_ = [("max_active_sequences", C.c_int32), ("scheduler_token_budget", C.c_int32), ("prefill_token_quantum", C.c_int32),
                ("queue_capacity", C.c_int32), ("record_logits", C.c_int32), ("host_sampling", C.c_int32)]


class Request(C.Structure):
    _fields_ = [("prompt", C.POINTER(C.c_uint32)), ("n_prompt", C.c_int32), ("max_new_tokens", C.c_int32),
                ("ignore_stop_tokens", C.c_int32), ("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float),
                ("repetition_penalty", C.c_float), ("presence_penalty", C.c_float), ("frequency_penalty", C.c_float),
                ("seed", C.c_uint64), ("no_prefix_publication", C.c_int32), ("event_capacity", C.c_int32),
                ("event_send_timeout_ms", C.c_double)]


class TickLane(C.Structure):
    _fields_ = [("request_id", C.c_int32), ("start_pos", C.c_int32), ("n_tokens", C.c_int32), ("phase", C.c_int32)]


class RequestMetrics(C.Structure):
    _fields_ = [("prompt_tokens", C.c_int32), ("cached_prompt_tokens", C.c_int32), ("generated_tokens", C.c_int32),
                ("decode_steps", C.c_int32), ("finish_reason", C.c_int32), ("reserved_", C.c_int32), ("suffix_prefill_ms", C.c_double),
                ("first_token_ms", C.c_double), ("prefill_ms", C.c_double), ("decode_ms", C.c_double)]


class TickInfo(C.Structure):
    _fields_ = [("kind", C.c_int32), ("lane_count", C.c_int32), ("input_tokens", C.c_int32), ("reserved_", C.c_int32),
                ("model_ms", C.c_double)]


class BatchTrace(C.Structure):
    _fields_ = [("expected_members", C.c_int32), ("admitted_members", C.c_int32), ("terminal_members", C.c_int32),
                ("rejected_members", C.c_int32), ("admission_active_sequences", C.c_int32), ("packed_forwards", C.c_int32),
                ("complete", C.c_int32), ("reserved_", C.c_int32), ("suffix_prefill_ms", C.c_double), ("first_token_ms", C.c_double),
                ("decode_ms", C.c_double), ("mixed_ms", C.c_double)]


class EngineStats(C.Structure):
    _fields_ = [("ticks", C.c_int64), ("prefill_tokens", C.c_int64), ("decode_tokens", C.c_int64),
                ("completed_requests", C.c_int64), ("failed_requests", C.c_int64), ("kv_shrinks", C.c_int64),
                ("device_ms", C.c_double), ("cleanup_drains", C.c_int64), ("device_sampled", C.c_int64), ("cancelled_requests", C.c_int64),
                ("suffix_prefill_ms", C.c_double), ("first_token_ms", C.c_double), ("decode_ms", C.c_double), ("mixed_ms", C.c_double)]


class LaneSampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("u", C.c_float)]


class KernelProfile(C.Structure):
    _fields_ = [("name", C.c_char * 32), ("launches", C.c_int64), ("ms", C.c_double), ("bytes", C.c_double), ("flops", C.c_double)]


class AttnCase(C.Structure):
    _fields_ = [("lanes", C.c_int32), ("total_tokens", C.c_int32), ("q_heads", C.c_int32), ("kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("block_tokens", C.c_int32), ("layers", C.c_int32), ("layer", C.c_int32),
                ("pool_blocks", C.c_int32), ("kv_f16", C.c_int32), ("scale", C.c_float), ("softcap", C.c_float),
                ("window", C.c_int32), ("rotary_dim", C.c_int32), ("rope_capacity", C.c_int32), ("norm_eps", C.c_float),
                ("start_pos", C.c_void_p), ("lane_len", C.c_void_p), ("table_off", C.c_void_p), ("table_len", C.c_void_p),
                ("tables", C.c_void_p), ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("q_norm_w", C.c_void_p),
                ("k_norm_w", C.c_void_p), ("cos_table", C.c_void_p), ("sin_table", C.c_void_p), ("k_pool", C.c_void_p),
                ("v_pool", C.c_void_p), ("out", C.c_void_p), ("q_rot_out", C.c_void_p), ("slots_out", C.c_void_p),
                ("positions_out", C.c_void_p), ("last_index_out", C.c_void_p), ("cu_seqlens_out", C.c_void_p),
                ("kernel", C.c_int32)]


# Every symbol include/macllm_b200.h declares, with its ctypes signature (restype is int32 unless noted).
P = C.c_void_p
_i32, _i64, _u32, _u64, _f32 = C.c_int32, C.c_int64, C.c_uint32, C.c_uint64, C.c_float
SIGNATURES = {
    "mk_last_error": (C.c_char_p, []),
    "mk_version": (C.c_char_p, []),
    "mk_device_count": (_i32, []),
    "mk_model_load_gguf": (_i32, [C.c_char_p, C.POINTER(LoadConfig), C.POINTER(P)]),
    "mk_model_new_fake": (_i32, [_i32, _i32, C.POINTER(LoadConfig), _i64, C.POINTER(P)]),
    "mk_model_fake_inject": (_i32, [P, _i32, _i64]),
    "mk_model_fake_on_barrier": (_i32, [P, C.c_void_p, C.c_void_p]),
    "mk_model_ep_idle_tick": (_i32, [P]),
    "mk_k_ep_exchange_emulated": (_i32, [_i32, _i32, _i32, _i32, P, P, _i32, _i32, _i64, P, P, P]),
    "mk_model_free": (_i32, [P]),
    "mk_gguf_inspect": (_i32, [C.c_char_p, C.POINTER(GgufSummary)]),
    "mk_ep_unique_id": (_i32, [P]),
    "mk_model_ep_init": (_i32, [P, P]),
    "mk_model_spec": (_i32, [P, C.POINTER(RuntimeSpec)]),
    "mk_session_new": (_i32, [P, C.POINTER(P)]),
    "mk_session_free": (_i32, [P]),
    "mk_session_fork_prefix": (_i32, [P, P, _i64, C.POINTER(P)]),
    "mk_session_clear": (_i32, [P]),
    "mk_session_len": (_i32, [P, C.POINTER(_i64)]),
    "mk_session_block_table": (_i32, [P, P, P, C.POINTER(_i32)]),
    "mk_reset_session_for_prompt": (_i32, [P, P, P, _i32, C.POINTER(_i64)]),
    "mk_publish_prompt_prefix": (_i32, [P, P, P, _i32]),
    "mk_kv_capacity_query": (_i32, [P, C.POINTER(KvCapacity)]),
    "mk_pool_stats_query": (_i32, [P, C.POINTER(PoolStats)]),
    "mk_prefix_diagnostics_query": (_i32, [P, C.POINTER(PrefixDiagnostics)]),
    "mk_reserve_batch": (_i32, [P, C.POINTER(Lane), _i32, C.POINTER(P)]),
    "mk_reservation_drop": (_i32, [P]),
    "mk_forward_batch_reserved": (_i32, [P, C.POINTER(Lane), _i32, P, _u32]),
    "mk_read_output": (_i32, [P, P, P]),
    "mk_synchronize": (_i32, [P]),
    "mk_last_forward_ms": (_i32, [P, C.POINTER(_f32)]),
    "mk_launch_count": (_i32, [P, C.POINTER(_i64)]),
    "mk_transfer_bytes": (_i32, [P, C.POINTER(_i64), C.POINTER(_i64)]),
    "mk_profile_enable": (_i32, [P, _i32]),
    "mk_profile_query": (_i32, [P, P, C.POINTER(_i32)]),
    "mk_engine_new": (_i32, [P, C.POINTER(EngineConfig), C.POINTER(P)]),
    "mk_engine_free": (_i32, [P]),
    "mk_engine_submit": (_i32, [P, C.POINTER(Request), _i32, _i32, P]),
    "mk_engine_step": (_i32, [P, C.POINTER(_i32)]),
    "mk_engine_run": (_i32, [P]),
    "mk_engine_pending": (_i32, [P, C.POINTER(_i32)]),
    "mk_engine_result": (_i32, [P, _i32, P, C.POINTER(_i32), C.POINTER(_i32), C.POINTER(_i64)]),
    "mk_engine_logits": (_i32, [P, _i32, P, C.POINTER(_i32)]),
    "mk_engine_trace": (_i32, [P, _i64, C.POINTER(TickLane), C.POINTER(_i32)]),
    "mk_engine_stats_query": (_i32, [P, C.POINTER(EngineStats)]),
    "mk_engine_status": (_i32, [P, C.POINTER(_i32)]),
    "mk_engine_failure_kind": (_i32, [P, _i32, C.POINTER(_i32)]),
    "mk_engine_cancel": (_i32, [P, _i32]),
    "mk_engine_step_at": (_i32, [P, C.c_double, C.POINTER(_i32)]),
    "mk_engine_consume_events": (_i32, [P, _i32, _i32]),
    "mk_engine_keep_trace": (_i32, [P, _i32]),
    "mk_engine_release_request": (_i32, [P, _i32]),
    "mk_engine_request_metrics": (_i32, [P, _i32, C.POINTER(RequestMetrics)]),
    "mk_model_fake_script": (_i32, [P, C.c_void_p, _i32, C.c_void_p, _i32]),
    "mk_engine_tick_info": (_i32, [P, _i64, C.POINTER(TickInfo)]),
    "mk_engine_batch_trace": (_i32, [P, _i32, C.POINTER(BatchTrace), C.POINTER(_i64), C.POINTER(_i32)]),
    "mk_kvpool_new": (_i32, [_i32, _i32, _i64, C.POINTER(P)]),
    "mk_kvpool_free": (_i32, [P]),
    "mk_kvpool_stats": (_i32, [P, C.POINTER(PoolStats)]),
    "mk_kvtable_new": (_i32, [P, C.POINTER(P)]),
    "mk_kvtable_free": (_i32, [P]),
    "mk_kvtable_len": (_i32, [P, C.POINTER(_i64)]),
    "mk_kvtable_blocks": (_i32, [P, P, P, C.POINTER(_i32)]),
    "mk_kvtable_clear": (_i32, [P]),
    "mk_kvtable_fork_prefix": (_i32, [P, _i64, C.POINTER(P)]),
    "mk_kvtable_attach_prefix": (_i32, [P, P, _i64]),
    "mk_kvpool_append_batch": (_i32, [P, C.POINTER(P), P, _i32, _i32, P, C.POINTER(_i32)]),
    "mk_kvpool_page_table": (_i32, [P, C.POINTER(P), P, _i32, P, C.POINTER(_i32), P, P, P]),
    "mk_kvpool_submit_epoch": (_i32, [P, C.POINTER(_i64)]),
    "mk_kvpool_complete_epoch": (_i32, [P, _i64]),
    "mk_prefix_cache_new": (_i32, [_i32, _i64, C.POINTER(P)]),
    "mk_prefix_cache_free": (_i32, [P]),
    "mk_prefix_cache_insert": (_i32, [P, P, _i32, _i64, _i64, P, C.POINTER(_i32)]),
    "mk_prefix_cache_lookup": (_i32, [P, P, _i32, C.POINTER(_i64), C.POINTER(_i64)]),
    "mk_prefix_cache_evict_lru": (_i32, [P, C.POINTER(_i64)]),
    "mk_prefix_cache_lookup_bounded": (_i32, [P, _i32, P, _i32, _i64, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "mk_prefix_cache_set_max_cost": (_i32, [P, _i64, P, C.POINTER(_i32)]),
    "mk_prefix_cache_force_collisions": (_i32, [P]),
    "mk_prefix_cache_diagnostics": (_i32, [P, C.POINTER(PrefixDiagnostics)]),
    "mk_prefix_block_digests": (_i32, [_i32, P, _i32, P, C.POINTER(_i32)]),
    "mk_sha256": (_i32, [P, _i64, P]),
    "mk_host_sample_greedy": (_i32, [P, _i32, P, _i32, _f32, P, _i32, _f32, _f32, C.POINTER(_u32)]),
    "mk_seed_tensor": (_i32, [_u64, _u64, _f32, _i32, _i64, _i64, P]),
    "mk_row_bytes": (_i64, [_i32, _i64]),
    "mk_decode_rows": (_i32, [_i32, P, _i64, _i64, P]),
    "mk_unpermute_qk_rows": (_i32, [C.c_void_p, _i64, _i64, _i32, C.c_void_p]),
    "mk_k_quantize": (_i32, [_i32, P, _i32, _i32, P, P, P]),
    "mk_k_add_norm": (_i32, [P, P, _f32, P, P, _f32, _i32, _i32, P]),
    "mk_k_qmatmul": (_i32, [_i32, P, _i64, _i64, P, _i32, P, _i32]),
    "mk_k_qmatmul_time": (_i32, [_i32, P, _i64, _i64, P, _i32, _i32, _i32, C.POINTER(_f32)]),
    "mk_k_q4k_matmul_tc_noalloc_dev": (_i32, [P, _i64, _i64, P, _i32, P, P]),
    "mk_k_embed": (_i32, [_i32, P, _i64, _i64, P, _i32, _f32, P]),
    "mk_k_actmul": (_i32, [P, P, _i32, _i32, _i32, P]),
    "mk_k_moe_combine_exchange": (_i32, [P, P, P, _i32, _i32, _i32, _i32, _i32, _i32, _i32, P, _i32, _i32, _i32, P, P, P]),
    "mk_k_matmul_plan": (_i32, [_i32, _i64, _i64, _i32, _i32, P]),
    "mk_k_attention_plan": (_i32, [P, P, _i32, _i32, _i32, _i32, P, P, P]),
    "mk_k_gated_ffn": (_i32, [_i32, P, P, _i64, _i64, P, _i32, _i32, P, _i32, P]),
    "mk_k_attention_step": (_i32, [C.POINTER(AttnCase)]),
    "mk_k_argmax": (_i32, [P, _i32, _i32, P]),
    "mk_k_gated_delta_decay": (_i32, [P, P, P, _i32, _i32, P]),
    "mk_k_gated_delta_recurrence": (_i32, [P, P, P, P, P, P, _i32, _i32, _i32, _i32, P, P, P]),
    "mk_k_mamba2_scan": (_i32, [P, _i64, P, P, P, P, P, _i32, _i32, _i32, _i32, P, P, P]),
    "mk_k_short_conv": (_i32, [P, P, P, _i32, _i32, _i32, P, P, P]),
    "mk_k_recurrent_time": (_i32, [_i32, _i32, _i32, _i32, _i32, _i32, _i32, C.POINTER(C.c_float), C.POINTER(C.c_double)]),
    "mk_k_grouped_qmatmul": (_i32, [_i32, P, P, _i32, _i64, _i64, P, P, P, _i32, _i32]),
    "mk_k_sample": (_i32, [P, _i32, _i32, P, _i32, P]),
    "mk_k_penalties": (_i32, [P, _i32, P, _i32, C.c_float, P, _i32, C.c_float, C.c_float]),
    "mk_forward_set_sampling": (_i32, [P, P, _i32]),
    "mk_k_moe_route": (_i32, [P, _i32, _i32, _i32, P, P]),
}

_lib = None


def lib() -> C.CDLL:
    """Load the shared library (once) and attach signatures.  Raises when it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise MkError(f"{LIB_PATH} is missing: run `python macllm-infer_b200/build.py` (there is no CPU fallback)")
        handle = C.CDLL(str(LIB_PATH))
        missing = [name for name in SIGNATURES if not hasattr(handle, name)]
        if missing:
            raise MkError(f"{LIB_PATH} does not export {missing}: rebuild it")
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> None:
    if status == MK_OK:
        return
    msg = lib().mk_last_error().decode("utf-8", "replace")
    if status == MK_KV_EXHAUSTED:
        raise KvExhausted(msg)
    raise MkError(msg)
