"""ctypes declarations for ``liborion_cuda.so`` (see ``include/orion_cuda.h``).

There is no fallback: if the shared library is missing, importing the package
works (so that the host-side logic can be tested) but the first call that
needs the device raises ``CudaLibraryMissing``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liborion_cuda.so")
HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "orion_cuda.h")

DRIVER_HEADER_PATH = os.path.join(os.path.dirname(_HERE), "include", "orion_driver.h")

(ORION_OK, ERR_INTERNAL, ERR_BACKEND, ERR_INVALID_REQUEST, ERR_UNAVAILABLE, ERR_MODEL, ERR_CONTEXT_LENGTH,
 ERR_QUEUE_FULL, ERR_CACHE_EXHAUSTED) = range(9)
NCCL_ID_BYTES = 128


class CudaLibraryMissing(RuntimeError):
    pass


class OrionModelDesc(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_uint32), ("num_layers", C.c_uint32),
        ("num_attention_heads", C.c_uint32), ("num_kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32), ("vocab_size", C.c_uint32), ("ffn_dim", C.c_uint32),
        ("max_position_embeddings", C.c_uint32), ("rope_theta", C.c_float),
        ("rms_norm_eps", C.c_float), ("has_qkv_bias", C.c_uint32), ("tied_lm_head", C.c_uint32),
        ("num_blocks", C.c_uint32), ("block_size", C.c_uint32), ("compute_dtype", C.c_uint32),
        ("max_batch_tokens", C.c_uint32), ("max_batch_sequences", C.c_uint32),
        ("tp_rank", C.c_uint32), ("tp_world", C.c_uint32),
        ("nccl_unique_id", C.c_uint8 * NCCL_ID_BYTES),
    ]


_lib = None

_f32p, _u32p, _u64p, _u8p = (C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64),
                             C.POINTER(C.c_uint8))
_vp, _u64, _u32, _int = C.c_void_p, C.c_uint64, C.c_uint32, C.c_int
_BATCH = [_u32p, _u64, _u32p, _u64, _u64p, _u64, _u64p, _u64, _u32p, _u64p, _u64, _u64, _int]

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "orion_cuda_last_error": (C.c_char_p, []),
    "orion_cuda_is_available": (_int, []),
    "orion_cuda_device_count": (_int, []),
    "orion_cuda_backend_create": (_int, [_int, C.POINTER(_vp)]),
    "orion_cuda_backend_destroy": (None, [_vp]),
    "orion_cuda_backend_name": (C.c_char_p, [_vp]),
    "orion_cuda_backend_ordinal": (_int, [_vp]),
    "orion_cuda_backend_device_name": (C.c_char_p, [_vp]),
    "orion_cuda_backend_total_memory": (_int, [_vp, _u64p]),
    "orion_cuda_backend_available_memory": (_int, [_vp, _u64p]),
    "orion_cuda_backend_synchronize": (_int, [_vp]),
    "orion_cuda_backend_supports_dtype": (_int, [_vp, _int]),
    "orion_cuda_model_create": (_int, [_vp, C.POINTER(OrionModelDesc), C.POINTER(_vp)]),
    "orion_cuda_model_destroy": (None, [_vp]),
    "orion_cuda_model_load_tensor": (_int, [_vp, C.c_char_p, _int, _u64p, _int, _vp]),
    "orion_cuda_model_finalize": (_int, [_vp]),
    "orion_cuda_model_init_random": (_int, [_vp, _u64, C.c_float]),
    "orion_cuda_model_forward": (_int, [_vp, *_BATCH, _vp, _u64]),
    "orion_cuda_model_forward_greedy": (_int, [_vp, *_BATCH, _u32p, _vp, _u64]),
    "orion_cuda_model_load_checkpoint": (_int, [_vp, C.c_char_p, C.POINTER(C.c_uint64)]),
    "orion_cuda_poll_wait_timeouts": (_int, [_vp, C.POINTER(C.c_uint32)]),
    "orion_cuda_selftest_peer_wait": (_int, [_vp, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "orion_cuda_selftest_bounded_wait": (_int, [_vp, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]),
    "orion_cuda_model_replay": (_int, [_vp, _int, _f32p]),
    "orion_cuda_model_replay_categories": (_int, [_vp, _int, C.c_uint32, _f32p]),
    "orion_cuda_model_profile": (_int, [_vp, _int, _f32p, _u64p]),
    "orion_cuda_model_fill_kv_random": (_int, [_vp, _u64, C.c_float]),
    "orion_cuda_model_last_launch_count": (_int, [_vp, _u64p]),
    "orion_cuda_model_read_kv": (_int, [_vp, _f32p, _u64]),
    "orion_cuda_model_desc": (_int, [_vp, C.POINTER(OrionModelDesc)]),
    "orion_cuda_host_alloc": (_vp, [_u64]),
    "orion_cuda_host_free": (None, [_vp]),
    "orion_cuda_gemm_set_tuning": (_int, [_u32, _int]),
    "orion_cuda_set_programmatic_launch": (_int, [_int]),
    "orion_cuda_attention_set_tuning": (_int, [_int, _u32]),
    "orion_cuda_tp_layout": (_int, [_u32, _u32, _u32, _u32, _u32, _u64p, _u64p, _u64p]),
    "orion_cuda_tp_unique_id": (_int, [_u8p]),
    "orion_cuda_collective_create": (_int, [_vp, _u8p, _u32, _u32, C.POINTER(_vp)]),
    "orion_cuda_collective_destroy": (None, [_vp]),
    "orion_cuda_collective_all_reduce_sum": (_int, [_vp, _f32p, _u64]),
    "orion_cuda_collective_all_gather": (_int, [_vp, _f32p, _u64, _f32p]),
    "orion_cuda_collective_reduce_scatter_sum": (_int, [_vp, _f32p, _u64, _f32p]),
    "orion_cuda_collective_barrier": (_int, [_vp]),
    "orion_cuda_tp_selftest_failure_handling": (_int, [_int, _u64, C.POINTER(C.c_uint32), _u64p]),
    "orion_cuda_linear": (_int, [_vp, _int, _f32p, _u64, _u64, _f32p, _u64, _u64, _f32p, _u64, _f32p]),
    "orion_cuda_linear_bench": (_int, [_vp, _u64, _u64, _u64, _int, _int, _f32p, C.POINTER(_u32)]),
    "orion_cuda_rms_norm": (_int, [_vp, _int, _f32p, _u64, _u64, _f32p, _u64, C.c_float]),
    "orion_cuda_swiglu": (_int, [_vp, _int, _f32p, _u64, _u64, _f32p, _u64, _u64]),
    "orion_cuda_rope": (_int, [_vp, _int, _f32p, _u64, _u64, _u64, _u32p, _u64, C.c_float]),
    "orion_cuda_paged_attention": (_int, [_vp, _int, _f32p, _u64, _u64, _u64, _u64, _f32p, _u64, _u64,
                                          _u32p, _u32p, _u32p, _u64p, _u64, _f32p]),
    "orion_cuda_argmax": (_int, [_vp, _f32p, _u64, _u64, _u32p]),
    "orion_cuda_attn_bench_create": (_int, [_vp, _u32, _u32, _u32, _u32, _u64, _u32p, _u64p, _u32, _u64,
                                            C.POINTER(_vp)]),
    "orion_cuda_attn_bench_run": (_int, [_vp, _int, _int, _f32p, _u64p]),
    "orion_cuda_attn_bench_output": (_int, [_vp, _f32p]),
    "orion_cuda_attn_bench_sequence": (_int, [_vp, _u32, _f32p, _f32p, _f32p]),
    "orion_cuda_attn_bench_device_views": (_int, [_vp, C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                                  C.POINTER(_vp), C.POINTER(_vp), C.POINTER(_vp),
                                                  C.POINTER(_u32)]),
    "orion_cuda_attn_bench_destroy": (None, [_vp]),
    "orion_cuda_paged_decode_attention_noalloc": (_int, [_int, _vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp,
                                                         _vp, _u32, _u32, _u32, _vp, _vp]),
}


class OrionAllocationOutcome(C.Structure):
    _fields_ = [("allocated", C.c_uint64), ("reused", C.c_uint64), ("cached_tokens", C.c_uint64)]


class OrionCacheStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("total_blocks", "used_blocks", "free_blocks", "block_size", "num_sequences",
                                          "prefix_cache_entries", "prefix_cache_hits", "prefix_cache_misses")]


class OrionSchedulerConfig(C.Structure):
    _fields_ = [("max_num_seqs", C.c_uint64), ("max_num_batched_tokens", C.c_uint64), ("max_model_len", C.c_uint64),
                ("enable_chunked_prefill", C.c_uint32), ("max_waiting_requests", C.c_uint64),
                ("request_timeout_secs", C.c_uint64), ("prioritize_decode", C.c_uint32),
                ("skip_cached_prefix", C.c_uint32), ("logical_decode_positions", C.c_uint32)]


class OrionSamplingParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("repetition_penalty", C.c_float),
                ("top_k", C.c_uint64), ("max_tokens", C.c_uint64), ("min_tokens", C.c_uint64),
                ("stop_token_ids", C.POINTER(C.c_uint32)), ("num_stop_token_ids", C.c_uint64)]


class OrionScheduledSequence(C.Structure):
    _fields_ = [("id", C.c_uint64), ("num_tokens", C.c_uint64), ("start_position", C.c_uint64),
                ("is_prefill", C.c_uint32)]


class OrionSchedulerStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("total_steps", "total_admitted", "total_finished", "total_preempted",
                                          "total_rejected", "total_batched_tokens", "total_prefill_tokens",
                                          "total_decode_tokens", "total_skipped_prefill_tokens")]


class OrionEngineEvent(C.Structure):
    _fields_ = [("id", C.c_uint64), ("kind", C.c_uint32), ("token", C.c_uint32), ("index", C.c_uint64),
                ("reason", C.c_uint32), ("prompt_tokens", C.c_uint64), ("completion_tokens", C.c_uint64)]


_u64 = C.c_uint64
_u32p, _u64p = C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)
FORWARD_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, _u32p, _u64, _u32p, _u64p, _u64p, _u64p, _u32p, _u64p, _u64, C.c_int,
                         _u32p)

# include/orion_driver.h
DRIVER_SIGNATURES = {
    "orion_hash_block": (_u64, [C.c_int, _u64, _u32p, _u64]),
    "orion_sequence_id_peek": (_u64, []),
    "orion_kv_manager_create": (C.c_void_p, [_u64, _u64, C.c_int]),
    "orion_kv_manager_destroy": (None, [C.c_void_p]),
    "orion_kv_manager_allocate": (C.c_int, [C.c_void_p, _u64, _u32p, _u64, C.POINTER(OrionAllocationOutcome)]),
    "orion_kv_manager_commit_prefill": (None, [C.c_void_p, _u64, _u32p, _u64]),
    "orion_kv_manager_append_token": (C.c_int, [C.c_void_p, _u64]),
    "orion_kv_manager_free": (None, [C.c_void_p, _u64]),
    "orion_kv_manager_preempt": (_u64, [C.c_void_p, _u64]),
    "orion_kv_manager_stats": (C.c_int, [C.c_void_p, C.POINTER(OrionCacheStats)]),
    "orion_kv_manager_can_allocate": (C.c_int, [C.c_void_p, _u64]),
    "orion_kv_manager_blocks_needed_for": (_u64, [C.c_void_p, _u64]),
    "orion_kv_manager_evict_cached": (_u64, [C.c_void_p, _u64]),
    "orion_kv_manager_clear_prefix_cache": (None, [C.c_void_p]),
    "orion_kv_manager_num_evictable": (_u64, [C.c_void_p]),
    "orion_kv_manager_block_table": (C.c_int, [C.c_void_p, _u64, _u32p, _u64, _u64p, _u64p]),
    "orion_kv_manager_block_info": (C.c_int, [C.c_void_p, C.c_uint32, _u32p, _u64p, C.POINTER(C.c_int), _u64p]),
    "orion_kv_manager_fail_next": (None, [C.c_void_p, C.c_int]),
    "orion_scheduler_create": (C.c_void_p, [C.POINTER(OrionSchedulerConfig), _u64, _u64, C.c_int]),
    "orion_scheduler_destroy": (None, [C.c_void_p]),
    "orion_scheduler_cache": (C.c_void_p, [C.c_void_p]),
    "orion_scheduler_add_request": (C.c_int, [C.c_void_p, _u32p, _u64, C.POINTER(OrionSamplingParams), _u64p]),
    "orion_scheduler_cancel": (C.c_int, [C.c_void_p, _u64]),
    "orion_scheduler_schedule": (C.c_int, [C.c_void_p, C.POINTER(OrionScheduledSequence), _u64, _u64p, _u64p, _u64,
                                           _u64p]),
    "orion_scheduler_on_token": (C.c_int, [C.c_void_p, _u64, C.c_uint32, _u32p, _u64]),
    "orion_scheduler_reap_finished": (_u64, [C.c_void_p, _u64p, _u64]),
    "orion_scheduler_commit_prefill": (None, [C.c_void_p, _u64]),
    "orion_scheduler_num_waiting": (_u64, [C.c_void_p]),
    "orion_scheduler_num_running": (_u64, [C.c_void_p]),
    "orion_scheduler_stats": (C.c_int, [C.c_void_p, C.POINTER(OrionSchedulerStats)]),
    "orion_scheduler_running_sequence": (C.c_int, [C.c_void_p, _u64, C.POINTER(C.c_int), _u64p, _u64p]),
    "orion_engine_create": (C.c_void_p, [C.c_void_p, FORWARD_FN, C.c_void_p, C.POINTER(OrionSchedulerConfig), _u64,
                                         _u64, C.c_int, _u32p, _u64]),
    "orion_engine_destroy": (None, [C.c_void_p]),
    "orion_engine_scheduler": (C.c_void_p, [C.c_void_p]),
    "orion_engine_submit": (C.c_int, [C.c_void_p, _u32p, _u64, C.POINTER(OrionSamplingParams), _u64p]),
    "orion_engine_cancel": (None, [C.c_void_p, _u64]),
    "orion_engine_has_work": (C.c_int, [C.c_void_p]),
    "orion_engine_step": (C.c_int, [C.c_void_p, _u64p]),
    "orion_engine_take_events": (_u64, [C.c_void_p, C.POINTER(OrionEngineEvent), _u64]),
    "orion_engine_num_active": (_u64, [C.c_void_p]),
    "orion_engine_last_batch": (C.c_int, [C.c_void_p, C.POINTER(_u32p), _u64p, C.POINTER(_u32p), C.POINTER(_u64p),
                                          C.POINTER(_u64p), C.POINTER(_u64p), C.POINTER(_u32p), C.POINTER(_u64p),
                                          _u64p, C.POINTER(C.c_int)]),
}


def lib() -> C.CDLL:
    """Loads the shared library, declaring every entry point; raises if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise CudaLibraryMissing(
            f"{LIB_PATH} is not built; run `python -c 'import __graft_entry__ as g; g.build()'`. "
            "There is no CPU fallback for the forward path.")
    L = C.CDLL(LIB_PATH)
    for name, (res, args) in list(SIGNATURES.items()) + list(DRIVER_SIGNATURES.items()):
        fn = getattr(L, name)  # AttributeError here means the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def last_error() -> str:
    return lib().orion_cuda_last_error().decode("utf-8", "replace")
