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

ORION_OK, ERR_INTERNAL, ERR_BACKEND, ERR_INVALID_REQUEST, ERR_UNAVAILABLE, ERR_MODEL = range(6)
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
    "orion_cuda_set_l2_prefetch_bytes": (_int, [_u64]),
    "orion_cuda_attention_set_tuning": (_int, [_int, _u32]),
    "orion_cuda_tp_layout": (_int, [_u32, _u32, _u32, _u32, _u32, _u64p, _u64p, _u64p]),
    "orion_cuda_tp_unique_id": (_int, [_u8p]),
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
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError here means the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def last_error() -> str:
    return lib().orion_cuda_last_error().decode("utf-8", "replace")
