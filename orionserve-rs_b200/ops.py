"""Op-level entry points: the functions of tensor.rs / attention.rs / sampling.rs run on the
GPU through the same kernels the model uses (host arrays in, host arrays out)."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _ffi
from .backend import CudaBackend
from .errors import check
from .types import DType

_F = C.POINTER(C.c_float)
_U32 = C.POINTER(C.c_uint32)
_U64 = C.POINTER(C.c_uint64)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def linear(backend: CudaBackend, x, weight, bias=None, dtype: DType = DType.F32) -> np.ndarray:
    """tensor::linear (tensor.rs:96-130)."""
    x, w = _f32(x), _f32(weight)
    out = np.zeros((x.shape[0], w.shape[0]), np.float32)
    b = _f32(bias) if bias is not None else None
    check(_ffi.lib().orion_cuda_linear(backend._h, int(dtype), x.ctypes.data_as(_F), x.shape[0], x.shape[1],
                                       w.ctypes.data_as(_F), w.shape[0], w.shape[1],
                                       b.ctypes.data_as(_F) if b is not None else None,
                                       b.size if b is not None else 0, out.ctypes.data_as(_F)))
    return out


def rms_norm(backend: CudaBackend, x, weight, eps: float, dtype: DType = DType.F32) -> np.ndarray:
    """tensor::rms_norm (tensor.rs:143-163)."""
    x, w = _f32(x).copy(), _f32(weight)
    check(_ffi.lib().orion_cuda_rms_norm(backend._h, int(dtype), x.ctypes.data_as(_F), x.shape[0], x.shape[1],
                                         w.ctypes.data_as(_F), w.size, eps))
    return x


def swiglu(backend: CudaBackend, gate, up, dtype: DType = DType.F32) -> np.ndarray:
    """tensor::swiglu (tensor.rs:175-189)."""
    g, u = _f32(gate).copy(), _f32(up)
    check(_ffi.lib().orion_cuda_swiglu(backend._h, int(dtype), g.ctypes.data_as(_F), g.shape[0], g.shape[1],
                                       u.ctypes.data_as(_F), u.shape[0], u.shape[1]))
    return g


def rope(backend: CudaBackend, x, positions, max_positions: int, theta: float,
         dtype: DType = DType.F32) -> np.ndarray:
    """RopeTable::new + apply_rope over ``[rows, heads, head_dim]`` (tensor.rs:228-298)."""
    x = _f32(x).copy()
    pos = np.ascontiguousarray(positions, dtype=np.uint32)
    rows, heads, hd = x.shape
    check(_ffi.lib().orion_cuda_rope(backend._h, int(dtype), x.ctypes.data_as(_F), rows, heads, hd,
                                     pos.ctypes.data_as(_U32), max_positions, theta))
    return x


def paged_attention(backend: CudaBackend, kv, query, query_positions, seq_of_row,
                    block_tables: Sequence[Sequence[int]], dtype: DType = DType.F32) -> np.ndarray:
    """attention::paged_attention for a batch of query rows (attention.rs:219-295).
    ``kv``: ``[block][k|v][slot][head][dim]`` of one layer; ``query``: ``[rows][heads][dim]``."""
    kv, q = _f32(kv), _f32(query)
    nb, _, bs, kvh, hd = kv.shape
    rows, qh, _ = q.shape
    pos = np.ascontiguousarray(query_positions, dtype=np.uint32)
    seq = np.ascontiguousarray(seq_of_row, dtype=np.uint32)
    offs = np.zeros(len(block_tables) + 1, np.uint64)
    for i, t in enumerate(block_tables):
        offs[i + 1] = offs[i] + len(t)
    flat = np.zeros(max(int(offs[-1]), 1), np.uint32)
    for i, t in enumerate(block_tables):
        flat[int(offs[i]):int(offs[i + 1])] = np.asarray(t, dtype=np.uint32)
    out = np.zeros_like(q)
    check(_ffi.lib().orion_cuda_paged_attention(
        backend._h, int(dtype), kv.ctypes.data_as(_F), nb, bs, kvh, hd, q.ctypes.data_as(_F), rows, qh,
        pos.ctypes.data_as(_U32), seq.ctypes.data_as(_U32), flat.ctypes.data_as(_U32),
        offs.ctypes.data_as(_U64), len(block_tables), out.ctypes.data_as(_F)))
    return out


def argmax(backend: CudaBackend, logits) -> np.ndarray:
    """sampling::argmax per row (sampling.rs:196-206); 0xFFFFFFFF where no value exceeds -inf."""
    l = _f32(logits)
    if l.ndim == 1:
        l = l[None]
    out = np.zeros(l.shape[0], np.uint32)
    check(_ffi.lib().orion_cuda_argmax(backend._h, l.ctypes.data_as(_F), l.shape[0], l.shape[1],
                                       out.ctypes.data_as(_U32)))
    return out
