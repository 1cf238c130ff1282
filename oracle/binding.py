"""ctypes binding for the CPU oracle (``liborion_oracle.so``).

TEST INFRASTRUCTURE ONLY: imported by the test-suite, by the smoke check and by
the CPU-baseline / reference legs of the benchmark. The product package never
imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Callable, Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liborion_oracle.so")

ORACLE_OK = 0
ORACLE_ERR_INTERNAL = 1
ORACLE_ERR_ARG = 2


class OracleInternalError(RuntimeError):
    """The reference's ``EngineError::Internal``."""


class OracleArgError(ValueError):
    pass


def build(force: bool = False) -> str:
    """Compiles the oracle with its Makefile when the library is missing or stale."""
    src = os.path.join(_HERE, "orion_oracle.c")
    hdr = os.path.join(_HERE, "orion_oracle.h")
    stale = (not os.path.exists(_LIB_PATH)) or any(
        os.path.exists(p) and os.path.getmtime(p) > os.path.getmtime(_LIB_PATH) for p in (src, hdr)
    )
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "liborion_oracle.so"], check=True,
                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    return _LIB_PATH


class ModelDesc(C.Structure):
    _fields_ = [
        ("hidden_size", C.c_uint32), ("num_layers", C.c_uint32),
        ("num_attention_heads", C.c_uint32), ("num_kv_heads", C.c_uint32),
        ("head_dim", C.c_uint32), ("vocab_size", C.c_uint32), ("ffn_dim", C.c_uint32),
        ("max_position_embeddings", C.c_uint32), ("rope_theta", C.c_float),
        ("rms_norm_eps", C.c_float), ("has_qkv_bias", C.c_uint32), ("tied_lm_head", C.c_uint32),
        ("num_blocks", C.c_uint32), ("block_size", C.c_uint32),
    ]


_lib = None
ALLREDUCE_FN = C.CFUNCTYPE(None, C.POINTER(C.c_float), C.c_size_t, C.c_void_p)


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        build()
    L = C.CDLL(_LIB_PATH)
    fp, u32p, u64p, u16p = (C.POINTER(C.c_float), C.POINTER(C.c_uint32), C.POINTER(C.c_uint64),
                            C.POINTER(C.c_uint16))
    sz = C.c_size_t
    L.oracle_last_error.restype = C.c_char_p
    L.oracle_set_threads.argtypes = [C.c_int]
    L.oracle_get_threads.restype = C.c_int
    L.oracle_linear.argtypes = [fp, sz, sz, fp, sz, sz, fp, sz, fp]
    L.oracle_rms_norm.argtypes = [fp, sz, sz, fp, sz, C.c_float]
    L.oracle_silu.argtypes = [C.c_float]
    L.oracle_silu.restype = C.c_float
    L.oracle_swiglu.argtypes = [fp, sz, sz, fp, sz, sz]
    L.oracle_softmax_inplace.argtypes = [fp, sz]
    L.oracle_softmax_inplace.restype = None
    L.oracle_rope_table.argtypes = [sz, sz, C.c_float, fp, fp]
    L.oracle_apply_rope.argtypes = [fp, sz, fp, fp, sz]
    L.oracle_kv_new.argtypes = [sz] * 5
    L.oracle_kv_new.restype = C.c_void_p
    L.oracle_kv_free.argtypes = [C.c_void_p]
    L.oracle_kv_free.restype = None
    L.oracle_kv_len.argtypes = [C.c_void_p]
    L.oracle_kv_len.restype = sz
    L.oracle_kv_data.argtypes = [C.c_void_p]
    L.oracle_kv_data.restype = fp
    L.oracle_kv_write.argtypes = [C.c_void_p, sz, C.c_uint32, sz, sz, C.c_int, fp, sz]
    L.oracle_kv_read.argtypes = [C.c_void_p, sz, C.c_uint32, sz, sz, C.c_int, fp]
    L.oracle_locate.argtypes = [u32p, sz, sz, sz, u32p, C.POINTER(sz)]
    L.oracle_paged_attention.argtypes = [C.c_void_p, fp, sz, u32p, sz, sz, sz, sz, sz, sz, sz, fp,
                                         sz]
    L.oracle_argmax.argtypes = [fp, sz]
    L.oracle_argmax.restype = C.c_int64
    L.oracle_bf16_to_f32.argtypes = [u16p, sz, fp]
    L.oracle_bf16_to_f32.restype = None
    L.oracle_f16_to_f32.argtypes = [u16p, sz, fp]
    L.oracle_f16_to_f32.restype = None
    L.oracle_f32_to_bf16.argtypes = [fp, sz, u16p]
    L.oracle_f32_to_bf16.restype = None
    L.oracle_model_new.argtypes = [C.POINTER(ModelDesc)]
    L.oracle_model_new.restype = C.c_void_p
    L.oracle_model_free.argtypes = [C.c_void_p]
    L.oracle_model_free.restype = None
    L.oracle_model_set_tensor.argtypes = [C.c_void_p, C.c_char_p, fp, sz]
    L.oracle_model_kv.argtypes = [C.c_void_p]
    L.oracle_model_kv.restype = C.c_void_p
    L.oracle_model_forward.argtypes = [C.c_void_p, u32p, u32p, sz, u64p, u64p, u32p, u64p, sz, sz,
                                       sz, sz, sz, fp]
    L.oracle_model_forward_tp.argtypes = [C.c_void_p, C.c_uint32, C.c_uint32, ALLREDUCE_FN,
                                          C.c_void_p, u32p, u32p, sz, u64p, u64p, u32p, u64p, sz,
                                          fp]
    _lib = L
    return L


def _check(rc: int) -> None:
    if rc == ORACLE_OK:
        return
    msg = lib().oracle_last_error().decode("utf-8", "replace")
    if rc == ORACLE_ERR_INTERNAL:
        raise OracleInternalError(msg)
    raise OracleArgError(msg)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: np.ndarray, ctype):
    return a.ctypes.data_as(C.POINTER(ctype))


def set_threads(n: int) -> None:
    lib().oracle_set_threads(int(n))


# ---- tensor.rs -------------------------------------------------------------

def linear(x, w, bias=None) -> np.ndarray:
    x, w = _f32(x), _f32(w)
    n, k = x.shape
    out_f, in_f = w.shape
    out = np.zeros((n, out_f), np.float32)
    b = _f32(bias) if bias is not None else None
    _check(lib().oracle_linear(_ptr(x, C.c_float), n, k, _ptr(w, C.c_float), out_f, in_f,
                               _ptr(b, C.c_float) if b is not None else None,
                               b.size if b is not None else 0, _ptr(out, C.c_float)))
    return out


def rms_norm(x, weight, eps: float) -> np.ndarray:
    x = _f32(x).copy()
    w = _f32(weight)
    rows, cols = x.shape
    _check(lib().oracle_rms_norm(_ptr(x, C.c_float), rows, cols, _ptr(w, C.c_float), w.size, eps))
    return x


def silu(x: float) -> float:
    return float(lib().oracle_silu(x))


def swiglu(gate, up) -> np.ndarray:
    g, u = _f32(gate).copy(), _f32(up)
    _check(lib().oracle_swiglu(_ptr(g, C.c_float), g.shape[0], g.shape[1], _ptr(u, C.c_float),
                               u.shape[0], u.shape[1]))
    return g


def softmax(x) -> np.ndarray:
    x = _f32(x).copy()
    lib().oracle_softmax_inplace(_ptr(x, C.c_float), x.size)
    return x


def rope_table(head_dim: int, max_positions: int, theta: float):
    half = head_dim // 2
    cos = np.zeros((max_positions, half), np.float32)
    sin = np.zeros((max_positions, half), np.float32)
    _check(lib().oracle_rope_table(head_dim, max_positions, theta, _ptr(cos, C.c_float),
                                   _ptr(sin, C.c_float)))
    return cos, sin


def apply_rope(vec, cos_row, sin_row) -> np.ndarray:
    v, c, s = _f32(vec).copy(), _f32(cos_row), _f32(sin_row)
    if c.size != s.size:
        raise OracleInternalError("cos/sin width mismatch")
    _check(lib().oracle_apply_rope(_ptr(v, C.c_float), v.size, _ptr(c, C.c_float),
                                   _ptr(s, C.c_float), c.size))
    return v


def argmax(logits) -> Optional[int]:
    a = _f32(logits)
    i = int(lib().oracle_argmax(_ptr(a, C.c_float), a.size))
    return None if i < 0 else i


def bf16_to_f32(bits) -> np.ndarray:
    b = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.zeros(b.shape, np.float32)
    lib().oracle_bf16_to_f32(_ptr(b, C.c_uint16), b.size, _ptr(out, C.c_float))
    return out


def f16_to_f32(bits) -> np.ndarray:
    b = np.ascontiguousarray(bits, dtype=np.uint16)
    out = np.zeros(b.shape, np.float32)
    lib().oracle_f16_to_f32(_ptr(b, C.c_uint16), b.size, _ptr(out, C.c_float))
    return out


def f32_to_bf16(x) -> np.ndarray:
    a = _f32(x)
    out = np.zeros(a.shape, np.uint16)
    lib().oracle_f32_to_bf16(_ptr(a, C.c_float), a.size, _ptr(out, C.c_uint16))
    return out


def round_to_bf16(x) -> np.ndarray:
    """f32 values rounded to the nearest bf16 and widened back."""
    return bf16_to_f32(f32_to_bf16(x))


# ---- attention.rs ------------------------------------------------------------

def locate(table: Sequence[int], position: int, block_size: int):
    t = np.ascontiguousarray(table, dtype=np.uint32)
    blk, slot = C.c_uint32(0), C.c_size_t(0)
    ok = lib().oracle_locate(_ptr(t, C.c_uint32), t.size, position, block_size, C.byref(blk),
                             C.byref(slot))
    return (blk.value, slot.value) if ok else None


class KvStore:
    def __init__(self, num_layers, num_blocks, block_size, num_kv_heads, head_dim, _handle=None):
        self.shape = (num_layers, num_blocks, 2, block_size, num_kv_heads, head_dim)
        self.head_dim = head_dim
        self._owned = _handle is None
        self._h = _handle or lib().oracle_kv_new(num_layers, num_blocks, block_size, num_kv_heads,
                                                 head_dim)
        if not self._h:
            raise MemoryError("oracle_kv_new failed")

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "_h", None):
            lib().oracle_kv_free(self._h)
            self._h = None

    def __len__(self):
        return int(lib().oracle_kv_len(self._h))

    def array(self) -> np.ndarray:
        """The arena as a numpy view ``[layer][block][k|v][slot][head][dim]``."""
        p = lib().oracle_kv_data(self._h)
        return np.ctypeslib.as_array(p, shape=(len(self),)).reshape(self.shape)

    def write(self, layer, block, slot, head, is_value, vector):
        v = _f32(vector)
        _check(lib().oracle_kv_write(self._h, layer, block, slot, head, int(bool(is_value)),
                                     _ptr(v, C.c_float), v.size))

    def read(self, layer, block, slot, head, is_value) -> np.ndarray:
        out = np.zeros(self.head_dim, np.float32)
        _check(lib().oracle_kv_read(self._h, layer, block, slot, head, int(bool(is_value)),
                                    _ptr(out, C.c_float)))
        return out


def paged_attention(store: KvStore, query, block_table, query_position, layer, num_query_heads,
                    num_kv_heads, head_dim, block_size) -> np.ndarray:
    q = _f32(query)
    t = np.ascontiguousarray(block_table, dtype=np.uint32)
    out = np.zeros(q.size, np.float32)
    _check(lib().oracle_paged_attention(store._h, _ptr(q, C.c_float), q.size, _ptr(t, C.c_uint32),
                                        t.size, query_position, layer, num_query_heads,
                                        num_kv_heads, head_dim, block_size, _ptr(out, C.c_float),
                                        out.size))
    return out


# ---- transformer.rs ----------------------------------------------------------

@dataclass
class Batch:
    """Mirror of ``ForwardBatch`` (orion-core/src/traits.rs:193-210) for the oracle."""
    tokens: Sequence[int]
    positions: Sequence[int]
    slot_token_counts: Sequence[int]
    context_lens: Sequence[int]
    block_tables: Sequence[Sequence[int]]
    sequence_ids: Optional[Sequence[int]] = None
    has_prefill: bool = True

    def flat(self):
        tokens = np.ascontiguousarray(self.tokens, dtype=np.uint32)
        positions = np.ascontiguousarray(self.positions, dtype=np.uint32)
        counts = np.ascontiguousarray(self.slot_token_counts, dtype=np.uint64)
        ctx = np.ascontiguousarray(self.context_lens, dtype=np.uint64)
        offs = np.zeros(len(self.block_tables) + 1, np.uint64)
        for i, t in enumerate(self.block_tables):
            offs[i + 1] = offs[i] + len(t)
        flat = np.zeros(max(int(offs[-1]), 1), np.uint32)
        for i, t in enumerate(self.block_tables):
            flat[int(offs[i]):int(offs[i + 1])] = np.asarray(t, dtype=np.uint32)
        return tokens, positions, counts, ctx, flat, offs


class Model:
    """Oracle ``TransformerModel`` (transformer.rs:137-205)."""

    def __init__(self, *, hidden_size, num_layers, num_attention_heads, num_kv_heads, head_dim,
                 vocab_size, ffn_dim, max_position_embeddings=2048, rope_theta=10000.0,
                 rms_norm_eps=1e-5, has_qkv_bias=False, tied_lm_head=False, num_blocks=16,
                 block_size=16):
        self.desc = ModelDesc(hidden_size, num_layers, num_attention_heads, num_kv_heads, head_dim,
                              vocab_size, ffn_dim, max_position_embeddings, rope_theta,
                              rms_norm_eps, int(has_qkv_bias), int(tied_lm_head), num_blocks,
                              block_size)
        self.vocab_size = vocab_size
        self._h = lib().oracle_model_new(C.byref(self.desc))
        if not self._h:
            raise MemoryError("oracle_model_new failed")

    def __del__(self):
        if getattr(self, "_h", None):
            lib().oracle_model_free(self._h)
            self._h = None

    def set_tensor(self, name: str, data) -> None:
        a = _f32(data)
        _check(lib().oracle_model_set_tensor(self._h, name.encode(), _ptr(a, C.c_float), a.size))

    def load(self, tensors: dict) -> "Model":
        for name, data in tensors.items():
            self.set_tensor(name, data)
        return self

    def kv(self) -> KvStore:
        d = self.desc
        return KvStore(d.num_layers, d.num_blocks, d.block_size, d.num_kv_heads, d.head_dim,
                       _handle=lib().oracle_model_kv(self._h))

    def forward(self, batch: Batch) -> np.ndarray:
        tokens, positions, counts, ctx, flat, offs = batch.flat()
        n_seq = len(batch.sequence_ids) if batch.sequence_ids is not None else len(
            batch.slot_token_counts)
        logits = np.zeros((n_seq, self.vocab_size), np.float32)
        _check(lib().oracle_model_forward(
            self._h, _ptr(tokens, C.c_uint32), _ptr(positions, C.c_uint32), tokens.size,
            _ptr(counts, C.c_uint64), _ptr(ctx, C.c_uint64), _ptr(flat, C.c_uint32),
            _ptr(offs, C.c_uint64), n_seq, counts.size, ctx.size, len(batch.block_tables),
            positions.size, _ptr(logits, C.c_float)))
        if tokens.size == 0:
            return logits[:0]
        return logits

    def forward_tp(self, batch: Batch, rank: int, world: int,
                   allreduce: Callable[[np.ndarray], None]) -> np.ndarray:
        tokens, positions, counts, ctx, flat, offs = batch.flat()
        n_seq = len(batch.slot_token_counts)
        logits = np.zeros((n_seq, self.vocab_size), np.float32)

        def _cb(ptr, n, _ctx):
            allreduce(np.ctypeslib.as_array(ptr, shape=(n,)))

        cb = ALLREDUCE_FN(_cb)
        _check(lib().oracle_model_forward_tp(
            self._h, rank, world, cb, None, _ptr(tokens, C.c_uint32), _ptr(positions, C.c_uint32),
            tokens.size, _ptr(counts, C.c_uint64), _ptr(ctx, C.c_uint64), _ptr(flat, C.c_uint32),
            _ptr(offs, C.c_uint64), n_seq, _ptr(logits, C.c_float)))
        return logits
