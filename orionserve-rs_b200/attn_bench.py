"""Device-resident paged GQA decode-attention microbenchmark (bf16, block 16, head_dim 128):
blocks drawn from a permutation of a large pool, ragged contexts, N(0,1) values."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np

from . import _ffi
from .backend import CudaBackend
from .errors import check


class PagedAttentionBench:
    def __init__(self, backend: CudaBackend, context_lens: Sequence[int], *, num_query_heads: int = 32,
                 num_kv_heads: int = 8, head_dim: int = 128, block_size: int = 16,
                 num_blocks: int = 200_000, seed: int = 0):
        self.context_lens = np.ascontiguousarray(context_lens, dtype=np.uint64)
        self.batch = int(self.context_lens.size)
        self.q_heads, self.kv_heads, self.head_dim, self.block_size = (num_query_heads, num_kv_heads,
                                                                      head_dim, block_size)
        self.num_blocks = num_blocks
        rng = np.random.default_rng(seed)
        need =int(((self.context_lens + block_size - 1) // block_size).sum())
        if need > num_blocks:
            raise ValueError(f"{need} blocks needed, pool has {num_blocks}")
        # each sequence's table is a consecutive slice of one random permutation of the pool
        self.block_ids = np.ascontiguousarray(rng.permutation(num_blocks)[:need], dtype=np.uint32)
        self._h = C.c_void_p()
        check(_ffi.lib().orion_cuda_attn_bench_create(
            backend._h, num_query_heads, num_kv_heads, head_dim, block_size, num_blocks,
            self.block_ids.ctypes.data_as(C.POINTER(C.c_uint32)),
            self.context_lens.ctypes.data_as(C.POINTER(C.c_uint64)), self.batch, seed, C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            _ffi.lib().orion_cuda_attn_bench_destroy(self._h)
            self._h = None

    def run(self, warmup: int = 3, iterations: int = 20):
        """Returns (mean ms per launch, algorithmic bytes per launch)."""
        ms, nbytes = C.c_float(), C.c_uint64()
        check(_ffi.lib().orion_cuda_attn_bench_run(self._h, warmup, iterations, C.byref(ms), C.byref(nbytes)))
        return ms.value, nbytes.value

    def device_views(self) -> dict:
        """Device addresses (ints) of the benchmark's inputs; valid while this object lives."""
        ptrs = [C.c_void_p() for _ in range(6)]
        max_pos = C.c_uint32()
        check(_ffi.lib().orion_cuda_attn_bench_device_views(self._h, *[C.byref(p) for p in ptrs],
                                                            C.byref(max_pos)))
        names = ("q", "kv_arena", "query_positions", "seq_of_row", "block_tables_flat", "block_table_offsets")
        views = {n: p.value for n, p in zip(names, ptrs)}
        views["max_position"] = max_pos.value
        return views

    def output(self) -> np.ndarray:
        out = np.zeros((self.batch, self.q_heads, self.head_dim), np.float32)
        check(_ffi.lib().orion_cuda_attn_bench_output(self._h, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def sequence(self, seq: int):
        """(q [heads, dim], k [ctx, kv heads, dim], v likewise) of one sequence, widened to f32."""
        ctx = int(self.context_lens[seq])
        q = np.zeros((self.q_heads, self.head_dim), np.float32)
        k = np.zeros((ctx, self.kv_heads, self.head_dim), np.float32)
        v = np.zeros_like(k)
        F = C.POINTER(C.c_float)
        check(_ffi.lib().orion_cuda_attn_bench_sequence(self._h, seq, q.ctypes.data_as(F), k.ctypes.data_as(F),
                                                       v.ctypes.data_as(F)))
        return q, k, v
