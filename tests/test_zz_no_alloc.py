"""Decode attention for callers that cannot allocate device memory (B200 only).

Some users of this library reach attention at a point where they may not call
cudaMalloc: while a stream is being captured into a CUDA graph, inside a serving
loop whose memory all belongs to an external pool, or as a plugin that receives
buffers and a stream and nothing else. ``orion_cuda_paged_decode_attention_noalloc``
serves them: same kernel as the allocating path, with the per-split partial
results kept in a fixed array inside the library.

This test calls it through the C ABI twice in a row on the same device (the
array is shared and keeps the previous call's contents) and compares each result
with what the existing, allocating entry point produced for the same inputs, under
the same tolerance the other bf16 attention tests use. The caller-owned output
buffer comes from torch, which is only the allocator here.

The file is named so that pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(pkg, views, bench, out_tensor, splits):
    lib = pkg._ffi.lib()
    rc = lib.orion_cuda_paged_decode_attention_noalloc(
        0, views["q"], views["kv_arena"], bench.num_blocks, bench.kv_heads, bench.q_heads,
        views["query_positions"], views["seq_of_row"], views["block_tables_flat"],
        views["block_table_offsets"], bench.batch, views["max_position"], splits,
        out_tensor.data_ptr(), None)
    return rc


def test_noalloc_decode_attention_matches_the_allocating_entry_point(pkg):
    import torch

    backend = pkg.CudaBackend(0)
    rng = np.random.default_rng(21)
    # small batches with long contexts, so that the context is split and the scratch array is used
    cases = [(rng.integers(3000, 8193, 3), 11), (rng.integers(512, 4097, 6), 12)]
    for ctxs, seed in cases:
        bench = pkg.PagedAttentionBench(backend, ctxs, num_blocks=4096, seed=seed)
        bench.run(0, 1)                 # existing entry point: allocates its scratch with cudaMalloc
        expected = bench.output()       # [batch, heads, dim] f32
        views = bench.device_views()
        out = torch.full((bench.batch, bench.q_heads * bench.head_dim), float("nan"),
                         dtype=torch.bfloat16, device="cuda:0")
        for splits in (0, 4):           # two calls in a row on the shared array, different slot layouts
            out.fill_(float("nan"))
            torch.cuda.synchronize()
            rc = _call(pkg, views, bench, out, splits)
            assert rc == 0, pkg._ffi.last_error()
            torch.cuda.synchronize()
            got = out.float().cpu().numpy().reshape(expected.shape)
            rep = pkg.validate(f"noalloc_decode_splits{splits}", expected, got, pkg.Tolerance.F16)
            assert rep.passed(), rep.render()


def test_noalloc_rejects_sizes_beyond_the_built_in_array(pkg):
    import torch

    backend = pkg.CudaBackend(0)
    bench = pkg.PagedAttentionBench(backend, [600] * 4, num_blocks=512, seed=5)
    views = bench.device_views()
    out = torch.zeros((4, bench.q_heads * bench.head_dim), dtype=torch.bfloat16, device="cuda:0")
    lib = pkg._ffi.lib()
    # 300 rows x 32 heads x 32 splits x 130 floats is far more than the 4 Mi floats the array holds;
    # the call is refused before anything is launched, so the oversized row count is never used.
    rc = lib.orion_cuda_paged_decode_attention_noalloc(
        0, views["q"], views["kv_arena"], bench.num_blocks, bench.kv_heads, bench.q_heads,
        views["query_positions"], views["seq_of_row"], views["block_tables_flat"],
        views["block_table_offsets"], 300, views["max_position"], 32, out.data_ptr(), None)
    assert rc == pkg._ffi.ERR_INVALID_REQUEST
    assert "built-in array" in pkg._ffi.last_error()
    # an unsupported shape (9 query heads per kv head) is refused as well
    rc = lib.orion_cuda_paged_decode_attention_noalloc(
        0, views["q"], views["kv_arena"], bench.num_blocks, 1, 9, views["query_positions"],
        views["seq_of_row"], views["block_tables_flat"], views["block_table_offsets"], 4,
        views["max_position"], 1, out.data_ptr(), None)
    assert rc == pkg._ffi.ERR_INVALID_REQUEST
