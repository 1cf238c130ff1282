"""Decode attention for callers that cannot allocate device memory (B200 only).

Some users of this library reach attention at a point where they may not call
cudaMalloc: while a stream is being captured into a CUDA graph, inside a serving
loop whose memory all belongs to an external pool, or as a plugin that receives
buffers and a stream and nothing else. ``orion_cuda_paged_decode_attention_noalloc``
serves them: same kernel as the allocating path, with the per-split partial
results kept in a fixed array inside the library.

This test calls it through the C ABI twice in a row on the same device (the
array is shared and keeps the previous call's contents) and compares each result
with what the existing, allocating entry point produced for the same inputs and,
for two sampled sequences, with the CPU oracle directly, under the same tolerance
the other bf16 attention tests use. The caller-owned output buffer comes from
torch, which is only the allocator here. When the box has a second GPU the same
check runs there: the shared-memory opt-in and the array's address belong to a
device, and the caller's current device must be what it was before the call.

The file is named so that pytest collects it last.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _call(pkg, views, bench, out_tensor, splits, device=0):
    lib = pkg._ffi.lib()
    rc = lib.orion_cuda_paged_decode_attention_noalloc(
        device, views["q"], views["kv_arena"], bench.num_blocks, bench.kv_heads, bench.q_heads,
        views["query_positions"], views["seq_of_row"], views["block_tables_flat"],
        views["block_table_offsets"], bench.batch, views["max_position"], splits,
        out_tensor.data_ptr(), None)
    return rc


def _oracle_rows(oracle, bench, ctxs, seqs):
    """paged_attention of the CPU oracle for the sampled sequences of the benchmark's inputs."""
    rows = {}
    for s in seqs:
        q, k, v = bench.sequence(s)
        ctx, hkv, hd = int(ctxs[s]), bench.kv_heads, bench.head_dim
        nblk = (ctx + 15) // 16
        store = oracle.KvStore(1, nblk, 16, hkv, hd)
        a = store.array()[0]  # [block][k|v][slot][head][dim]
        pad = (-ctx) % 16
        a[:, 0] = np.concatenate([k, np.zeros((pad, hkv, hd), np.float32)]).reshape(-1, 16, hkv, hd)
        a[:, 1] = np.concatenate([v, np.zeros((pad, hkv, hd), np.float32)]).reshape(-1, 16, hkv, hd)
        rows[s] = oracle.paged_attention(store, q.reshape(-1), list(range(nblk)), ctx - 1, 0, bench.q_heads, hkv, hd, 16)
    return rows


def _check_device(pkg, oracle, device):
    import torch

    backend = pkg.CudaBackend(device)
    rng = np.random.default_rng(21 + device)
    # small batches with long contexts, so that the context is split and the scratch array is used
    cases = [(rng.integers(3000, 8193, 3), 11), (rng.integers(512, 4097, 6), 12)]
    for ctxs, seed in cases:
        bench = pkg.PagedAttentionBench(backend, ctxs, num_blocks=4096, seed=seed)
        bench.run(0, 1)                 # existing entry point: allocates its scratch with cudaMalloc
        expected = bench.output()       # [batch, heads, dim] f32
        sampled = _oracle_rows(oracle, bench, ctxs, (0, bench.batch - 1))
        views = bench.device_views()
        out = torch.full((bench.batch, bench.q_heads * bench.head_dim), float("nan"),
                         dtype=torch.bfloat16, device=f"cuda:{device}")
        torch.cuda.set_device(0)        # the caller's current device is not the one the call names
        for splits in (0, 4):           # two calls in a row on the shared array, different slot layouts
            out.fill_(float("nan"))
            torch.cuda.synchronize(device)
            rc = _call(pkg, views, bench, out, splits, device)
            assert rc == 0, pkg._ffi.last_error()
            assert torch.cuda.current_device() == 0, "the call must put the caller's device back"
            torch.cuda.synchronize(device)
            got = out.float().cpu().numpy().reshape(expected.shape)
            rep = pkg.validate(f"noalloc_decode_splits{splits}", expected, got, pkg.Tolerance.F16)
            assert rep.passed(), rep.render()
            for s, exp in sampled.items():
                rep = pkg.validate(f"noalloc_vs_oracle_seq{s}_splits{splits}", exp, got[s].reshape(-1), pkg.Tolerance.F16)
                assert rep.passed(), rep.render()
        mask = C.c_uint32(99)
        assert pkg._ffi.lib().orion_cuda_poll_wait_timeouts(backend._h, C.byref(mask)) == 0
        assert mask.value == 0          # no bounded wait of these launches gave up


def test_noalloc_decode_attention_matches_the_allocating_entry_point_and_the_oracle(pkg, oracle):
    _check_device(pkg, oracle, 0)


def test_noalloc_decode_attention_on_a_second_device(pkg, oracle):
    if pkg.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    _check_device(pkg, oracle, 1)


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
