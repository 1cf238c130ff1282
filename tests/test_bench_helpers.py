"""Host-side arithmetic of the benchmark: algorithmic byte counts and the synthetic decode batch."""
import numpy as np

import bench


def test_algorithmic_bytes_of_the_headline_step():
    m = bench.LLAMA3_8B
    # 218.1 M parameters per layer x 32 + 525.3 M of LM head, bf16: 15.0 GB of weights per step
    assert bench.layer_param_count(m) == 218_103_808
    assert bench.weight_bytes_per_step(m) == 2 * (32 * 218_103_808 + 128256 * 4096)
    # 4096 B per context token per sequence per layer + q/out + table entries
    kv = bench.kv_bytes_per_step(m, [bench.CONTEXT] * bench.BATCH)
    per_layer = 64 * (1024 * 4096 + 32 * 128 * 2 * 2 + 64 * 4)
    assert kv == 32 * per_layer
    assert abs(kv / 1e9 - 8.62) < 0.01


def test_tensor_parallel_ranks_share_the_layers_and_the_head():
    for m in (bench.LLAMA3_8B, bench.LLAMA3_70B):
        whole = bench.weight_bytes_per_step(m)
        head = 2 * m["vocab_size"] * m["hidden_size"]
        for world in (2, 4, 8):
            # the head is split by vocabulary in multiples of 128 rows; the busiest rank holds the rounded-up share
            rows = -(-(-(-m["vocab_size"] // world)) // 128) * 128
            assert bench.head_rows_per_rank(m, world) == rows and rows * world >= m["vocab_size"] > rows * (world - 1)
            assert bench.weight_bytes_per_step(m, world) == (whole - head) // world + 2 * rows * m["hidden_size"]
            ctx = [1024, 4096, 2000]
            tables = m["num_layers"] * sum((c + 15) // 16 for c in ctx) * 4  # every rank reads the whole table
            assert bench.kv_bytes_per_step(m, ctx, world) * world - bench.kv_bytes_per_step(m, ctx) == tables * (world - 1)


def test_decode_batches_are_valid_and_their_tables_disjoint(pkg):
    rng = np.random.default_rng(0)
    for contexts in ([1024] * 8, [1024, 4096, 1500, 16, 17, 1]):
        num_blocks = sum(c // 16 + 1 for c in contexts) + 4
        b = bench.make_decode_batch(pkg, rng, num_blocks, contexts, 1000)
        b.validate()
        tokens, positions, counts, ctx, flat, offsets = b.flatten()
        assert positions.tolist() == [c - 1 for c in contexts] and ctx.tolist() == contexts
        assert counts.tolist() == [1] * len(contexts) and int(tokens.max()) < 1000
        lens = np.diff(offsets).tolist()
        assert lens == [(c + 15) // 16 for c in contexts]
        used = flat[:int(offsets[-1])]
        assert len(set(used.tolist())) == len(used) and int(used.max()) < num_blocks
