"""One rank of a tensor-parallel parity run; launched by torch.distributed.run from the tests.

    --mode cpu   the sharded CPU oracle over a gloo all-reduce must equal the unsharded oracle
    --mode gpu   the device model with tp_world = WORLD_SIZE (NCCL inside the library) must match
                 the unsharded oracle within the build's tolerance; needs one GPU per rank
Exit status 0 = parity held on every rank.
"""
import argparse
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
for p in (ROOT, HERE):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch.distributed as dist  # noqa: E402

import __graft_entry__ as ge  # noqa: E402
from conftest import random_tensors  # noqa: E402
from oracle import binding as oracle  # noqa: E402

META = dict(hidden_size=256, num_layers=2, num_attention_heads=8, num_kv_heads=4, head_dim=128,
            vocab_size=512, ffn_dim=768, max_position_embeddings=512, rope_theta=10000.0, rms_norm_eps=1e-5,
            has_qkv_bias=True, tied_lm_head=False, num_blocks=32, block_size=16)


def batches(pkg):
    """A mixed prefill batch, then a decode batch on the same sequences."""
    rng = np.random.default_rng(5)
    lens = [37, 16, 50]
    tables = [[7, 2, 9, 30], [4, 11], [1, 0, 13, 21]]
    toks = rng.integers(0, META["vocab_size"], sum(lens)).tolist()
    pos = [p for n in lens for p in range(n)]
    prefill = pkg.ForwardBatch(toks, pos, [1, 2, 3], lens, lens, tables, has_prefill=True)
    nxt = rng.integers(0, META["vocab_size"], 3).tolist()
    decode = pkg.ForwardBatch(nxt, lens, [1, 2, 3], [1, 1, 1], [n + 1 for n in lens], tables, has_prefill=False)
    return [prefill, decode]


def to_oracle(b):
    return oracle.Batch(b.tokens, b.positions, b.slot_token_counts, b.context_lens, b.block_tables)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", choices=("cpu", "gpu"), required=True)
    ap.add_argument("--dtype", choices=("F32", "BF16"), default="F32")
    ap.add_argument("--model", choices=("small", "kv8", "wide", "collective"), default="small",
                    help="gpu mode: small = 4 kv heads, 3 sequences; kv8 = the benchmark's own check model (8 kv heads, "
                         "up to 8 ranks, 160-row decode and a mixed batch of 1274 rows); wide = hidden 4096 at 256 rows, "
                         "1 Mi elements per hand-over")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = ge.load_package()
    if args.mode == "gpu" and args.model != "small":
        import bench

        backend = pkg.CudaBackend(int(os.environ.get("LOCAL_RANK", rank)))
        if args.model == "collective":
            # the Collective trait over NCCL at the C boundary (lib.rs:243-253), same checks as over gloo
            box = [pkg.NcclCollectiveId.create() if rank == 0 else None]
            dist.broadcast_object_list(box, src=0)
            coll = pkg.NcclCollective(backend, box[0], pkg.Rank(rank, world))
            good = coll.rank() == pkg.Rank(rank, world)
            buf = np.full(5, rank + 1.0, np.float32)
            coll.all_reduce_sum(buf)
            good &= bool(np.all(buf == sum(range(1, world + 1))))
            out = np.zeros(3 * world, np.float32)
            coll.all_gather(np.full(3, float(rank), np.float32), out)
            good &= out.tolist() == [float(r) for r in range(world) for _ in range(3)]
            piece = np.zeros(2, np.float32)
            coll.reduce_scatter_sum(np.arange(2 * world, dtype=np.float32), piece)
            good &= piece.tolist() == [world * (2 * rank + i) for i in range(2)]
            big = np.random.default_rng(rank).standard_normal(1 << 20).astype(np.float32)
            total = big.astype(np.float64)
            for r in range(world):
                if r != rank:
                    total = total + np.random.default_rng(r).standard_normal(1 << 20).astype(np.float32)
            coll.all_reduce_sum(big)
            good &= bool(np.allclose(big, total, atol=1e-5))
            coll.barrier()
            flags = [None] * world
            dist.all_gather_object(flags, bool(good))
            dist.destroy_process_group()
            return 0 if all(flags) else 1
        if args.model == "kv8":
            report = bench.tp_parity(pkg, backend, dist, rank, world, args.dtype)
        else:
            # 256 one-token sequences at hidden 4096: rows x hidden = 1 Mi elements, where the bf16 build moves
            # from the one-shot to the two-shot hand-over at 2 ranks; 256 rows is also the largest fused batch
            wide = dict(bench.TP_CHECK, hidden_size=4096, num_layers=1, num_attention_heads=8, ffn_dim=1024, vocab_size=512)
            rng = np.random.default_rng(31)
            n = 256
            b = pkg.ForwardBatch(rng.integers(0, 512, n).tolist(), [0] * n, list(range(1, n + 1)), [1] * n, [1] * n,
                                 [[int(x)] for x in rng.permutation(300)[:n]], has_prefill=False)
            report = bench.tp_parity(pkg, backend, dist, rank, world, args.dtype, model=wide, num_blocks=300, batches=[b])
        ok = [report.get("ok", True)]
        dist.broadcast_object_list(ok, src=0)
        if rank == 0:
            print(report, file=sys.stderr)
        dist.destroy_process_group()
        return 0 if ok[0] else 1
    weights = random_tensors(np.random.default_rng(17), META, std=0.06)
    if args.dtype == "BF16":
        weights = {k: oracle.round_to_bf16(v) if v.ndim == 2 else v for k, v in weights.items()}
    full = oracle.Model(**META).load(weights)
    ok = True
    if args.mode == "cpu":
        from orionserve_rs_b200.distributed import TorchCollective

        coll = TorchCollective()
        assert coll.rank() == pkg.Rank(rank, world)
        sharded = oracle.Model(**META).load(weights)
        for b in batches(pkg):
            exp = full.forward(to_oracle(b))
            got = sharded.forward_tp(to_oracle(b), rank, world, coll.all_reduce_sum)
            err = float(np.max(np.abs(got - exp)))
            ok &= err < 2e-5  # same arithmetic, the row-parallel sums are split in two
        # each rank wrote only its own KV heads
        lay = pkg.ParallelLayout.compute(pkg.ModelMetadata("llama", "m", **{k: v for k, v in META.items()
                                                                             if k not in ("num_blocks", "block_size")}),
                                         pkg.Rank(rank, world), META["ffn_dim"])
        kv_s, kv_f = sharded.kv().array(), full.kv().array()
        mine = slice(lay.kv_heads.start, lay.kv_heads.end())
        ok &= bool(np.allclose(kv_s[..., mine, :], kv_f[..., mine, :], atol=2e-5))
        other = np.ones(META["num_kv_heads"], bool)
        other[mine] = False
        ok &= not kv_s[..., other, :].any()
        # the collective trait over gloo
        buf = np.full(5, rank + 1.0, np.float32)
        coll.all_reduce_sum(buf)
        ok &= bool(np.all(buf == sum(range(1, world + 1))))
        out = np.zeros(3 * world, np.float32)
        coll.all_gather(np.full(3, float(rank), np.float32), out)
        ok &= out.tolist() == [float(r) for r in range(world) for _ in range(3)]
        piece = np.zeros(2, np.float32)
        coll.reduce_scatter_sum(np.arange(2 * world, dtype=np.float32), piece)
        ok &= piece.tolist() == [world * (2 * rank + i) for i in range(2)]
        coll.barrier()
    else:
        box = [pkg.NcclCollectiveId.create() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        backend = pkg.CudaBackend(int(os.environ.get("LOCAL_RANK", rank)))
        dtype = getattr(pkg.DType, args.dtype)
        meta = pkg.ModelMetadata("qwen2", "tp", **{k: v for k, v in META.items() if k not in ("num_blocks", "block_size")})
        dev = pkg.CudaTransformerModel.new(meta, weights, META["num_blocks"], META["block_size"], backend,
                                           compute_dtype=dtype, max_batch_tokens=128, max_batch_sequences=4,
                                           tp_rank=rank, tp_world=world, nccl_unique_id=box[0])
        for b in batches(pkg):
            exp = full.forward(to_oracle(b))
            got = dev.forward(b).logits
            if rank == 0:  # only the leader returns logits
                scale = float(np.max(np.abs(exp)))
                err = float(np.max(np.abs(got - exp))) / scale
                ok &= err < (1e-3 if args.dtype == "F32" else 3e-2)
        lkv = META["num_kv_heads"] // world
        kv_dev, kv_ref = dev.read_kv(), full.kv().array()[..., rank * lkv:(rank + 1) * lkv, :]
        tol = 1e-4 if args.dtype == "F32" else 3e-2
        ok &= bool(np.allclose(kv_dev, kv_ref, atol=tol, rtol=tol))
        ok &= bool(np.array_equal(kv_dev != 0, kv_ref != 0))
    flags = [None] * world
    dist.all_gather_object(flags, bool(ok))
    dist.destroy_process_group()
    if not all(flags):
        print(f"rank {rank}: parity failed ({flags})", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
