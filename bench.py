"""Benchmark of the forward path: decode tokens/s at batch 64 on the Llama-3-8B shape.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward pass over a decode batch (64 sequences, one new token each,
1024-token contexts in a paged bf16 KV cache, random-init bf16 weights). With N > 1 the
same step runs tensor-parallel over N GPUs (one process per GPU, launched by torchrun).
Rank 0 prints one JSON line. ``--impl reference`` times the CPU restatement of the
reference's scalar f32 path on the host cores over a bounded sample of the same step.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

LLAMA3_8B = dict(hidden_size=4096, num_layers=32, num_attention_heads=32, num_kv_heads=8, head_dim=128,
                 vocab_size=128256, ffn_dim=14336, max_position_embeddings=8192, rope_theta=500000.0,
                 rms_norm_eps=1e-5)
QWEN2_7B = dict(hidden_size=3584, num_layers=28, num_attention_heads=28, num_kv_heads=4, head_dim=128,
                vocab_size=152064, ffn_dim=18944, max_position_embeddings=8192, rope_theta=1000000.0,
                rms_norm_eps=1e-6, has_qkv_bias=True)
LLAMA3_70B = dict(hidden_size=8192, num_layers=80, num_attention_heads=64, num_kv_heads=8, head_dim=128,
                  vocab_size=128256, ffn_dim=28672, max_position_embeddings=8192, rope_theta=500000.0,
                  rms_norm_eps=1e-5)
BATCH, CONTEXT, BLOCK = 64, 1024, 16
WORKLOAD = "llama3_8b_decode_batch64_ctx1024_bf16"
METRIC = "decode tokens/s at batch 64 (Llama-3-8B shape)"
GEMM_PROFILE = os.path.join(ROOT, "profiles", "gemm_tc_kernel_decode_batch64_llama3_8b_shape.md")


def gemm_traffic_bytes_per_step():
    """DRAM bytes (read + write) of the projection launches of one 32-layer headline step, as the ncu
    capture summarised in the profile file measured them. The summary carries the figures on two lines,
    `dram_bytes_per_layer: <n>` (the four projections of one layer) and `dram_bytes_lm_head: <n>` (the
    head's launches), next to the commit the capture was taken at; nothing is typed in here, so a
    stale capture shows in that file and not as a silent constant. None when the file lacks them."""
    import re
    try:
        text = open(GEMM_PROFILE).read()
    except OSError:
        return None
    layer = re.search(r"^dram_bytes_per_layer:\s*(\d+)", text, re.M)
    head = re.search(r"^dram_bytes_lm_head:\s*(\d+)", text, re.M)
    if not layer or not head:
        return None
    return LLAMA3_8B["num_layers"] * int(layer.group(1)) + int(head.group(1))


def measured_peaks():
    """HBM GB/s and which source it came from (driver-written file, else the stated fallback)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except (OSError, ValueError, KeyError):
        return 6650.0, "fallback"


def layer_param_count(m, world=1):
    H, hd = m["hidden_size"], m["head_dim"]
    q, kv, f = m["num_attention_heads"] // world, m["num_kv_heads"] // world, m["ffn_dim"] // world
    return H * (q + 2 * kv) * hd + q * hd * H + 3 * H * f


def head_rows_per_rank(m, world=1):
    """Rows of the LM head the busiest rank streams: all of them on one GPU; under tensor parallelism the head
    is split by vocabulary in multiples of the 128-row weight tile (ORION_TP_VOCAB_PARALLEL=0: replicated)."""
    if world == 1 or os.environ.get("ORION_TP_VOCAB_PARALLEL") == "0":
        return m["vocab_size"]
    return min(m["vocab_size"], ((m["vocab_size"] + world - 1) // world + 127) // 128 * 128)


def weight_bytes_per_step(m, world=1):
    """Algorithmic bytes of the projection GEMMs of one decode step on one rank: every bf16
    weight of the rank once (layers and LM head sharded under TP)."""
    return 2 * (m["num_layers"] * layer_param_count(m, world) + head_rows_per_rank(m, world) * m["hidden_size"])


def kv_bytes_per_step(m, contexts, world=1):
    """Algorithmic bytes of paged decode attention per step on one rank: K and V once per KV
    head and context token, q in and out once per sequence, 4 B per block-table entry."""
    kvh, hd, q = m["num_kv_heads"] // world, m["head_dim"], m["num_attention_heads"] // world
    per_layer = sum(c * kvh * hd * 2 * 2 + q * hd * 2 * 2 + ((c + BLOCK - 1) // BLOCK) * 4 for c in contexts)
    return m["num_layers"] * per_layer


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# CPU leg: the oracle (a restatement of the reference's CPU path) on a bounded sample
# ---------------------------------------------------------------------------------------------

def cpu_sample_step(oracle, threads: int, sample_batch: int, rng):
    """One layer of the Llama-3-8B shape at `sample_batch` decode tokens with 1024-token contexts,
    plus 1/16 of the LM head rows, in the reference's operation order. Returns seconds for the
    layer and for the head slice."""
    m = LLAMA3_8B
    H, hd, Hq, Hkv, F = m["hidden_size"], m["head_dim"], m["num_attention_heads"], m["num_kv_heads"], m["ffn_dim"]
    oracle.set_threads(threads)
    f32 = np.float32
    w = {k: (rng.standard_normal(s, dtype=f32) * f32(0.02)) for k, s in
         dict(q=(Hq * hd, H), k=(Hkv * hd, H), v=(Hkv * hd, H), o=(H, Hq * hd), gate=(F, H), up=(F, H),
              down=(H, F)).items()}
    head = rng.standard_normal((m["vocab_size"] // 16, H), dtype=f32) * f32(0.02)
    ones = np.ones(H, f32)
    nblk = CONTEXT // BLOCK
    store = oracle.KvStore(1, sample_batch * nblk, BLOCK, Hkv, hd)
    store.array()[...] = rng.standard_normal(store.array().shape, dtype=f32)
    cos, sin = oracle.rope_table(hd, CONTEXT, m["rope_theta"])
    hidden = rng.standard_normal((sample_batch, H), dtype=f32)
    tables = [list(range(s * nblk, (s + 1) * nblk)) for s in range(sample_batch)]
    pos = CONTEXT - 1

    t0 = time.perf_counter()
    normed = oracle.rms_norm(hidden, ones, m["rms_norm_eps"])
    q, k, v = oracle.linear(normed, w["q"]), oracle.linear(normed, w["k"]), oracle.linear(normed, w["v"])
    for r in range(sample_batch):
        for h in range(Hq):
            q[r, h * hd:(h + 1) * hd] = oracle.apply_rope(q[r, h * hd:(h + 1) * hd], cos[pos], sin[pos])
        for h in range(Hkv):
            k[r, h * hd:(h + 1) * hd] = oracle.apply_rope(k[r, h * hd:(h + 1) * hd], cos[pos], sin[pos])
            store.write(0, tables[r][-1], pos % BLOCK, h, False, k[r, h * hd:(h + 1) * hd])
            store.write(0, tables[r][-1], pos % BLOCK, h, True, v[r, h * hd:(h + 1) * hd])
    attn = np.stack([oracle.paged_attention(store, q[r], tables[r], pos, 0, Hq, Hkv, hd, BLOCK)
                     for r in range(sample_batch)])
    hidden = hidden + oracle.linear(attn, w["o"])
    normed = oracle.rms_norm(hidden, ones, m["rms_norm_eps"])
    act = oracle.swiglu(oracle.linear(normed, w["gate"]), oracle.linear(normed, w["up"]))
    hidden = hidden + oracle.linear(act, w["down"])
    t_layer = time.perf_counter() - t0
    t0 = time.perf_counter()
    oracle.linear(oracle.rms_norm(hidden, ones, m["rms_norm_eps"]), head)
    t_head = time.perf_counter() - t0
    return t_layer, t_head


def cpu_tokens_per_s(t_layer, t_head, sample_batch):
    """Extrapolates the sampled layer and head slice to a full 32-layer step with the whole head."""
    step = LLAMA3_8B["num_layers"] * t_layer + 16.0 * t_head
    return sample_batch / step


def headline_config(world, layers, workload=WORKLOAD, nbatch=BATCH, context=CONTEXT, full_layers=32, wbytes=None, kbytes=None):
    """The `config` object of the JSON line; both arms print the same keys for the same workload."""
    m = LLAMA3_8B
    if wbytes is None:
        wbytes, kbytes = weight_bytes_per_step(m, world), kv_bytes_per_step(m, [CONTEXT] * BATCH, world)
    return {"workload": workload if layers == full_layers else f"{workload}_first{layers}layers",
            "batch": nbatch, "context": context, "block_size": BLOCK, "layers": layers, "parallelism": f"tp{world}",
            "l2": f"inputs exceed L2: {wbytes / 1e9:.1f} GB of weights + {kbytes / 1e9:.1f} GB of KV read "
                  f"per step and rank"}


def run_reference(args):
    """--impl reference: the reference's CPU path (restated; the Rust reference cannot be built
    where this runs) on the host cores, all threads, bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    from oracle import binding as oracle

    oracle.build()
    cores = os.cpu_count() or 1
    threads = min(cores, 64)
    sample_batch = 8
    rng = np.random.default_rng(0)
    # one sampled step costs ~0.15 s of wall clock on 16 threads: K steps and W warm-ups as asked
    for _ in range(max(0, args.warmup)):
        cpu_sample_step(oracle, threads, sample_batch, rng)
    times = [cpu_sample_step(oracle, threads, sample_batch, rng) for _ in range(max(1, args.steps))]
    t_layer = float(np.mean([t[0] for t in times]))
    t_head = float(np.mean([t[1] for t in times]))
    value = cpu_tokens_per_s(t_layer, t_head, sample_batch)
    sample = (f"1 of 32 layers at {sample_batch} decode tokens (ctx {CONTEXT}) + 1/16 of the LM head rows per step, "
              f"extrapolated to 32 layers + full head; {threads} threads over output elements (bit-identical to 1)")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": len(times), "warmup": max(0, args.warmup), "ms_per_step": 1000.0 * (t_layer + t_head),
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": headline_config(max(1, args.gpus), LLAMA3_8B["num_layers"]),
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# GPU leg
# ---------------------------------------------------------------------------------------------

def make_decode_batch(pkg, rng, num_blocks, contexts, vocab):
    """One decode step: every sequence feeds one token at position context - 1; the block tables are
    consecutive slices of one random permutation of the pool."""
    perm = rng.permutation(num_blocks).astype(np.uint32)
    n = len(contexts)
    nblk = (np.asarray(contexts) + BLOCK - 1) // BLOCK
    if int(nblk.min()) == int(nblk.max()):
        # the batch as contiguous host arrays, the form the reference's ForwardBatch vectors have
        tables = np.ascontiguousarray(perm[:n * int(nblk[0])].reshape(n, int(nblk[0])))
    else:
        ends = np.cumsum(nblk)
        tables = [np.ascontiguousarray(perm[e - k:e]) for e, k in zip(ends, nblk)]
    tokens = rng.integers(0, vocab, n).astype(np.uint32)
    ctx = np.asarray(contexts, dtype=np.uint64)
    return pkg.ForwardBatch(tokens, (ctx - 1).astype(np.uint32), np.arange(1, n + 1, dtype=np.uint64),
                            np.ones(n, np.uint64), ctx, tables, has_prefill=False)


def attention_sweep(pkg, backend, peak):
    """Paged GQA decode-attention microbenchmark (bf16, 32 query / 8 KV heads, head_dim 128, block 16):
    batch in {1, 8, 64, 256}, context lengths uniform in [512, 8192], each table a consecutive slice of
    one random permutation of a 200 000-block pool, N(0, 1) values. GB/s = algorithmic bytes / launch."""
    out = []
    rng = np.random.default_rng(2024)
    for batch in (1, 8, 64, 256):
        ctx = rng.integers(512, 8193, batch)
        bench = pkg.PagedAttentionBench(backend, ctx, num_blocks=200_000, seed=batch)
        ms, nbytes = bench.run(3, 20)
        gbs = nbytes / (ms / 1000.0) / 1e9
        out.append({"batch": batch, "context_tokens": int(ctx.sum()), "ms": ms, "algorithmic_bytes": nbytes,
                    "gbs": gbs, "frac_of_measured_peak": gbs / peak, "frac_of_8tbs_nominal": gbs / 8000.0})
        del bench
    return out


def run_serving(args):
    """Continuous batching through the engine loop (not the headline): the third configuration of the
    benchmark definition, Llama-3-8B shape, `--requests` requests with prompts U[128,2048] and outputs
    U[64,512], chunked prefill with a 512-token step budget, greedy sampling on the device."""
    import __graft_entry__ as ge

    pkg = ge.load_package()
    E = pkg.engine
    backend = pkg.CudaBackend(0)
    rng = np.random.default_rng(11)
    if args.workload == "prefix":
        # the fourth configuration: Qwen2-7B shape, one shared 1024-token prefix + unique 64-256-token
        # suffixes, 128 output tokens each (blocks are shared; compute is skipped only with the flag)
        m = dict(QWEN2_7B, num_layers=min(args.layers, QWEN2_7B["num_layers"]))
        meta = pkg.ModelMetadata(architecture="qwen2", name="qwen2-7b-shape", dtype=pkg.DType.BF16, **m)
        shared = rng.integers(0, m["vocab_size"], 1024)
        prompts = [np.concatenate([shared, rng.integers(0, m["vocab_size"], int(rng.integers(64, 257)))]).astype(np.uint32)
                   for _ in range(args.requests)]
        outputs = [128] * args.requests
        name, shape = "qwen2_7b_shared_prefix_bf16", "1024 shared + U[64,256]"
    else:
        m = dict(LLAMA3_8B, num_layers=args.layers)
        meta = pkg.ModelMetadata(architecture="llama", name="llama3-8b-shape", dtype=pkg.DType.BF16, **m)
        prompts = [rng.integers(0, m["vocab_size"], int(rng.integers(128, 2049))).astype(np.uint32) for _ in range(args.requests)]
        outputs = [int(rng.integers(64, 513)) for _ in range(args.requests)]
        name, shape = "llama3_8b_continuous_batching_bf16", "U[128,2048]"
    # every sequence fully resident at once, plus the slot the reference's decode position skips
    num_blocks = sum((len(p) + o + 2) // BLOCK + 1 for p, o in zip(prompts, outputs)) + 64
    budget = 512
    model = pkg.CudaTransformerModel(meta, num_blocks, BLOCK, backend, compute_dtype=pkg.DType.BF16,
                                     max_batch_tokens=budget, max_batch_sequences=min(256, args.requests))
    model.init_random(seed=1, std=0.02)
    cfg = E.SchedulerConfig(max_num_seqs=min(256, args.requests), max_num_batched_tokens=budget, max_model_len=4096,
                            enable_chunked_prefill=True, max_waiting_requests=4096, request_timeout_secs=None,
                            skip_cached_prefix=args.skip_cached_prefix)
    eng = E.Engine(model, cfg, num_blocks, BLOCK, True, [])
    for p, o in zip(prompts, outputs):
        eng.submit(p, E.SamplingParams(temperature=0.0, max_tokens=o))
    steps = failed = 0
    backend.synchronize()
    with ClockSampler(0) as clocks:
        t0 = time.perf_counter()
        while eng.has_work():
            try:
                eng.step()
            except pkg.InternalError:
                failed += 1  # the reference's off-by-one decode position: refused before any launch, retried next step
            steps += 1
            if steps % 64 == 0:
                eng.take_events()
        backend.synchronize()
        dt = time.perf_counter() - t0
    stats = eng.scheduler().stats()
    out_tokens, prompt_tokens = sum(outputs), int(sum(len(p) for p in prompts))
    print(json.dumps({
        "metric": f"continuous-batching output tokens/s ({meta.name})", "value": out_tokens / dt, "unit": "tokens/s",
        "n_gpus": 1, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": name, "requests": args.requests, "prompts": shape,
                   "outputs": "128" if args.workload == "prefix" else "U[64,512]", "step_token_budget": budget,
                   "block_size": BLOCK, "layers": m["num_layers"], "num_blocks": num_blocks,
                   "sampling": "greedy on the device", "skip_cached_prefix": bool(args.skip_cached_prefix)},
        "prefix_cache_hits": eng.scheduler().cache().stats()["prefix_cache_hits"],
        "skipped_prefill_tokens": stats["total_skipped_prefill_tokens"],
        "seconds": dt, "engine_steps": steps, "refused_steps": failed, "prompt_tokens": prompt_tokens,
        "output_tokens": out_tokens, "total_tokens_per_s": (prompt_tokens + out_tokens) / dt,
        "preemptions": stats["total_preempted"], "mean_batch_tokens": stats["total_batched_tokens"] / max(1, stats["total_steps"]),
        "clocks": clocks.summary()}))
    return 0


# ---------------------------------------------------------------------------------------------
# Tensor-parallel parity, checked before anything is timed at N > 1
# ---------------------------------------------------------------------------------------------

# A small Llama/Qwen2-shaped model with EIGHT kv heads (so that 2, 4 and 8 ranks all get whole heads),
# QKV bias, head_dim 128 and 16-token blocks: every rank runs the tuned kernels of the headline step.
TP_CHECK = dict(hidden_size=1024, num_layers=2, num_attention_heads=16, num_kv_heads=8, head_dim=128,
                vocab_size=2048, ffn_dim=2048, max_position_embeddings=64, rope_theta=10000.0, rms_norm_eps=1e-5,
                has_qkv_bias=True, tied_lm_head=False)
TP_CHECK_BLOCKS = 384


def round_bf16(a):
    """Nearest-even rounding of f32 to bf16 precision, kept as f32 (what the device does at load)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def tp_check_weights(m=None, seed=23):
    """Seeded host checkpoint of the check model (every rank draws the same values and slices its own)."""
    m, rng = m or TP_CHECK, np.random.default_rng(seed)
    H, V, F, hd = m["hidden_size"], m["vocab_size"], m["ffn_dim"], m["head_dim"]
    qd, kvd = m["num_attention_heads"] * hd, m["num_kv_heads"] * hd

    def mat(r, c, std):
        return round_bf16((rng.standard_normal((r, c)) * std).astype(np.float32))

    def gain():
        return (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)

    t = {"model.embed_tokens.weight": mat(V, H, 1.0), "model.norm.weight": gain(), "lm_head.weight": mat(V, H, 0.05)}
    for i in range(m["num_layers"]):
        p = f"model.layers.{i}"
        t[f"{p}.input_layernorm.weight"], t[f"{p}.post_attention_layernorm.weight"] = gain(), gain()
        t[f"{p}.self_attn.q_proj.weight"], t[f"{p}.self_attn.k_proj.weight"] = mat(qd, H, 0.04), mat(kvd, H, 0.04)
        t[f"{p}.self_attn.v_proj.weight"], t[f"{p}.self_attn.o_proj.weight"] = mat(kvd, H, 0.04), mat(H, qd, 0.03)
        for n, d in (("q", qd), ("k", kvd), ("v", kvd)):
            t[f"{p}.self_attn.{n}_proj.bias"] = (rng.standard_normal(d) * 0.1).astype(np.float32)
        t[f"{p}.mlp.gate_proj.weight"], t[f"{p}.mlp.up_proj.weight"] = mat(F, H, 0.04), mat(F, H, 0.04)
        t[f"{p}.mlp.down_proj.weight"] = mat(H, F, 0.03)
    return t


def tp_check_batches(pkg, seed=29):
    """Four steps on 160 sequences (two blocks each, prompts of 2..20 tokens): a ragged prefill of the
    first 48; a mixed batch (those 48 decode one token, the other 112 prefill); a decode batch of 48
    rows (the small token tiles and, at 2 ranks, the one-shot hand-over); a decode batch of all 160
    rows (the 256-token tile and more than 128 rows through the hand-over)."""
    rng = np.random.default_rng(seed)
    n, first, V = 160, 48, TP_CHECK["vocab_size"]
    lens = rng.integers(2, 21, n)
    perm = rng.permutation(TP_CHECK_BLOCKS)[:2 * n].reshape(n, 2)
    tables = [row.tolist() for row in perm]
    ids = list(range(1, n + 1))
    done = np.zeros(n, np.int64)  # tokens each sequence has in the cache so far
    steps = []

    def step(feed):  # feed: list of (sequence index, number of tokens)
        toks, pos, cnt, ctx, tbl, sid = [], [], [], [], [], []
        for s, k in feed:
            toks += rng.integers(0, V, k).tolist()
            pos += list(range(int(done[s]), int(done[s]) + k))
            done[s] += k
            cnt.append(k), ctx.append(int(done[s])), tbl.append(tables[s]), sid.append(ids[s])
        steps.append(pkg.ForwardBatch(toks, pos, sid, cnt, ctx, tbl, has_prefill=any(k > 1 for _, k in feed)))

    step([(s, int(lens[s])) for s in range(first)])
    step([(s, 1) for s in range(first)] + [(s, int(lens[s])) for s in range(first, n)])
    step([(s, 1) for s in range(first)])
    step([(s, 1) for s in range(n)])
    return steps


GRAPH_REPEATS = 34  # two more than the repeats after which the library captures a decode step (32)


def tp_parity(pkg, backend, dist, rank, world, dtype_name="BF16", model=None, num_blocks=TP_CHECK_BLOCKS, batches=None):
    """Runs the check model at tp_world = `world` and compares rank 0's logits and every rank's KV arena
    with the CPU oracle's unsharded forward (the oracle is the checker here, nothing of it is timed).
    Bars: bf16 build 2e-2 max-abs after softmax and logits within 3e-2 of their range; f32 build 1e-3."""
    import torch

    m = model or TP_CHECK
    weights = tp_check_weights(m)
    box = [pkg.NcclCollectiveId.create() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    dtype = getattr(pkg.DType, dtype_name)
    meta = pkg.ModelMetadata(architecture="qwen2", name="tp-check", dtype=dtype, **m)
    batches = batches or tp_check_batches(pkg)
    max_tokens = max(len(b.tokens) for b in batches)
    max_seqs = max(len(b.slot_token_counts) for b in batches)
    dev = pkg.CudaTransformerModel.new(meta, weights, num_blocks, BLOCK, backend, compute_dtype=dtype,
                                       max_batch_tokens=max_tokens, max_batch_sequences=max_seqs, tp_rank=rank,
                                       tp_world=world, nccl_unique_id=box[0])
    got = [dev.forward(b).logits for b in batches]
    # A decode batch whose layout repeats is replayed as a CUDA graph after GRAPH_REPEATS - 2 steps: the first decode
    # batch of the check is run that often once more (the same tokens at the same positions rewrite the same KV
    # slots with the same values), and the last result, produced by a graph, must be the first one bit for bit.
    decode = next((i for i, b in enumerate(batches) if not b.has_prefill and len(b.tokens) <= 256), None)
    graph_same = None
    if decode is not None and dtype_name == "BF16":
        for _ in range(GRAPH_REPEATS):
            again = dev.forward(batches[decode]).logits
        graph_same = bool(rank != 0 or np.array_equal(again, got[decode]))
    kv_dev = dev.read_kv()
    del dev
    lkv = m["num_kv_heads"] // world
    kv_shape = (m["num_layers"], num_blocks, 2, BLOCK, m["num_kv_heads"], m["head_dim"])
    kv_ref = torch.zeros(kv_shape, dtype=torch.float32)
    report = {"ranks": world, "dtype": dtype_name.lower(),
              "model": f"{m['num_layers']} layers, hidden {m['hidden_size']}, {m['num_attention_heads']}/"
                       f"{m['num_kv_heads']} heads, head_dim {m['head_dim']}, ffn {m['ffn_dim']}, QKV bias",
              "steps": [f"{len(b.slot_token_counts)} sequences / {len(b.tokens)} rows" for b in batches]}
    if rank == 0:
        from oracle import binding as oracle

        oracle.build()
        oracle.set_threads(min(os.cpu_count() or 1, 64))
        ref = oracle.Model(num_blocks=num_blocks, block_size=BLOCK, **m).load(weights)
        rel = soft = 0.0
        for b, g in zip(batches, got):
            exp = ref.forward(oracle.Batch(b.tokens, b.positions, b.slot_token_counts, b.context_lens, b.block_tables))
            rel = max(rel, float(np.max(np.abs(g - exp)) / np.max(np.abs(exp))))
            pe, pg = (np.exp(x - x.max(axis=1, keepdims=True)) for x in (exp.astype(np.float64), g.astype(np.float64)))
            soft = max(soft, float(np.max(np.abs(pe / pe.sum(1, keepdims=True) - pg / pg.sum(1, keepdims=True)))))
        kv_ref.copy_(torch.from_numpy(np.ascontiguousarray(ref.kv().array()).reshape(kv_shape)))
        report.update(max_rel_err=rel, softmax_max_abs=soft)
    dist.broadcast(kv_ref, src=0)
    mine = kv_ref.numpy()[..., rank * lkv:(rank + 1) * lkv, :]
    tol = 3e-2 if dtype_name == "BF16" else 1e-4
    kv_ok = bool(np.array_equal(kv_dev != 0, mine != 0) and np.allclose(kv_dev, mine, atol=tol, rtol=tol))
    flags = [None] * world
    dist.all_gather_object(flags, kv_ok)
    if graph_same is not None:
        same = [None] * world
        dist.all_gather_object(same, graph_same)
        report["graph_replay_identical"] = all(same)
    if rank == 0:
        report["kv_slots_equal"] = all(flags)
        bars = (2e-2, 3e-2) if dtype_name == "BF16" else (1e-3, 1e-3)
        report["ok"] = bool(report["softmax_max_abs"] <= bars[0] and report["max_rel_err"] <= bars[1] and all(flags) and
                            report.get("graph_replay_identical", True))
    return report


def run_ours(args):
    if args.workload in ("serving", "prefix"):
        return run_serving(args)
    import __graft_entry__ as ge

    pkg = ge.load_package()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    nccl_id = None
    json_out = sys.stdout
    if world > 1:
        # NCCL prints its version banner on stdout: keep the original stdout for the one JSON line and send
        # everything else that is written to descriptor 1 to stderr
        sys.stdout.flush()
        json_out = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)
        import torch.distributed as dist  # plumbing only: rendezvous, id broadcast, max over ranks

        dist.init_process_group("gloo", rank=rank, world_size=world)
        box = [pkg.NcclCollectiveId.create() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        nccl_id = box[0]
    backend = pkg.CudaBackend(local_rank)
    parity = tp_parity(pkg, backend, dist, rank, world) if world > 1 and not args.no_tp_parity else None
    if args.no_pdl:
        pkg._ffi.lib().orion_cuda_set_programmatic_launch(0)
    if args.attn_stages or args.attn_ctas:
        pkg._ffi.lib().orion_cuda_attention_set_tuning(args.attn_stages, args.attn_ctas)
    if args.gemm_ctas or args.gemm_stages:
        pkg._ffi.lib().orion_cuda_gemm_set_tuning(args.gemm_ctas, args.gemm_stages)
    rng = np.random.default_rng(3)
    if args.shape == "llama3-70b":
        # the fifth configuration of the benchmark definition (not the headline): Llama-3-70B shape under
        # tensor parallelism, decode at batch 128, contexts uniform in [1024, 4096]
        full_layers = LLAMA3_70B["num_layers"]
        layers = full_layers if args.layers == 32 else args.layers
        m = dict(LLAMA3_70B, num_layers=layers)
        contexts = [int(c) for c in np.random.default_rng(5).integers(1024, 4097, 128)]
        name, metric = "llama3-70b-shape", "decode tokens/s at batch 128 (Llama-3-70B shape, tensor parallel)"
        workload = "llama3_70b_decode_batch128_ctx1024to4096_bf16"
    else:
        full_layers, layers = 32, args.layers
        m = dict(LLAMA3_8B, num_layers=layers)
        contexts = [CONTEXT] * args.batch
        name, metric, workload = "llama3-8b-shape", METRIC, WORKLOAD
        if args.batch != BATCH:  # not the headline: the same step at another batch size
            metric = f"decode tokens/s at batch {args.batch} (Llama-3-8B shape)"
            workload = f"llama3_8b_decode_batch{args.batch}_ctx1024_bf16"
    nbatch = len(contexts)
    meta = pkg.ModelMetadata(architecture="llama", name=name, dtype=pkg.DType.BF16, **m)
    num_blocks = sum(c // BLOCK + 1 for c in contexts) + 64
    model = pkg.CudaTransformerModel(meta, num_blocks, BLOCK, backend, compute_dtype=pkg.DType.BF16,
                                     max_batch_tokens=nbatch, max_batch_sequences=nbatch, tp_rank=rank,
                                     tp_world=world, nccl_unique_id=nccl_id)
    model.init_random(seed=1, std=0.02)
    model.fill_kv_random(seed=2, std=1.0)
    batch = make_decode_batch(pkg, rng, num_blocks, contexts, m["vocab_size"])
    from orionserve_rs_b200.model import pinned_empty

    logits, owner = pinned_empty(nbatch * m["vocab_size"])

    def barrier():
        backend.synchronize()
        if dist is not None:
            dist.barrier()

    def max_over_ranks(x: float) -> float:
        if dist is None:
            return x
        import torch

        t = torch.tensor([x], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # warm-up through the public call (also uploads the batch the replays reuse)
    for _ in range(max(args.warmup, 3)):
        model.forward(batch, out=logits)
    launches_per_step = model.last_launch_count()

    with ClockSampler(local_rank) as clocks:
        # (1) device-resident: inputs and block tables already in HBM, CUDA events on the launch stream
        barrier()
        dev_ms = model.replay(args.steps)
        barrier()
        dev_ms = max_over_ranks(dev_ms)
        # (2) end to end through forward(): host batch in, host logits out, every step
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            model.forward(batch, out=logits)
        barrier()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        # (2b) the same through forward_greedy(): argmax on the device, token ids out (what the
        # engine loop uses); reported beside the headline e2e, not instead of it
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            model.forward_greedy(batch)
        barrier()
        greedy_s = max_over_ranks(time.perf_counter() - t0)
    # (3) per-kernel device time for the roofline, event pair around every launch
    prof = model.profile(args.steps)
    barrier()
    # (4) one kernel family at a time, launched back to back as inside the step (dependent-launch
    # overlap included) with the other families left out: the per-launch duration of the roofline
    gemm_chain_ms = max_over_ranks(model.replay_categories(args.steps, "gemm"))
    attn_chain_ms = max_over_ranks(model.replay_categories(args.steps, "attention"))
    barrier()
    # (5) the same step at small batches (the projections in their GEMV regime, 16- and 32-token tiles):
    # device-resident step time and the two kernel families run back to back, 20 steps each
    small = []
    if world == 1 and args.shape == "llama3-8b" and args.batch == BATCH and not args.no_small_batch:
        peak_gbs = measured_peaks()[0]
        for b in (1, 8, 16):
            sb = make_decode_batch(pkg, np.random.default_rng(40 + b), num_blocks, contexts[:b], m["vocab_size"])
            for _ in range(3):
                model.forward(sb, out=logits)
            n = 20
            step_ms = model.replay(n) / n
            g_ms, a_ms = model.replay_categories(n, "gemm") / n, model.replay_categories(n, "attention") / n
            wb, kb = weight_bytes_per_step(m), kv_bytes_per_step(m, contexts[:b])
            small.append({"batch": b, "ms_per_step": step_ms, "tokens_per_s": b / (step_ms / 1000.0),
                          "gemm_ms": g_ms, "gemm_frac": wb / (g_ms / 1000.0) / 1e9 / peak_gbs,
                          "attn_ms": a_ms, "attn_frac": kb / (a_ms / 1000.0) / 1e9 / peak_gbs,
                          "step_frac": (wb + kb) / (step_ms / 1000.0) / 1e9 / peak_gbs})
    model.forward(batch, out=logits)  # leave the buffers holding a real step again
    if rank != 0:
        return 0

    ms_per_step = dev_ms / args.steps
    value = nbatch / (ms_per_step / 1000.0)
    e2e_value = nbatch * args.steps / e2e_s
    peak, peak_src = measured_peaks()
    gemm_ms, gemm_n = prof["gemm"]
    attn_ms, attn_n = prof["attention"]
    wbytes = weight_bytes_per_step(m, world)
    kbytes = kv_bytes_per_step(m, contexts, world)
    gemm_gbs = wbytes * args.steps / (gemm_chain_ms / 1000.0) / 1e9
    attn_gbs = kbytes * args.steps / (attn_chain_ms / 1000.0) / 1e9
    gemm_gbs_serial = wbytes * args.steps / (gemm_ms / 1000.0) / 1e9 if gemm_ms > 0 else None
    attn_gbs_serial = kbytes * args.steps / (attn_ms / 1000.0) / 1e9 if attn_ms > 0 else None
    meta_bytes = 4 * (5 * nbatch + 2 * nbatch + 1 + sum(len(t) for t in batch.block_tables))
    line = {
        "metric": metric, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": headline_config(world, layers, workload, nbatch, CONTEXT if args.shape == "llama3-8b" else "U[1024,4096]",
                                  full_layers, wbytes, kbytes),
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": meta_bytes,
                "d2h_bytes_per_step": nbatch * m["vocab_size"] * 4},
        "e2e_greedy": {"value": nbatch * args.steps / greedy_s, "unit": "tokens/s", "h2d_bytes_per_step": meta_bytes,
                       "d2h_bytes_per_step": nbatch * 4,
                       "note": "forward_greedy: host batch in, argmax on the device, 4 bytes per sequence out"},
        "gpu_launches": int(launches_per_step * args.steps),
        "launch": ("kernel by kernel (ORION_STEP_GRAPH=0)" if os.environ.get("ORION_STEP_GRAPH", "1") == "0" else
                   "decode step replayed as a CUDA graph of the embedding and the layers once its batch layout has stayed; "
                   "LM head by stream launches; gpu_launches counts the kernels inside the graph too"),
        "clocks": clocks.summary(),
        "roofline": {"bound": "hbm", "kernel": "gemm_tc_kernel (projection weights streamed once per step)",
                     "achieved": gemm_gbs, "peak": peak, "peak_source": peak_src, "unit": "GB/s",
                     "frac": gemm_gbs / peak, "traffic": gemm_traffic_bytes_per_step()
                     if world == 1 and args.layers == 32 and args.shape == "llama3-8b" and args.batch == BATCH else None,
                     "algorithmic_bytes_per_step": wbytes, "launches_per_step": gemm_n // max(args.steps, 1),
                     "ms_per_step": gemm_chain_ms / args.steps,
                     "timing": "CUDA events around the step's projection launches run back to back on the launch "
                               "stream (dependent-launch overlap as in the step, other kernels left out)",
                     "serialised": {"achieved": gemm_gbs_serial, "frac": (gemm_gbs_serial / peak) if gemm_gbs_serial else None,
                                    "ms_per_step": gemm_ms / args.steps,
                                    "timing": "event pair around every single launch (no overlap between launches)"}},
        "roofline_attention": {"bound": "hbm", "kernel": "paged_decode_kernel", "achieved": attn_gbs, "peak": peak,
                               "unit": "GB/s", "frac": attn_gbs / peak,
                               "algorithmic_bytes_per_step": kbytes, "ms_per_step": attn_chain_ms / args.steps,
                               "serialised": {"achieved": attn_gbs_serial,
                                              "frac": (attn_gbs_serial / peak) if attn_gbs_serial else None,
                                              "ms_per_step": attn_ms / args.steps}},
        # whole step: every weight byte and every KV byte once per step over the device step time
        "roofline_step": {"bound": "hbm", "achieved": (wbytes + kbytes) / (ms_per_step / 1000.0) / 1e9,
                          "peak": peak, "unit": "GB/s",
                          "frac": (wbytes + kbytes) / (ms_per_step / 1000.0) / 1e9 / peak,
                          "algorithmic_bytes_per_step": wbytes + kbytes},
        "step_breakdown_ms": {k: v[0] / args.steps for k, v in prof.items()},
        "step_breakdown_note": "event pair around every launch in a separate pass: serialises the launches, so "
                               "the parts add up to more than ms_per_step",
    }
    if small:
        line["small_batch"] = small
    if parity is not None:
        line["tp_parity"] = parity
    if world == 1 and not args.no_attention_sweep:
        line["attention_microbench"] = attention_sweep(pkg, backend, peak)
    if world == 1 and not args.no_cpu_baseline and args.shape == "llama3-8b" and args.batch == BATCH:
        from oracle import binding as oracle

        oracle.build()
        t_layer, t_head = cpu_sample_step(oracle, 1, 16, np.random.default_rng(0))
        line["cpu_baseline"] = {
            "value": cpu_tokens_per_s(t_layer, t_head, 16), "unit": "tokens/s", "cores": 1, "kind": "port",
            "sample": "1 of 32 layers at 16 decode tokens (ctx 1024) + 1/16 of the LM head rows, single thread like "
                      "the reference's engine loop, extrapolated to 32 layers + full head"}
    print(json.dumps(line), file=json_out, flush=True)
    if dist is not None:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        print(f"tensor-parallel parity failed: {parity}", file=sys.stderr)
        return 1
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=("ours", "reference"), default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", choices=("decode", "serving", "prefix"), default="decode",
                    help="decode = the headline step (default); serving = continuous batching through the engine "
                         "loop; prefix = shared-prefix requests on the Qwen2-7B shape through the engine loop")
    ap.add_argument("--skip-cached-prefix", action="store_true",
                    help="engine workloads: start prefill after the tokens adopted from the prefix cache "
                         "(an extension; the reference shares the blocks but recomputes them)")
    ap.add_argument("--shape", choices=("llama3-8b", "llama3-70b"), default="llama3-8b",
                    help="decode workload: llama3-8b = the headline (batch 64, 1k contexts); llama3-70b = batch 128, "
                         "contexts U[1024,4096], meant for --gpus 2..8 (141 GB of weights)")
    ap.add_argument("--batch", type=int, default=BATCH,
                    help="sequences of the llama3-8b decode step; anything but 64 is not the headline")
    ap.add_argument("--requests", type=int, default=256, help="requests of the serving workload")
    ap.add_argument("--layers", type=int, default=32,
                    help="layers of the Llama-3-8B shape to build; fewer than 32 gives a small case with the "
                         "same per-launch kernel shapes, for profiler captures (not a benchmark number)")
    ap.add_argument("--no-small-batch", action="store_true",
                    help="skip the batch 1 / 8 / 16 steps that are appended at N=1")
    ap.add_argument("--no-attention-sweep", action="store_true",
                    help="skip the paged-attention microbenchmark sweep that is appended at N=1")
    ap.add_argument("--no-tp-parity", action="store_true",
                    help="N > 1: skip the parity check of the tensor-parallel path against the CPU oracle that "
                         "precedes the timed region (tuning runs)")
    ap.add_argument("--no-pdl", action="store_true", help="plain stream-ordered launches (tuning A/B)")
    ap.add_argument("--gemm-ctas", type=int, default=0, help="split-K CTA target (tuning A/B)")
    ap.add_argument("--gemm-stages", type=int, default=0, help="decode GEMM ring depth 3..4 (tuning A/B)")
    ap.add_argument("--attn-stages", type=int, default=0, help="decode attention ring depth 2..4 (tuning A/B)")
    ap.add_argument("--attn-ctas", type=int, default=0, help="decode attention CTA target (tuning A/B)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
