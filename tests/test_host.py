"""Host-side logic and the C-ABI surface; runs without a GPU (no compute calls)."""
import ctypes
import json
import os
import re

import numpy as np
import pytest

from conftest import ROOT


def test_library_exports_every_symbol_the_header_declares(pkg):
    header = open(os.path.join(ROOT, "include", "orion_cuda.h")).read()
    declared = set(re.findall(r"\b(orion_cuda_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 35
    lib = ctypes.CDLL(pkg._ffi.LIB_PATH)
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert declared == set(pkg._ffi.SIGNATURES), "the ctypes table and the header must list the same symbols"
    pkg._ffi.lib()


def test_library_exports_every_driver_symbol_the_header_declares(pkg):
    header = open(os.path.join(ROOT, "include", "orion_driver.h")).read()
    declared = set(re.findall(r"\b(orion_(?:hash_block|sequence_id|kv_manager|scheduler|engine)[a-z0-9_]*)\s*\(", header))
    assert len(declared) >= 40
    lib = ctypes.CDLL(pkg._ffi.LIB_PATH)
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"
    assert declared == set(pkg._ffi.DRIVER_SIGNATURES), "the ctypes table and the header must list the same symbols"


def test_without_a_device_construction_fails_loudly(pkg):
    if pkg.is_available():
        pytest.skip("a CUDA device is present")
    assert pkg.device_count() == 0
    with pytest.raises(pkg.CudaUnavailable):
        pkg.CudaBackend(0)


def test_tolerance_semantics(pkg, kats):
    t = kats["tolerance"]
    assert (pkg.Tolerance.F32.abs, pkg.Tolerance.F32.rel) == (t["F32"]["abs"], t["F32"]["rel"])
    assert (pkg.Tolerance.F16.abs, pkg.Tolerance.F16.rel) == (t["F16"]["abs"], t["F16"]["rel"])
    tol = pkg.Tolerance.F32
    assert tol.matches(1.0, 1.0 + 5e-6) and not tol.matches(1.0, 1.001)
    assert tol.matches(1e6, 1e6 + 5.0), "relative tolerance carries large values"
    assert tol.matches(0.0, 5e-6), "absolute tolerance carries values near zero"
    assert tol.matches(float("nan"), float("nan")) and not tol.matches(float("nan"), 1.0)
    assert tol.matches(float("inf"), float("inf")) and not tol.matches(float("inf"), float("-inf"))
    rep = pkg.validate("k", [1.0, 2.0, 3.0], [1.0, 2.5, 3.0], tol)
    assert not rep.passed() and rep.mismatches == 1 and rep.worst_index == 1 and "FAIL" in rep.render()
    assert pkg.validate("k", [1.0], [1.0], tol).passed()
    with pytest.raises(pkg.InternalError):
        pkg.validate("k", [1.0, 2.0], [1.0], tol)


def test_tp_calculus_matches_the_reference_tests(pkg, kats):
    k = kats["tp_layout"]
    m = k["llama3_8b"]
    meta = pkg.ModelMetadata(architecture="llama", name="8b", hidden_size=m["hidden_size"],
                             num_layers=m["num_layers"], num_attention_heads=m["num_attention_heads"],
                             num_kv_heads=m["num_kv_heads"], head_dim=m["head_dim"], vocab_size=128256,
                             dtype=pkg.DType.F16)
    with pytest.raises(pkg.InvalidRequest):
        pkg.Rank(4, 4)
    with pytest.raises(pkg.InvalidRequest):
        pkg.Rank(0, 0)
    assert pkg.Rank.single().is_leader() and not pkg.Rank.single().is_distributed()
    shards = [pkg.shard_dimension(32, pkg.Rank(i, 4)) for i in range(4)]
    assert shards[0] == pkg.Shard(0, 8) and shards[3] == pkg.Shard(24, 8)
    assert all(a.end() == b.start for a, b in zip(shards, shards[1:]))
    with pytest.raises(pkg.InvalidRequest, match="30"):
        pkg.shard_dimension(30, pkg.Rank(0, 4))
    for compute in (pkg.ParallelLayout.compute, pkg.ParallelLayout.compute_native):
        one = compute(meta, pkg.Rank.single(), m["ffn_dim"])
        assert (one.query_heads.len, one.kv_heads.len, one.ffn.len) == (32, 8, 14336)
        r1 = compute(meta, pkg.Rank(1, 2), m["ffn_dim"])
        exp = k["world2_rank1"]
        assert [r1.query_heads.start, r1.query_heads.len] == exp["query_heads"]
        assert [r1.kv_heads.start, r1.kv_heads.len] == exp["kv_heads"]
        assert [r1.ffn.start, r1.ffn.len] == exp["ffn"]
        assert compute(meta, pkg.Rank(0, 8), m["ffn_dim"]).kv_heads.len == 1
        with pytest.raises(pkg.InvalidRequest, match="KV heads"):
            compute(meta, pkg.Rank(0, 16), m["ffn_dim"])
        q = compute(meta, pkg.Rank(0, 4), m["ffn_dim"])
        assert q.local_attention_dim(meta.head_dim) == 1024
        assert q.local_kv_bytes_per_token(meta) * 4 == meta.kv_bytes_per_token()
    assert pkg.CommunicationEstimate.for_model(meta, 1) == pkg.CommunicationEstimate(0, 0)
    two, eight = pkg.CommunicationEstimate.for_model(meta, 2), pkg.CommunicationEstimate.for_model(meta, 8)
    assert two.all_reduce_count == eight.all_reduce_count == k["all_reduce_count_world2"]
    assert eight.bytes_per_token > two.bytes_per_token > 100_000


def test_single_rank_collectives_are_identities(pkg):
    c = pkg.SingleRank()
    buf = np.array([1.0, 2.0, 3.0], np.float32)
    c.all_reduce_sum(buf)
    assert buf.tolist() == [1.0, 2.0, 3.0]
    out = np.zeros(3, np.float32)
    c.all_gather(buf, out)
    assert out.tolist() == buf.tolist()
    c.reduce_scatter_sum(buf, out)
    c.barrier()
    with pytest.raises(pkg.InternalError):
        c.all_gather(buf[:2], out)
    with pytest.raises(pkg.InternalError):
        c.reduce_scatter_sum(buf[:2], out)


def test_forward_batch_validation_and_flattening(pkg):
    b = pkg.ForwardBatch([1, 2, 3, 4], [0, 1, 2, 0], [1, 2], [3, 1], [3, 1], [[0], [1]])
    b.validate()
    assert b.num_sequences() == 2 and b.num_tokens() == 4 and not b.is_empty()
    tokens, positions, counts, ctx, flat, offs = b.flatten()
    assert offs.tolist() == [0, 1, 2] and flat[:2].tolist() == [0, 1]
    for mutate in (lambda x: x.context_lens.pop(), lambda x: x.positions.pop(),
                   lambda x: setattr(x, "slot_token_counts", [2, 1])):
        bad = pkg.ForwardBatch([1, 2, 3, 4], [0, 1, 2, 0], [1, 2], [3, 1], [3, 1], [[0], [1]])
        mutate(bad)
        with pytest.raises(pkg.InternalError):
            bad.validate()
    out = pkg.ForwardOutput(np.zeros(6, np.float32), 3, [1, 2])
    assert out.row(0).size == 3 and out.row(1).size == 3 and out.row(2) is None


def test_metadata_and_dtype_arithmetic(pkg):
    assert pkg.DType.I4.size_in_bytes(3) == 2 and pkg.DType.F16.size_in_bytes(4) == 8
    m = pkg.ModelMetadata("LlamaForCausalLM", "t", 4096, 32, 32, 8, 128, 32000, dtype=pkg.DType.F16)
    assert m.kv_bytes_per_token() == 2 * 32 * 8 * 128 * 2 and m.uses_gqa() and m.gqa_group_size() == 4
    assert str(pkg.Device("cuda", 1)) == "cuda:1" and pkg.Device("cpu").is_cpu()


def test_hf_config_defaults_and_aliases(pkg):
    cfg = pkg.HfConfig.from_dict({"architectures": ["LlamaForCausalLM"], "hidden_size": 64, "n_layer": 2,
                                  "n_head": 4, "vocab_size": 100, "unknown_field": 1})
    meta = cfg.to_metadata("m")
    assert (meta.num_kv_heads, meta.head_dim, meta.max_position_embeddings, meta.rope_theta,
            meta.rms_norm_eps, meta.ffn_dim) == (4, 16, 2048, 10000.0, 1e-5, 256)
    assert not meta.has_qkv_bias and not meta.tied_lm_head
    q = pkg.HfConfig.from_dict({"model_type": "qwen2", "hidden_size": 64, "num_hidden_layers": 1,
                                "num_attention_heads": 4, "num_key_value_heads": 2, "vocab_size": 10,
                                "torch_dtype": "bfloat16", "eos_token_id": [1, 2], "tie_word_embeddings": True})
    qm = q.to_metadata("q")
    assert qm.has_qkv_bias and qm.tied_lm_head and qm.dtype == pkg.DType.BF16 and qm.eos_token_ids == [1, 2]
    with pytest.raises(pkg.ModelError):
        pkg.HfConfig.from_dict({"architectures": ["GPT2"], "hidden_size": 1, "num_hidden_layers": 1,
                                "num_attention_heads": 1, "vocab_size": 1}).to_metadata("x")
    with pytest.raises(pkg.ModelError):
        pkg.HfConfig.from_dict({"model_type": "llama", "hidden_size": 64, "num_hidden_layers": 1,
                                "num_attention_heads": 4, "num_key_value_heads": 3, "vocab_size": 1}).to_metadata("x")


def test_safetensors_round_trip(pkg, oracle, tmp_path):
    rng = np.random.default_rng(0)
    t = {"a.weight": rng.standard_normal((3, 5)).astype(np.float32), "b": np.arange(4, dtype=np.float32)}
    p = str(tmp_path / "m.safetensors")
    pkg.write_safetensors(p, t)
    back = pkg.read_safetensors(p)
    assert back["a.weight"][0] == pkg.DType.F32 and back["a.weight"][1] == (3, 5)
    assert np.array_equal(back["a.weight"][2].reshape(3, 5), t["a.weight"])
    pkg.write_safetensors(p, t, dtype=pkg.DType.BF16)
    back = pkg.read_safetensors(p)
    assert back["a.weight"][0] == pkg.DType.BF16
    assert np.array_equal(back["a.weight"][2], oracle.f32_to_bf16(t["a.weight"]).reshape(-1))


def test_greedy_driver_is_deterministic_and_consistent():
    from drivers import GreedyDriver

    a = GreedyDriver(num_blocks=64, block_size=16, seed=3, num_sequences=4, prompt_range=(5, 40), vocab=50)
    b = GreedyDriver(num_blocks=64, block_size=16, seed=3, num_sequences=4, prompt_range=(5, 40), vocab=50)
    ba, bb = a.next_batch(), b.next_batch()
    ba.validate()
    assert ba.tokens == bb.tokens and ba.block_tables == bb.block_tables
    used = [blk for t in ba.block_tables for blk in t]
    assert len(used) == len(set(used)), "no block is handed out twice"
    a.accept([1, 2, 3, 4])
    d = a.next_batch()
    d.validate()
    assert d.slot_token_counts == [1] * 4 and not d.has_prefill
    assert d.positions == [len(p) for p in a.prompts]
    for s in range(4):
        assert len(d.block_tables[s]) * 16 >= d.context_lens[s]


def test_nccl_failures_abort_the_communicator_and_surface_as_backend_errors(pkg):
    """The failure handling of the NCCL leg, on the host against a stand-in NCCL (no GPU, no library):
    a rank that never joins, a peer that dies during a step and a step that never ends must each end
    in ncclCommAbort and EngineError::Backend within the time limit; a healthy group must not."""
    import time

    lib = pkg._ffi.lib()
    aborted, polls = ctypes.c_uint32(7), ctypes.c_uint64(0)
    assert lib.orion_cuda_tp_selftest_failure_handling(0, 200, ctypes.byref(aborted), ctypes.byref(polls)) == 0, \
        pkg._ffi.last_error()
    assert aborted.value == 0 and polls.value >= 4  # the rendezvous was polled until every rank had joined
    for scenario, text in ((1, "did not answer within the time limit"), (2, "remote process exited"),
                           (3, "did not end within the time limit")):
        t0 = time.monotonic()
        rc = lib.orion_cuda_tp_selftest_failure_handling(scenario, 150, ctypes.byref(aborted), ctypes.byref(polls))
        took = time.monotonic() - t0
        assert rc == pkg._ffi.ERR_BACKEND, (scenario, rc, pkg._ffi.last_error())
        msg = pkg._ffi.last_error()
        assert text in msg and "communicator aborted" in msg and msg.startswith("backend cuda failed at "), msg
        assert aborted.value == 1 and polls.value > 0
        assert took < 5.0, f"scenario {scenario} took {took:.2f} s with a 150 ms limit"
    assert lib.orion_cuda_tp_selftest_failure_handling(9, 10, None, None) == pkg._ffi.ERR_INVALID_REQUEST
