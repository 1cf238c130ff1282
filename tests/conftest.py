"""Shared fixtures: marker registration, import paths, oracle build, tiny models."""
import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box only)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding

    binding.build()
    binding.lib()
    return binding


@pytest.fixture(scope="session")
def kats():
    with open(os.path.join(ROOT, "tests", "golden", "reference_kats.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as ge

    return ge.load_package()


def sin_weights(rows, cols, seed):
    """The reference's deterministic test weights (transformer.rs:479-484)."""
    i = np.arange(rows * cols, dtype=np.float32)
    x = (i * np.float32(0.37) + np.float32(seed)).astype(np.float32)
    return (np.sin(x).astype(np.float32) * np.float32(0.5)).reshape(rows, cols)


def tiny_sin_tensors(num_layers, hidden=4, heads=2, kv_heads=1, head_dim=2, vocab=8, ffn=8):
    """Weights of the reference's tiny test model (transformer.rs:486-517); tied head."""
    q_dim, kv_dim = heads * head_dim, kv_heads * head_dim
    t = {"model.embed_tokens.weight": sin_weights(vocab, hidden, 0.5),
         "model.norm.weight": np.ones(hidden, np.float32)}
    for i in range(num_layers):
        p = f"model.layers.{i}"
        s = float(i)
        t[f"{p}.input_layernorm.weight"] = np.ones(hidden, np.float32)
        t[f"{p}.self_attn.q_proj.weight"] = sin_weights(q_dim, hidden, s + 1.0)
        t[f"{p}.self_attn.k_proj.weight"] = sin_weights(kv_dim, hidden, s + 2.0)
        t[f"{p}.self_attn.v_proj.weight"] = sin_weights(kv_dim, hidden, s + 3.0)
        t[f"{p}.self_attn.o_proj.weight"] = sin_weights(hidden, q_dim, s + 4.0)
        t[f"{p}.post_attention_layernorm.weight"] = np.ones(hidden, np.float32)
        t[f"{p}.mlp.gate_proj.weight"] = sin_weights(ffn, hidden, s + 5.0)
        t[f"{p}.mlp.up_proj.weight"] = sin_weights(ffn, hidden, s + 6.0)
        t[f"{p}.mlp.down_proj.weight"] = sin_weights(hidden, ffn, s + 7.0)
    return t


TINY_SIN_META = dict(hidden_size=4, num_attention_heads=2, num_kv_heads=1, head_dim=2,
                     vocab_size=8, ffn_dim=8, max_position_embeddings=32, rope_theta=10000.0,
                     rms_norm_eps=1e-5, tied_lm_head=True, num_blocks=16, block_size=4)


SMALL_META = dict(hidden_size=16, num_layers=2, num_attention_heads=4, num_kv_heads=2, head_dim=4,
                  vocab_size=32, ffn_dim=24, max_position_embeddings=64, rope_theta=10000.0,
                  rms_norm_eps=1e-5, has_qkv_bias=False, tied_lm_head=False, num_blocks=8,
                  block_size=4)


def random_tensors(rng, meta, std=0.3, norm_jitter=0.1):
    """Random f32 checkpoint with Hugging Face tensor names (transformer.rs:12-18)."""
    H, L, V, F = meta["hidden_size"], meta["num_layers"], meta["vocab_size"], meta["ffn_dim"]
    hd = meta["head_dim"]
    qd, kvd = meta["num_attention_heads"] * hd, meta["num_kv_heads"] * hd

    def mat(r, c):
        return (rng.standard_normal((r, c)) * std).astype(np.float32)

    def nrm():
        return (1 + norm_jitter * rng.standard_normal(H)).astype(np.float32)

    t = {"model.embed_tokens.weight": mat(V, H), "model.norm.weight": nrm()}
    if not meta.get("tied_lm_head"):
        t["lm_head.weight"] = mat(V, H)
    for i in range(L):
        p = f"model.layers.{i}"
        t[f"{p}.input_layernorm.weight"] = nrm()
        t[f"{p}.post_attention_layernorm.weight"] = nrm()
        t[f"{p}.self_attn.q_proj.weight"] = mat(qd, H)
        t[f"{p}.self_attn.k_proj.weight"] = mat(kvd, H)
        t[f"{p}.self_attn.v_proj.weight"] = mat(kvd, H)
        t[f"{p}.self_attn.o_proj.weight"] = mat(H, qd)
        if meta.get("has_qkv_bias"):
            t[f"{p}.self_attn.q_proj.bias"] = (rng.standard_normal(qd) * 0.1).astype(np.float32)
            t[f"{p}.self_attn.k_proj.bias"] = (rng.standard_normal(kvd) * 0.1).astype(np.float32)
            t[f"{p}.self_attn.v_proj.bias"] = (rng.standard_normal(kvd) * 0.1).astype(np.float32)
        t[f"{p}.mlp.gate_proj.weight"] = mat(F, H)
        t[f"{p}.mlp.up_proj.weight"] = mat(F, H)
        t[f"{p}.mlp.down_proj.weight"] = mat(H, F)
    return t
