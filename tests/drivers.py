"""Test-side batch drivers and checkpoint recipes (host only, no GPU needed)."""
from __future__ import annotations

import numpy as np

import __graft_entry__ as ge

# Configuration 1 of the benchmark definition: a tiny Llama-architecture model.
C1_META = dict(hidden_size=256, num_layers=2, num_attention_heads=4, num_kv_heads=2, head_dim=64,
               vocab_size=1024, ffn_dim=688, max_position_embeddings=256, rope_theta=10000.0,
               rms_norm_eps=1e-5, has_qkv_bias=False, tied_lm_head=False)


def c1_tensors(seed: int, meta: dict = C1_META, std: float = 0.02, bf16_round=None) -> dict:
    """Seeded random init: every matrix N(0, std), RMSNorm weights 1.0, separate lm_head."""
    rng = np.random.default_rng(seed)
    H, L, V, F, hd = (meta["hidden_size"], meta["num_layers"], meta["vocab_size"], meta["ffn_dim"],
                      meta["head_dim"])
    qd, kvd = meta["num_attention_heads"] * hd, meta["num_kv_heads"] * hd

    def mat(r, c):
        a = (rng.standard_normal((r, c)) * std).astype(np.float32)
        return bf16_round(a) if bf16_round else a

    t = {"model.embed_tokens.weight": mat(V, H), "lm_head.weight": mat(V, H),
         "model.norm.weight": np.ones(H, np.float32)}
    for i in range(L):
        p = f"model.layers.{i}"
        t[f"{p}.input_layernorm.weight"] = np.ones(H, np.float32)
        t[f"{p}.post_attention_layernorm.weight"] = np.ones(H, np.float32)
        t[f"{p}.self_attn.q_proj.weight"] = mat(qd, H)
        t[f"{p}.self_attn.k_proj.weight"] = mat(kvd, H)
        t[f"{p}.self_attn.v_proj.weight"] = mat(kvd, H)
        t[f"{p}.self_attn.o_proj.weight"] = mat(H, qd)
        t[f"{p}.mlp.gate_proj.weight"] = mat(F, H)
        t[f"{p}.mlp.up_proj.weight"] = mat(F, H)
        t[f"{p}.mlp.down_proj.weight"] = mat(H, F)
    return t


def softmax_rows(x: np.ndarray) -> np.ndarray:
    x = np.asarray(x, np.float64)
    e = np.exp(x - x.max(axis=-1, keepdims=True))
    return e / e.sum(axis=-1, keepdims=True)


class GreedyDriver:
    """Minimal continuous-batching driver: one prefill step for all sequences, then one decode
    token per sequence per step. Blocks come from a shuffled free list, so tables are scattered.
    Decode feeds the last generated token at position ``total_len - 1``."""

    def __init__(self, *, num_blocks: int, block_size: int, seed: int, num_sequences: int,
                 prompt_range=(32, 128), vocab: int = 1024):
        rng = np.random.default_rng(seed)
        self.block_size = block_size
        self.free = rng.permutation(num_blocks).tolist()
        self.prompts = [rng.integers(0, vocab, int(rng.integers(prompt_range[0], prompt_range[1] + 1))).tolist()
                        for _ in range(num_sequences)]
        self.generated = [[] for _ in range(num_sequences)]
        self.tables = [[] for _ in range(num_sequences)]
        self.prefilled = False
        self.pkg = ge.load_package()

    def _ensure(self, s: int, total_len: int) -> None:
        need = (total_len + self.block_size - 1) // self.block_size
        while len(self.tables[s]) < need:
            self.tables[s].append(self.free.pop(0))

    def next_batch(self):
        n = len(self.prompts)
        tokens, positions, counts, ctx = [], [], [], []
        if not self.prefilled:
            for s, p in enumerate(self.prompts):
                self._ensure(s, len(p))
                tokens += p
                positions += list(range(len(p)))
                counts.append(len(p))
                ctx.append(len(p))
            self.prefilled = True
            has_prefill = True
        else:
            for s in range(n):
                total = len(self.prompts[s]) + len(self.generated[s])
                self._ensure(s, total)
                tokens.append(self.generated[s][-1])
                positions.append(total - 1)
                counts.append(1)
                ctx.append(total)
            has_prefill = False
        return self.pkg.ForwardBatch(tokens, positions, list(range(1, n + 1)), counts, ctx,
                                     [list(t) for t in self.tables], has_prefill=has_prefill)

    def accept(self, token_ids) -> None:
        for s, t in enumerate(token_ids):
            self.generated[s].append(int(t))
