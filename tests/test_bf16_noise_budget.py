"""Where the logit noise of a bf16 build comes from, on the configuration-1 model (host only).

The benchmark definition asks the bf16 build for identical greedy tokens over 32 steps. With the
prescribed random initialisation (N(0, 0.02) matrices) the logits of that model are nearly flat
(standard deviation 0.32 over 1024 entries) and the oracle's own top-2 gaps go down to 1e-3 and
below, so the question is how much a logit may move for reasons no kernel can avoid. This test
restates the model's forward in numpy (same operation order as the oracle at f32) and rounds to
bf16 at one storage site at a time:

  normed / attn / act / tail  activations that feed the projections (a build could carry them wider)
  q, p                        query and softmax weights inside attention
  kv                          the KV cache itself, which a bf16 build stores in bf16 by definition

What it pins: rounding the stored keys and values alone already moves logits by more than 1e-3, and
carrying every projection input at twice the precision (a hi + lo bf16 pair) removes less than two
thirds of the total noise. Identical tokens at oracle gaps below ~5e-3 are therefore not something
a bf16-KV build can promise; the GPU parity test allows a different token only below that gap.
"""
import numpy as np

from drivers import C1_META, c1_tensors


def round_bf16(a):
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(np.float32)


def hi_lo(a):
    hi = round_bf16(a)
    return hi + round_bf16(a - hi)


def forward(w, m, tokens, rounding):
    """Prefill of one sequence; logits of every row. `rounding` maps a site name to a rounding function."""
    H, L, hd, Hq, Hkv = m["hidden_size"], m["num_layers"], m["head_dim"], m["num_attention_heads"], m["num_kv_heads"]
    f = lambda site, a: rounding[site](a) if site in rounding else a  # noqa: E731
    T, half = len(tokens), hd // 2
    pos = np.arange(T, dtype=np.float32)
    inv = 1.0 / np.power(np.float32(m["rope_theta"]), np.arange(half, dtype=np.float32) * 2 / hd)
    cos, sin = np.cos(pos[:, None] * inv)[:, None, :], np.sin(pos[:, None] * inv)[:, None, :]

    def rope(x):
        x0, x1 = x[..., :half], x[..., half:]
        return np.concatenate([x0 * cos - x1 * sin, x0 * sin + x1 * cos], -1).astype(np.float32)

    def rms(x, g):
        ss = (x.astype(np.float64) ** 2).mean(-1, keepdims=True)
        return ((x * (1.0 / np.sqrt(ss + m["rms_norm_eps"])).astype(np.float32)) * g).astype(np.float32)

    causal = np.tril(np.ones((T, T), bool))
    h = w["model.embed_tokens.weight"][tokens].astype(np.float32)
    for layer in range(L):
        p = f"model.layers.{layer}."
        n = f("normed", rms(h, w[p + "input_layernorm.weight"]))
        q = f("q", rope((n @ w[p + "self_attn.q_proj.weight"].T).reshape(T, Hq, hd)))
        k = f("kv", rope((n @ w[p + "self_attn.k_proj.weight"].T).reshape(T, Hkv, hd)))
        v = f("kv", (n @ w[p + "self_attn.v_proj.weight"].T).reshape(T, Hkv, hd))
        out = np.zeros((T, Hq, hd), np.float32)
        for head in range(Hq):
            kh = head // (Hq // Hkv)
            s = np.where(causal, (q[:, head] @ k[:, kh].T) / np.sqrt(np.float32(hd)), -np.inf)
            e = np.exp(s - s.max(-1, keepdims=True)).astype(np.float32)
            out[:, head] = (f("p", e) @ v[:, kh]) / e.sum(-1, keepdims=True)
        h = h + f("attn", out.reshape(T, Hq * hd)) @ w[p + "self_attn.o_proj.weight"].T
        n = f("normed", rms(h, w[p + "post_attention_layernorm.weight"]))
        g, u = n @ w[p + "mlp.gate_proj.weight"].T, n @ w[p + "mlp.up_proj.weight"].T
        h = h + f("act", (g / (1 + np.exp(-g)) * u).astype(np.float32)) @ w[p + "mlp.down_proj.weight"].T
    return f("tail", rms(h, w["model.norm.weight"])) @ w["lm_head.weight"].T


def test_bf16_kv_storage_alone_explains_greedy_flips_at_small_oracle_gaps():
    m = dict(C1_META, head_dim=128)
    w = c1_tensors(seed=1234, meta=m, bf16_round=round_bf16)
    tokens = np.random.default_rng(0).integers(0, m["vocab_size"], 128)
    exact = forward(w, m, tokens, {})
    srt = np.sort(exact, axis=1)
    gaps = srt[:, -1] - srt[:, -2]
    assert 0.25 < exact.std() < 0.4 and gaps.min() < 2e-3, "flat logits with near-ties, as the random init gives"

    def noise(rounding):
        d = forward(w, m, tokens, rounding) - exact
        return float(np.abs(d).max()), float(np.sqrt((d ** 2).mean()))

    sites = ["normed", "q", "kv", "p", "attn", "act", "tail"]
    all_max, all_rms = noise({s: round_bf16 for s in sites})
    kv_max, kv_rms = noise({"kv": round_bf16})
    wide = {s: round_bf16 for s in sites}
    wide.update({s: hi_lo for s in ("normed", "attn", "act", "tail")})
    wide_max, wide_rms = noise(wide)
    assert 3e-3 < all_max < 1.2e-2 and 8e-4 < all_rms < 2e-3       # every site in bf16: ~6e-3 max, ~1.2e-3 rms
    assert kv_max > 1.5e-3 and kv_rms > 3e-4                       # the KV cache alone: ~2.5e-3 max, ~5.5e-4 rms
    assert wide_rms > all_rms / 3 and wide_max > all_max / 3       # wider projection inputs remove < 2/3 of it
    assert 2 * kv_max > gaps.min(), "two logits this close can swap under bf16 KV storage alone"
