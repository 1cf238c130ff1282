"""Pins the CPU oracle against the reference's own known-answer tests."""
import math

import numpy as np
import pytest

from conftest import TINY_SIN_META, tiny_sin_tensors


def _close(a, b, tol):
    return np.all(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)) < tol)


def test_linear_kats(oracle, kats):
    for k in kats["linear"]:
        out = oracle.linear(np.array(k["x"]), np.array(k["w"]), k["bias"])
        assert out.shape == np.array(k["out"]).shape
        assert np.array_equal(out, np.array(k["out"], np.float32)), k["cite"]


def test_linear_shape_errors(oracle, kats):
    for k in kats["linear_errors"]:
        x, w = np.ones(k["x_shape"]), np.ones(k["w_shape"])
        bias = None if k["bias_len"] is None else np.ones(k["bias_len"])
        with pytest.raises(oracle.OracleInternalError):
            oracle.linear(x, w, bias)


def test_linear_threads_are_bit_identical(oracle):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((7, 300)).astype(np.float32)
    w = rng.standard_normal((129, 300)).astype(np.float32)
    b = rng.standard_normal(129).astype(np.float32)
    oracle.set_threads(1)
    one = oracle.linear(x, w, b)
    oracle.set_threads(5)
    many = oracle.linear(x, w, b)
    oracle.set_threads(1)
    assert np.array_equal(one, many)
    # sequential f32 accumulation, k ascending, no FMA
    acc = np.float32(0)
    for t in range(300):
        acc = np.float32(acc + np.float32(x[3, t] * w[17, t]))
    assert one[3, 17] == np.float32(acc + b[17])


def test_rms_norm_kats(oracle, kats):
    for k in kats["rms_norm"]:
        out = oracle.rms_norm(np.array(k["x"]), k["w"], k["eps"])
        assert _close(out, k["out"], k["tol"]), k["cite"]
    k = kats["rms_norm_rows_equal"]
    out = oracle.rms_norm(np.array(k["x"]), k["w"], k["eps"])
    assert abs(out[0, 0] - out[1, 0]) < k["tol"]
    k = kats["rms_norm_zero_row_finite"]
    assert np.all(np.isfinite(oracle.rms_norm(np.array(k["x"]), k["w"], k["eps"])))
    with pytest.raises(oracle.OracleInternalError):  # tensor.rs:401-404
        oracle.rms_norm(np.ones((1, 4)), [1.0, 1.0], 1e-5)


def test_rms_norm_recipe_is_f64_sum_then_two_f32_multiplies(oracle):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 257)).astype(np.float32)
    w = rng.standard_normal(257).astype(np.float32)
    out = oracle.rms_norm(x, w, 1e-5)
    for r in range(3):
        ss = 0.0
        for v in x[r]:
            ss += float(v) * float(v)
        scale = np.float32(1.0 / math.sqrt(ss / 257 + float(np.float32(1e-5))))
        exp = (x[r] * scale).astype(np.float32) * w
        assert np.array_equal(out[r], exp.astype(np.float32))


def test_silu_and_swiglu_kats(oracle, kats):
    for k in kats["silu"]:
        assert abs(oracle.silu(k["x"]) - k["y"]) < k["tol"], k["cite"]
    k = kats["silu_negative_range"]
    assert k["lo"] < oracle.silu(k["x"]) < k["hi"]
    k = kats["swiglu"]
    assert _close(oracle.swiglu(np.array(k["gate"]), np.array(k["up"])), k["out"], k["tol"])
    with pytest.raises(oracle.OracleInternalError):  # tensor.rs:428-432
        oracle.swiglu(np.zeros((1, 2)), np.zeros((1, 3)))


def test_softmax_kats(oracle, kats):
    for k in kats["softmax"]:
        p = oracle.softmax(k["x"])
        assert np.all(np.isfinite(p)) and abs(p.sum() - k["sum"]) < k["tol"]
        assert np.all(np.diff(p) > 0)
    # tensor.rs:194-198: a non-finite maximum gives the uniform distribution
    assert np.allclose(oracle.softmax([-np.inf, -np.inf]), [0.5, 0.5])


def test_rope_kats(oracle, kats):
    k = kats["rope_pairing"]
    assert _close(oracle.apply_rope(k["vec"], k["cos"], k["sin"]), k["out"], k["tol"])
    k = kats["rope_table_pos0"]
    cos, sin = oracle.rope_table(k["head_dim"], k["max_positions"], k["theta"])
    assert cos.shape == (8, 2)
    assert _close(cos[0], k["cos0"], k["tol"]) and _close(sin[0], k["sin0"], k["tol"])
    with pytest.raises(oracle.OracleInternalError):  # tensor.rs:461-463
        oracle.rope_table(3, 8, 10000.0)
    with pytest.raises(oracle.OracleInternalError):  # tensor.rs:533-536
        oracle.apply_rope(np.ones(4), [1.0], [0.0])
    k = kats["rope_norm"]
    cos, sin = oracle.rope_table(k["head_dim"], k["max_positions"], k["theta"])
    v = np.array(k["vec"], np.float32)
    r = oracle.apply_rope(v, cos[k["pos"]], sin[k["pos"]])
    assert abs(np.linalg.norm(v) - np.linalg.norm(r)) < k["tol"]
    k = kats["rope_relative"]
    cos, sin = oracle.rope_table(k["head_dim"], k["max_positions"], k["theta"])
    base = np.arange(1, 9, dtype=np.float32) * np.float32(0.1)
    rot = lambda p: oracle.apply_rope(base, cos[p], sin[p])
    d = [float(np.dot(rot(a), rot(b))) for a, b in k["pairs"]]
    assert abs(d[0] - d[1]) < k["tol"]
    # position 0 is the identity (tensor.rs:466-475)
    cos, sin = oracle.rope_table(4, 4, 10000.0)
    assert _close(oracle.apply_rope([1, 2, 3, 4], cos[0], sin[0]), [1, 2, 3, 4], 1e-6)


def test_rope_table_recipe(oracle):
    cos, sin = oracle.rope_table(64, 40, 10000.0)
    for pos in (1, 17, 39):
        for i in (0, 5, 31):
            inv = np.float32(1.0) / np.float32(np.power(np.float32(10000.0),
                                                         np.float32(np.float32(2.0 * i) / np.float32(64))))
            ang = np.float32(pos) * inv
            assert abs(cos[pos, i] - math.cos(float(ang))) < 1e-5
            assert abs(sin[pos, i] - math.sin(float(ang))) < 1e-5


def test_locate_kats(oracle, kats):
    for k in kats["locate"]:
        for pos, exp in k["cases"]:
            got = oracle.locate(k["table"], pos, k["block_size"])
            assert got == (tuple(exp) if exp is not None else None), k["cite"]


def test_kv_store_layout_and_bounds(oracle, kats):
    k = kats["kv_store"]
    s = oracle.KvStore(*k["dims"])
    assert len(s) == k["len"]
    assert not s.array().any(), "the arena starts zeroed (attention.rs:55)"
    s.write(1, 2, 1, 0, False, [1, 2, 3, 4])
    assert s.read(1, 2, 1, 0, False).tolist() == [1, 2, 3, 4]
    # [layer][block][k|v][slot][head][dim]
    assert s.array()[1, 2, 0, 1, 0].tolist() == [1, 2, 3, 4]
    s.write(0, 0, 0, 0, True, [2, 2, 2, 2])
    assert s.read(0, 0, 0, 0, False)[0] == 0.0 and s.read(0, 0, 0, 0, True)[0] == 2.0
    for args in ((9, 0, 0, 0), (0, 9, 0, 0), (0, 0, 9, 0), (0, 0, 0, 9)):
        with pytest.raises(oracle.OracleInternalError):
            s.write(*args, False, [0, 0, 0, 0])
    with pytest.raises(oracle.OracleInternalError):
        s.write(0, 0, 0, 0, False, [0, 0, 0])


def _run_attention(oracle, k):
    s = oracle.KvStore(*k["store"])
    for layer, block, slot, head, is_v, vec in k.get("writes", []):
        s.write(layer, block, slot, head, is_v, vec)
    return oracle.paged_attention(s, k["query"], k["table"], k["query_position"], 0, k.get("hq", 1),
                                  k.get("hkv", 1), k.get("hd", 2), k["bs"])


def test_attention_kats(oracle, kats):
    for k in kats["attention"]:
        out = _run_attention(oracle, k)
        if k.get("exact"):
            assert out.tolist() == k["out"], k["cite"]
        else:
            assert _close(out, k["out"], k["tol"]), k["cite"]
    k = kats["attention_favours_similar"]
    out = _run_attention(oracle, k)
    assert out[1] > k["out1_gt"] and out[0] < k["out0_lt"]


def test_attention_convex_and_scattered(oracle, kats):
    k = kats["attention_convex"]
    s = oracle.KvStore(*k["store"])
    for pos in range(4):
        s.write(0, 0, pos, 0, False, [float(pos), 0.0])
        s.write(0, 0, pos, 0, True, [pos * 10.0, 1.0])
    out = oracle.paged_attention(s, k["query"], k["table"], k["query_position"], 0, 1, 1, 2, k["bs"])
    assert k["range0"][0] <= out[0] <= k["range0"][1] and abs(out[1] - k["out1"]) < k["tol"]
    k = kats["attention_scattered"]
    outs = []
    for table in k["tables"]:
        s = oracle.KvStore(*k["store"])
        for pos in range(4):
            b, slot = oracle.locate(table, pos, k["bs"])
            s.write(0, b, slot, 0, False, [pos * 0.5, 1.0])
            s.write(0, b, slot, 0, True, [float(pos), 2.0])
        outs.append(oracle.paged_attention(s, k["query"], table, k["query_position"], 0, 1, 1, 2,
                                           k["bs"]))
    assert _close(outs[0], outs[1], k["tol"])


def test_attention_errors(oracle, kats):
    for k in kats["attention_errors"]:
        s = oracle.KvStore(*k["store"])
        with pytest.raises(oracle.OracleInternalError):
            oracle.paged_attention(s, np.zeros(k["query_len"]), k["table"], k["query_position"], 0,
                                   k["hq"], k["hkv"], k["hd"], k["bs"])


def test_argmax_kats(oracle, kats):
    for k in kats["argmax"]:
        assert oracle.argmax([float(v) for v in k["logits"]]) == k["index"], k["cite"]


def test_widening_matches_numpy(oracle):
    rng = np.random.default_rng(3)
    f = rng.standard_normal(1000).astype(np.float32)
    bits = oracle.f32_to_bf16(f)
    wide = oracle.bf16_to_f32(bits)
    assert np.array_equal(wide.view(np.uint32), bits.astype(np.uint32) << 16)
    assert np.max(np.abs(wide - f) / np.abs(f)) < 2 ** -8
    h = rng.standard_normal(1000).astype(np.float16)
    h[:4] = [0.0, 6e-8, -6e-5, np.inf]
    assert np.array_equal(oracle.f16_to_f32(h.view(np.uint16)), h.astype(np.float32))


# ---- transformer.rs invariants on the reference's tiny sin-weight model ----

def _tiny(oracle, layers):
    return oracle.Model(num_layers=layers, **TINY_SIN_META).load(tiny_sin_tensors(layers))


def _one(oracle, tokens, positions, blocks, ctx=None):
    n = len(tokens)
    return oracle.Batch(tokens, positions, [n], [ctx or n], [blocks])


def test_tiny_model_shapes_and_errors(oracle):
    m = _tiny(oracle, 2)
    out = m.forward(_one(oracle, [1, 2, 3], [0, 1, 2], [0]))
    assert out.shape == (1, 8) and np.all(np.isfinite(out))
    assert _tiny(oracle, 1).forward(_one(oracle, [1, 2, 3, 4, 5], [0, 1, 2, 3, 4], [0, 1])).shape == (1, 8)
    assert m.forward(oracle.Batch([], [], [], [], [])).shape == (0, 8)
    two = m.forward(oracle.Batch([1, 2, 3, 4], [0, 1, 0, 1], [2, 2], [2, 2], [[0], [1]]))
    assert two.shape == (2, 8)
    m1 = _tiny(oracle, 1)
    with pytest.raises(oracle.OracleInternalError):  # transformer.rs:770-776
        m1.forward(_one(oracle, [999], [0], [0]))
    with pytest.raises(oracle.OracleInternalError):  # transformer.rs:779-793
        m1.forward(_one(oracle, [1], [100], list(range(26))))
    bad = _one(oracle, [1, 2], [0, 1], [0])
    bad.slot_token_counts = [5]
    with pytest.raises(oracle.OracleInternalError):  # transformer.rs:796-801
        m1.forward(bad)
    with pytest.raises(oracle.OracleInternalError):  # transformer.rs:380-385: no block for position 4
        m1.forward(_one(oracle, [1], [4], [0]))


def test_tiny_model_invariants(oracle, kats):
    tol = {i["name"]: i["tol"] for i in kats["tiny_model"]["invariants"]}
    # batch independence
    m = _tiny(oracle, 2)
    alone = m.forward(_one(oracle, [1, 2], [0, 1], [0]))[0]
    together = m.forward(oracle.Batch([1, 2, 5, 6, 7], [0, 1, 0, 1, 2], [2, 3], [2, 3], [[0], [4]]))[0]
    assert _close(alone, together, tol["batch_independence"])
    # incremental decode == full prefill
    full = _tiny(oracle, 2).forward(_one(oracle, [1, 2, 3], [0, 1, 2], [0]))[0]
    m = _tiny(oracle, 2)
    m.forward(_one(oracle, [1, 2], [0, 1], [0]))
    inc = m.forward(oracle.Batch([3], [2], [1], [3], [[0]], has_prefill=False))[0]
    assert _close(full, inc, tol["incremental_decode_matches_full_prefill"])
    # chunked prefill == single pass
    whole = _tiny(oracle, 2).forward(_one(oracle, [1, 2, 3, 4], [0, 1, 2, 3], [0]))[0]
    m = _tiny(oracle, 2)
    m.forward(_one(oracle, [1, 2], [0, 1], [0]))
    chunked = m.forward(oracle.Batch([3, 4], [2, 3], [2], [4], [[0]]))[0]
    assert _close(whole, chunked, tol["chunked_prefill_matches_single_pass"])
    # scattered block table
    a = _tiny(oracle, 2).forward(_one(oracle, [1, 2, 3, 4, 5], [0, 1, 2, 3, 4], [0, 1]))[0]
    b = _tiny(oracle, 2).forward(_one(oracle, [1, 2, 3, 4, 5], [0, 1, 2, 3, 4], [11, 3]))[0]
    assert _close(a, b, tol["scattered_block_table_identical"])
    # the model reads its input (transformer.rs:749-767)
    m = _tiny(oracle, 2)
    x = m.forward(_one(oracle, [1, 1, 1], [0, 1, 2], [0]))[0]
    y = m.forward(_one(oracle, [5, 6, 4], [0, 1, 2], [2]))[0]
    assert np.any(np.abs(x - y) > 1e-4)


def test_forward_matches_a_numpy_restatement(oracle):
    """Independent float64 numpy forward on a small random model (guards the C plumbing)."""
    rng = np.random.default_rng(7)
    H, L, Hq, Hkv, hd, V, F, B = 16, 2, 4, 2, 4, 32, 24, 4
    t = {"model.embed_tokens.weight": rng.standard_normal((V, H)) * 0.5,
         "model.norm.weight": 1 + 0.1 * rng.standard_normal(H),
         "lm_head.weight": rng.standard_normal((V, H)) * 0.5}
    for i in range(L):
        p = f"model.layers.{i}"
        t[f"{p}.input_layernorm.weight"] = 1 + 0.1 * rng.standard_normal(H)
        t[f"{p}.post_attention_layernorm.weight"] = 1 + 0.1 * rng.standard_normal(H)
        for n, shape in (("q", (Hq * hd, H)), ("k", (Hkv * hd, H)), ("v", (Hkv * hd, H)),
                         ("o", (H, Hq * hd))):
            t[f"{p}.self_attn.{n}_proj.weight"] = rng.standard_normal(shape) * 0.3
        for n in "qkv":
            t[f"{p}.self_attn.{n}_proj.bias"] = rng.standard_normal((Hq if n == "q" else Hkv) * hd) * 0.1
        t[f"{p}.mlp.gate_proj.weight"] = rng.standard_normal((F, H)) * 0.3
        t[f"{p}.mlp.up_proj.weight"] = rng.standard_normal((F, H)) * 0.3
        t[f"{p}.mlp.down_proj.weight"] = rng.standard_normal((H, F)) * 0.3
    t = {k: v.astype(np.float32) for k, v in t.items()}
    m = oracle.Model(hidden_size=H, num_layers=L, num_attention_heads=Hq, num_kv_heads=Hkv,
                     head_dim=hd, vocab_size=V, ffn_dim=F, max_position_embeddings=64,
                     has_qkv_bias=True, num_blocks=8, block_size=B).load(t)
    toks = rng.integers(0, V, 7)
    got = m.forward(oracle.Batch(toks, np.arange(7), [7], [7], [[5, 2]]))[0]

    def norm(x, w):
        return x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * w

    def rope(x, pos):  # x [n, heads, hd]
        half = hd // 2
        inv = 1.0 / 10000.0 ** (2.0 * np.arange(half) / hd)
        ang = pos[:, None] * inv[None]
        c, s = np.cos(ang)[:, None], np.sin(ang)[:, None]
        x0, x1 = x[..., :half], x[..., half:]
        return np.concatenate([x0 * c - x1 * s, x0 * s + x1 * c], -1)

    h = t["model.embed_tokens.weight"][toks].astype(np.float64)
    pos = np.arange(7, dtype=np.float64)
    for i in range(L):
        p = f"model.layers.{i}"
        x = norm(h, t[f"{p}.input_layernorm.weight"])
        q = (x @ t[f"{p}.self_attn.q_proj.weight"].T + t[f"{p}.self_attn.q_proj.bias"]).reshape(7, Hq, hd)
        k = (x @ t[f"{p}.self_attn.k_proj.weight"].T + t[f"{p}.self_attn.k_proj.bias"]).reshape(7, Hkv, hd)
        v = (x @ t[f"{p}.self_attn.v_proj.weight"].T + t[f"{p}.self_attn.v_proj.bias"]).reshape(7, Hkv, hd)
        q, k = rope(q, pos), rope(k, pos)
        att = np.zeros((7, Hq, hd))
        for r in range(7):
            for qh in range(Hq):
                kh = qh // (Hq // Hkv)
                sc = (k[: r + 1, kh] @ q[r, qh]) / math.sqrt(hd)
                w = np.exp(sc - sc.max())
                att[r, qh] = (w / w.sum()) @ v[: r + 1, kh]
        h = h + att.reshape(7, -1) @ t[f"{p}.self_attn.o_proj.weight"].T
        x = norm(h, t[f"{p}.post_attention_layernorm.weight"])
        g = x @ t[f"{p}.mlp.gate_proj.weight"].T
        u = x @ t[f"{p}.mlp.up_proj.weight"].T
        h = h + ((g / (1 + np.exp(-g))) * u) @ t[f"{p}.mlp.down_proj.weight"].T
    exp = norm(h, t["model.norm.weight"])[-1] @ t["lm_head.weight"].T
    assert np.max(np.abs(got - exp)) < 2e-4 * max(1.0, np.max(np.abs(exp)))


def test_tp_single_rank_is_the_plain_forward(oracle):
    """world_size 1 is the degenerate case of the same path (orion-distributed lib.rs:95-102)."""
    from conftest import random_tensors, SMALL_META

    t = random_tensors(np.random.default_rng(11), SMALL_META)
    batch = oracle.Batch([3, 1, 4, 1, 5], [0, 1, 2, 0, 1], [3, 2], [3, 2], [[2], [5]])
    full = oracle.Model(**SMALL_META).load(t).forward(batch)
    one = oracle.Model(**SMALL_META).load(t).forward_tp(batch, 0, 1, lambda buf: None)
    assert np.array_equal(one, full)
    with pytest.raises(oracle.OracleArgError):  # more ranks than KV heads (lib.rs:193-200)
        oracle.Model(**SMALL_META).load(t).forward_tp(batch, 0, 4, lambda buf: None)
