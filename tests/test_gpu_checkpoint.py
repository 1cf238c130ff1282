"""Checkpoint directory -> device model through the library's own safetensors reader
(``orion_cuda_model_load_checkpoint``): same logits as the tensor-by-tensor path, the reference's
rules for several shard files, and its error wording (crates/orion-models/src/loader.rs:112-235,
transformer.rs:62-120,180-205)."""
import json
import os
import struct

import numpy as np
import pytest

from drivers import C1_META, c1_tensors

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def backend(pkg):
    return pkg.CudaBackend(0)


def _config(meta, **over):
    cfg = dict(architectures=["LlamaForCausalLM"], hidden_size=meta["hidden_size"], num_hidden_layers=meta["num_layers"],
               num_attention_heads=meta["num_attention_heads"], num_key_value_heads=meta["num_kv_heads"],
               head_dim=meta["head_dim"], vocab_size=meta["vocab_size"], intermediate_size=meta["ffn_dim"],
               max_position_embeddings=meta["max_position_embeddings"], rope_theta=meta["rope_theta"],
               rms_norm_eps=meta["rms_norm_eps"], tie_word_embeddings=False)
    cfg.update(over)
    return cfg


def _batch(pkg):
    toks = list(range(5, 45))
    return pkg.ForwardBatch(toks, list(range(40)), [1], [40], [40], [[3, 9, 1]], has_prefill=True)


def test_directory_load_matches_tensor_by_tensor_load(pkg, backend, tmp_path):
    weights = c1_tensors(seed=99)
    names = sorted(weights)
    half = len(names) // 2
    d = tmp_path / "ckpt"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(_config(C1_META)))
    # two shard files of different dtypes; the second repeats one tensor of the first with other
    # values (the first file wins) and carries a buffer the model never asks for
    first = {n: weights[n] for n in names[:half]}
    second = {n: weights[n] for n in names[half:]}
    second[names[0]] = weights[names[0]] + 1.0
    second["model.layers.0.self_attn.rotary_emb.inv_freq"] = np.ones(32, np.float32)
    pkg.write_safetensors(str(d / "model-00001-of-00002.safetensors"), first, pkg.DType.F32)
    pkg.write_safetensors(str(d / "model-00002-of-00002.safetensors"), second, pkg.DType.F32)
    m = pkg.CudaTransformerModel.from_directory(str(d), 16, 16, backend, compute_dtype=pkg.DType.F32,
                                                max_batch_tokens=64, max_batch_sequences=2)
    meta = pkg.ModelMetadata(architecture="llama", name="c1", **C1_META)
    ref = pkg.CudaTransformerModel.new(meta, weights, 16, 16, backend, compute_dtype=pkg.DType.F32,
                                       max_batch_tokens=64, max_batch_sequences=2)
    assert np.array_equal(m.forward(_batch(pkg)).logits, ref.forward(_batch(pkg)).logits)

    # bf16 storage on disk, bf16 build: the same tensors after the same rounding
    db = tmp_path / "ckpt_bf16"
    db.mkdir()
    (db / "config.json").write_text(json.dumps(_config(C1_META)))
    pkg.write_safetensors(str(db / "model.safetensors"), weights, pkg.DType.BF16)
    mb = pkg.CudaTransformerModel.from_directory(str(db), 16, 16, backend, compute_dtype=pkg.DType.BF16,
                                                 max_batch_tokens=64, max_batch_sequences=2)
    rb = pkg.CudaTransformerModel.new(meta, weights, 16, 16, backend, compute_dtype=pkg.DType.BF16,
                                      max_batch_tokens=64, max_batch_sequences=2)
    assert np.array_equal(mb.forward(_batch(pkg)).logits, rb.forward(_batch(pkg)).logits)
    assert mb.load_checkpoint(str(db)) == len(weights), "every tensor of the layout is used, nothing else"


def test_checkpoint_errors_use_the_reference_wording(pkg, backend, tmp_path):
    weights = c1_tensors(seed=3)
    meta = pkg.ModelMetadata(architecture="llama", name="c1", **C1_META)

    def fresh():
        return pkg.CudaTransformerModel(meta, 16, 16, backend, compute_dtype=pkg.DType.F32, max_batch_tokens=64,
                                        max_batch_sequences=2)

    with pytest.raises(pkg.ModelError, match="path not found"):
        fresh().load_checkpoint(str(tmp_path / "nowhere"))
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(pkg.ModelError, match=r"missing file: .*\*\.safetensors"):
        fresh().load_checkpoint(str(empty))
    # a tensor is absent: reported by name (transformer.rs:73-118)
    part = tmp_path / "part"
    part.mkdir()
    some = dict(weights)
    del some["model.layers.1.mlp.down_proj.weight"]
    pkg.write_safetensors(str(part / "model.safetensors"), some)
    with pytest.raises(pkg.ModelError, match=r"missing tensor `model\.layers\.1\.mlp\.down_proj\.weight`"):
        fresh().load_checkpoint(str(part))
    # an unsupported dtype names the tensor (loader.rs:89-93)
    bad = tmp_path / "bad"
    bad.mkdir()
    header = json.dumps({"model.norm.weight": {"dtype": "I64", "shape": [256], "data_offsets": [0, 2048]}}).encode()
    (bad / "model.safetensors").write_bytes(struct.pack("<Q", len(header)) + header + bytes(2048))
    with pytest.raises(pkg.ModelError, match=r"unsupported dtype I64 \(tensor `model\.norm\.weight`\)"):
        fresh().load_checkpoint(str(bad))
    # truncated and garbled files are malformed, not a crash
    for name, blob in (("short", b"\x01\x02"), ("liar", struct.pack("<Q", 1 << 40) + b"{}"),
                       ("garbled", struct.pack("<Q", 9) + b"not json!")):
        dd = tmp_path / name
        dd.mkdir()
        (dd / "model.safetensors").write_bytes(blob)
        with pytest.raises(pkg.ModelError, match="malformed"):
            fresh().load_checkpoint(str(dd))
    # a wrong shape is refused by the tensor loader with both shapes in the message
    shp = tmp_path / "shape"
    shp.mkdir()
    wrong = dict(weights)
    wrong["model.norm.weight"] = np.ones(255, np.float32)
    pkg.write_safetensors(str(shp / "model.safetensors"), wrong)
    with pytest.raises(pkg.ModelError, match="model.norm.weight"):
        fresh().load_checkpoint(str(shp))
    assert os.path.isdir(str(shp))
