"""``CudaTransformerModel: LanguageModel`` — the drop-in for ``TransformerModel``
(crates/orion-models/src/transformer.rs:137-443) — plus the checkpoint plumbing the
constructor convention needs (``HfConfig`` config.rs:20-246, safetensors loader.rs:100-235)."""
from __future__ import annotations

import ctypes as C
import json
import os
import struct
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import numpy as np

from . import _ffi
from .backend import CudaBackend
from .errors import ModelError, check
from .types import DType, ForwardBatch, ForwardOutput, ModelMetadata

_ST_DTYPES = {"F32": (DType.F32, np.float32), "F16": (DType.F16, np.uint16),
              "BF16": (DType.BF16, np.uint16)}


def read_safetensors(path: str) -> Dict[str, Tuple[DType, Tuple[int, ...], np.ndarray]]:
    """Minimal safetensors reader: 8-byte LE header length, JSON header, raw LE data.
    Returns name -> (dtype, shape, flat array view); 16-bit floats come back as uint16 bits."""
    data = np.memmap(path, dtype=np.uint8, mode="r")
    if data.size < 8:
        raise ModelError(f"{path} is malformed: shorter than its header length")
    (hlen,) = struct.unpack("<Q", bytes(data[:8]))
    if 8 + hlen > data.size:
        raise ModelError(f"{path} is malformed: header length {hlen} exceeds the file")
    try:
        header = json.loads(bytes(data[8:8 + hlen]).decode("utf-8"))
    except ValueError as e:
        raise ModelError(f"{path} is malformed: {e}") from e
    out = {}
    base = 8 + hlen
    for name, info in header.items():
        if name == "__metadata__":
            continue
        if info["dtype"] not in _ST_DTYPES:
            raise ModelError(f"unsupported dtype {info['dtype']} (tensor `{name}`)")  # loader.rs:89-93
        dt, npdt = _ST_DTYPES[info["dtype"]]
        b, e = info["data_offsets"]
        arr = np.frombuffer(data, dtype=npdt, count=(e - b) // np.dtype(npdt).itemsize, offset=base + b)
        out[name] = (dt, tuple(info["shape"]), arr)
    return out


def write_safetensors(path: str, tensors: Dict[str, np.ndarray], dtype: DType = DType.F32) -> None:
    """Writes f32 arrays as F32 or (rounded to nearest even) BF16."""
    header, blobs, off = {}, [], 0
    for name, a in tensors.items():
        a = np.ascontiguousarray(a, dtype=np.float32)
        if dtype == DType.BF16:
            bits = a.view(np.uint32)
            rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
            blob, tag = rounded.tobytes(), "BF16"
        else:
            blob, tag = a.tobytes(), "F32"
        header[name] = {"dtype": tag, "shape": list(a.shape), "data_offsets": [off, off + len(blob)]}
        blobs.append(blob)
        off += len(blob)
    h = json.dumps(header).encode()
    h += b" " * ((8 - len(h) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(h)))
        f.write(h)
        for b in blobs:
            f.write(b)


@dataclass
class HfConfig:
    """config.rs:20-71 with its serde aliases and defaults."""
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    vocab_size: int
    architectures: List[str] = field(default_factory=list)
    model_type: Optional[str] = None
    num_key_value_heads: Optional[int] = None
    head_dim: Optional[int] = None
    intermediate_size: Optional[int] = None
    max_position_embeddings: Optional[int] = None
    rope_theta: Optional[float] = None
    rms_norm_eps: Optional[float] = None
    torch_dtype: Optional[str] = None
    eos_token_id: object = None
    bos_token_id: Optional[int] = None
    tie_word_embeddings: Optional[bool] = None

    _ALIASES = {"n_layer": "num_hidden_layers", "num_layers": "num_hidden_layers",
                "n_head": "num_attention_heads", "n_positions": "max_position_embeddings",
                "max_sequence_length": "max_position_embeddings", "layer_norm_eps": "rms_norm_eps",
                "rms_norm_epsilon": "rms_norm_eps"}

    @classmethod
    def from_dict(cls, d: dict) -> "HfConfig":
        known = {f for f in cls.__dataclass_fields__}
        kw = {}
        for k, v in d.items():
            k = cls._ALIASES.get(k, k)
            if k in known:  # unknown fields are ignored (config.rs:16-18)
                kw[k] = v
        try:
            return cls(**kw)
        except TypeError as e:
            raise ModelError(f"config.json is malformed: {e}") from e

    @classmethod
    def load(cls, directory: str) -> "HfConfig":
        path = os.path.join(directory, "config.json")
        try:
            with open(path) as f:
                return cls.from_dict(json.load(f))
        except OSError as e:
            raise ModelError(f"{path}: {e}") from e
        except ValueError as e:
            raise ModelError(f"config.json is malformed: {e}") from e

    def architecture(self) -> str:
        """Architecture::detect (config.rs:106-131)."""
        for a in self.architectures:
            if a in ("LlamaForCausalLM", "MistralForCausalLM"):
                return "llama"
            if a == "Qwen2ForCausalLM":
                return "qwen2"
        if self.model_type in ("llama", "mistral"):
            return "llama"
        if self.model_type == "qwen2":
            return "qwen2"
        raise ModelError(f"unsupported architecture {self.architectures or self.model_type}")

    def ffn_dim(self) -> int:
        return self.intermediate_size if self.intermediate_size is not None else 4 * self.hidden_size

    def ties_embeddings(self) -> bool:
        return bool(self.tie_word_embeddings)

    def to_metadata(self, name: str) -> ModelMetadata:
        """config.rs:179-233."""
        arch = self.architecture()
        kv = self.num_key_value_heads if self.num_key_value_heads is not None else self.num_attention_heads
        hd = self.head_dim if self.head_dim is not None else self.hidden_size // max(self.num_attention_heads, 1)
        if self.num_attention_heads == 0 or self.num_hidden_layers == 0:
            raise ModelError("config.json is malformed: num_attention_heads and num_hidden_layers must be non-zero")
        if kv == 0:
            raise ModelError("config.json is malformed: num_key_value_heads must be non-zero")
        if self.num_attention_heads % kv != 0:
            raise ModelError(f"config.json is malformed: num_attention_heads ({self.num_attention_heads}) "
                             f"must be a multiple of num_key_value_heads ({kv})")
        if hd == 0:
            raise ModelError("config.json is malformed: head_dim resolved to zero")
        if self.vocab_size == 0:
            raise ModelError("config.json is malformed: vocab_size must be non-zero")
        dt = {None: DType.F32, "float32": DType.F32, "float16": DType.F16, "bfloat16": DType.BF16}.get(self.torch_dtype)
        if dt is None:
            raise ModelError(f"unsupported dtype {self.torch_dtype}")
        eos = self.eos_token_id
        eos_ids = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        return ModelMetadata(
            architecture=arch, name=name, hidden_size=self.hidden_size, num_layers=self.num_hidden_layers,
            num_attention_heads=self.num_attention_heads, num_kv_heads=kv, head_dim=hd,
            vocab_size=self.vocab_size,
            max_position_embeddings=self.max_position_embeddings if self.max_position_embeddings is not None else 2048,
            rope_theta=self.rope_theta if self.rope_theta is not None else 10000.0,
            rms_norm_eps=self.rms_norm_eps if self.rms_norm_eps is not None else 1e-5,
            dtype=dt, eos_token_ids=eos_ids, bos_token_id=self.bos_token_id, ffn_dim=self.ffn_dim(),
            has_qkv_bias=(arch == "qwen2"), tied_lm_head=self.ties_embeddings())


class CudaTransformerModel:
    """A GPU-executing decoder-only transformer with the reference's constructor convention."""

    def __init__(self, meta: ModelMetadata, num_blocks: int, block_size: int, backend: CudaBackend, *,
                 compute_dtype: DType = DType.BF16, max_batch_tokens: int = 8192,
                 max_batch_sequences: int = 256, tp_rank: int = 0, tp_world: int = 1,
                 nccl_unique_id: Optional[bytes] = None):
        """``TransformerModel::new`` minus the weights, which arrive through ``load_tensor`` /
        ``load_state`` (transformer.rs:148-177)."""
        self._meta, self._backend, self._h = meta, backend, C.c_void_p()
        d = _ffi.OrionModelDesc(
            meta.hidden_size, meta.num_layers, meta.num_attention_heads, meta.num_kv_heads, meta.head_dim,
            meta.vocab_size, meta.ffn_dim or 4 * meta.hidden_size, meta.max_position_embeddings,
            meta.rope_theta, meta.rms_norm_eps, int(meta.has_qkv_bias), int(meta.tied_lm_head),
            num_blocks, block_size, int(compute_dtype), max_batch_tokens, max_batch_sequences, tp_rank,
            tp_world)
        if nccl_unique_id is not None:
            C.memmove(d.nccl_unique_id, nccl_unique_id, _ffi.NCCL_ID_BYTES)
        self.compute_dtype, self.num_blocks, self.block_size = compute_dtype, num_blocks, block_size
        self.tp_rank, self.tp_world = tp_rank, tp_world
        check(_ffi.lib().orion_cuda_model_create(backend._h, C.byref(d), C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            _ffi.lib().orion_cuda_model_destroy(self._h)
            self._h = None

    # ---- construction -------------------------------------------------------
    @classmethod
    def new(cls, meta: ModelMetadata, weights: Dict[str, np.ndarray], num_blocks: int, block_size: int,
            backend: CudaBackend, **kw) -> "CudaTransformerModel":
        m = cls(meta, num_blocks, block_size, backend, **kw)
        m.load_state(weights)
        return m

    @classmethod
    def from_directory(cls, directory: str, num_blocks: int, block_size: int, backend: CudaBackend,
                       **kw) -> "CudaTransformerModel":
        """transformer.rs:180-205: config.json + one or more safetensors shards."""
        cfg = HfConfig.load(directory)
        meta = cfg.to_metadata(os.path.basename(os.path.normpath(directory)) or "model")
        if cfg.ties_embeddings():  # transformer.rs:108-112; an absent lm_head falls back to the embedding too
            meta.tied_lm_head = True
        m = cls(meta, num_blocks, block_size, backend, **kw)
        m.load_checkpoint(directory)
        return m

    def load_checkpoint(self, directory: str) -> int:
        """Every ``*.safetensors`` file of ``directory`` straight from its memory mapping to the
        device (this rank's slices only), then ``finalize``; returns the number of tensors used.
        The files are opened and parsed inside the library (``CheckpointLoader``, loader.rs:112-235)."""
        n = C.c_uint64()
        check(_ffi.lib().orion_cuda_model_load_checkpoint(self._h, os.fsencode(directory), C.byref(n)))
        return int(n.value)

    def load_tensor(self, name: str, data: np.ndarray, shape=None, dtype: Optional[DType] = None) -> None:
        if dtype is None:
            data = np.ascontiguousarray(data, dtype=np.float32)
            dtype = DType.F32
        else:
            data = np.ascontiguousarray(data)
        shape = tuple(shape if shape is not None else data.shape)
        shp = (C.c_uint64 * max(len(shape), 1))(*shape)
        check(_ffi.lib().orion_cuda_model_load_tensor(self._h, name.encode(), int(dtype), shp, len(shape),
                                                     data.ctypes.data_as(C.c_void_p)))

    def load_state(self, weights: Dict[str, np.ndarray]) -> None:
        for name, w in weights.items():
            self.load_tensor(name, w)
        self.finalize()

    def finalize(self) -> None:
        check(_ffi.lib().orion_cuda_model_finalize(self._h))

    def init_random(self, seed: int, std: float = 0.02) -> None:
        check(_ffi.lib().orion_cuda_model_init_random(self._h, seed, std))

    # ---- LanguageModel ------------------------------------------------------
    def metadata(self) -> ModelMetadata:
        return self._meta

    def backend(self) -> CudaBackend:
        return self._backend

    def _batch_args(self, batch: ForwardBatch):
        tokens, positions, counts, ctx, flat, offs = batch.flatten()
        keep = (tokens, positions, counts, ctx, flat, offs)
        P = lambda a, t: a.ctypes.data_as(C.POINTER(t))
        args = [P(tokens, C.c_uint32), tokens.size, P(positions, C.c_uint32), positions.size,
                P(counts, C.c_uint64), counts.size, P(ctx, C.c_uint64), ctx.size, P(flat, C.c_uint32),
                P(offs, C.c_uint64), len(batch.block_tables), len(batch.sequence_ids), int(batch.has_prefill)]
        return args, keep

    def forward(self, batch: ForwardBatch, out: Optional[np.ndarray] = None) -> ForwardOutput:
        """``LanguageModel::forward`` (traits.rs:305). ``out`` may be a preallocated (for instance
        page-locked) float32 buffer of at least ``num_sequences * vocab_size`` elements."""
        args, keep = self._batch_args(batch)
        n = len(batch.sequence_ids) * self._meta.vocab_size
        if out is None:
            out = np.empty(max(n, 1), np.float32)
        check(_ffi.lib().orion_cuda_model_forward(self._h, *args, out.ctypes.data_as(C.c_void_p), out.size))
        rows = 0 if batch.is_empty() else len(batch.sequence_ids)
        logits = out.reshape(-1)[:rows * self._meta.vocab_size].reshape(rows, self._meta.vocab_size)
        return ForwardOutput(logits, self._meta.vocab_size, list(batch.sequence_ids) if rows else [])

    def forward_greedy(self, batch: ForwardBatch, want_logits: bool = False):
        """forward + device-side greedy argmax; returns (token ids, logits or None)."""
        args, keep = self._batch_args(batch)
        S = len(batch.sequence_ids)
        ids = np.zeros(max(S, 1), np.uint32)
        logits = np.empty(max(S * self._meta.vocab_size, 1), np.float32) if want_logits else None
        check(_ffi.lib().orion_cuda_model_forward_greedy(
            self._h, *args, ids.ctypes.data_as(C.POINTER(C.c_uint32)),
            logits.ctypes.data_as(C.c_void_p) if want_logits else None,
            logits.size if want_logits else 0))
        return ids[:S], (logits[:S * self._meta.vocab_size].reshape(S, -1) if want_logits else None)

    def replay(self, iterations: int) -> float:
        """Re-runs the previous batch on the device ``iterations`` times; returns elapsed ms."""
        ms = C.c_float()
        check(_ffi.lib().orion_cuda_model_replay(self._h, iterations, C.byref(ms)))
        return ms.value

    CATEGORIES = ("gemm", "attention", "elementwise", "collective")

    def replay_categories(self, iterations: int, *names: str) -> float:
        """Timing only: replays just the kernels of the named categories back to back, as they
        run inside a step; returns elapsed ms. Buffer contents are meaningless afterwards."""
        mask = 0
        for n in names:
            mask |= 1 << self.CATEGORIES.index(n)
        ms = C.c_float()
        check(_ffi.lib().orion_cuda_model_replay_categories(self._h, iterations, mask, C.byref(ms)))
        return ms.value

    def profile(self, iterations: int):
        """Per-category device time of the previous batch: dict name -> (ms, launches), summed
        over ``iterations`` replays."""
        ms, n = (C.c_float * 4)(), (C.c_uint64 * 4)()
        check(_ffi.lib().orion_cuda_model_profile(self._h, iterations, ms, n))
        names = ("gemm", "attention", "elementwise", "collective")
        return {k: (float(ms[i]), int(n[i])) for i, k in enumerate(names)}

    def fill_kv_random(self, seed: int, std: float = 1.0) -> None:
        check(_ffi.lib().orion_cuda_model_fill_kv_random(self._h, seed, std))

    def last_launch_count(self) -> int:
        v = C.c_uint64()
        check(_ffi.lib().orion_cuda_model_last_launch_count(self._h, C.byref(v)))
        return v.value

    def read_kv(self) -> np.ndarray:
        """This rank's arena as ``[layer][block][k|v][slot][local kv head][dim]`` f32."""
        m = self._meta
        lkv = m.num_kv_heads // self.tp_world
        shape = (m.num_layers, self.num_blocks, 2, self.block_size, lkv, m.head_dim)
        out = np.zeros(shape, np.float32)
        check(_ffi.lib().orion_cuda_model_read_kv(self._h, out.ctypes.data_as(C.POINTER(C.c_float)), out.size))
        return out


def pinned_empty(n: int) -> Tuple[np.ndarray, object]:
    """A page-locked float32 array of ``n`` elements and the owner that keeps it alive."""
    p = _ffi.lib().orion_cuda_host_alloc(max(n, 1) * 4)
    if not p:
        raise MemoryError("orion_cuda_host_alloc failed")

    class _Owner:
        def __init__(self, ptr):
            self.ptr = ptr

        def __del__(self):
            if self.ptr:
                _ffi.lib().orion_cuda_host_free(self.ptr)
                self.ptr = None

    owner = _Owner(p)
    arr = np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(max(n, 1),))
    return arr, owner
