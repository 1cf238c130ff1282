"""Boundary types of the forward path (crates/orion-core/src/traits.rs)."""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from .errors import InternalError


class DType(enum.IntEnum):
    """traits.rs:21-57."""
    F32 = 0
    F16 = 1
    BF16 = 2
    I8 = 3
    I4 = 4

    def bits(self) -> int:
        return {DType.F32: 32, DType.F16: 16, DType.BF16: 16, DType.I8: 8, DType.I4: 4}[self]

    def size_in_bytes(self, n: int) -> int:
        return (n * self.bits() + 7) // 8

    def as_str(self) -> str:
        return self.name.lower()


@dataclass(frozen=True)
class Device:
    """traits.rs:60-87: ``Device::Cpu`` or ``Device::Cuda(ordinal)``."""
    kind: str
    ordinal: int = 0

    def is_cpu(self) -> bool:
        return self.kind == "cpu"

    def as_str(self) -> str:
        return self.kind

    def __str__(self) -> str:
        return "cpu" if self.is_cpu() else f"cuda:{self.ordinal}"


@dataclass
class ModelMetadata:
    """traits.rs:95-150 plus the two values the reference keeps beside it:
    ``HfConfig::ffn_dim`` (config.rs:238) and ``Architecture::has_qkv_bias`` (config.rs:134)."""
    architecture: str
    name: str
    hidden_size: int
    num_layers: int
    num_attention_heads: int
    num_kv_heads: int
    head_dim: int
    vocab_size: int
    max_position_embeddings: int = 2048
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-5
    dtype: DType = DType.F32
    eos_token_ids: List[int] = field(default_factory=list)
    bos_token_id: Optional[int] = None
    ffn_dim: int = 0
    has_qkv_bias: bool = False
    tied_lm_head: bool = False

    def kv_bytes_per_token(self) -> int:
        return self.dtype.size_in_bytes(2 * self.num_layers * self.num_kv_heads * self.head_dim)

    def uses_gqa(self) -> bool:
        return self.num_kv_heads < self.num_attention_heads

    def gqa_group_size(self) -> int:
        return self.num_attention_heads // self.num_kv_heads if self.num_kv_heads else 0


@dataclass
class ForwardBatch:
    """traits.rs:193-262: the ragged batch of one forward pass."""
    tokens: Sequence[int]
    positions: Sequence[int]
    sequence_ids: Sequence[int]
    slot_token_counts: Sequence[int]
    context_lens: Sequence[int]
    block_tables: Sequence[Sequence[int]]
    has_prefill: bool = True

    def num_sequences(self) -> int:
        return len(self.sequence_ids)

    def num_tokens(self) -> int:
        return len(self.tokens)

    def is_empty(self) -> bool:
        return len(self.tokens) == 0

    def validate(self) -> None:
        """traits.rs:232-261 (the library applies the same checks again)."""
        n = len(self.sequence_ids)
        if len(self.slot_token_counts) != n or len(self.context_lens) != n or len(self.block_tables) != n:
            raise InternalError(
                f"ForwardBatch arrays disagree: {n} sequence ids, {len(self.slot_token_counts)} token "
                f"counts, {len(self.context_lens)} context lens, {len(self.block_tables)} block tables")
        if len(self.positions) != len(self.tokens):
            raise InternalError(
                f"ForwardBatch has {len(self.tokens)} tokens but {len(self.positions)} positions")
        summed = int(sum(int(c) for c in self.slot_token_counts))
        if summed != len(self.tokens):
            raise InternalError(
                f"ForwardBatch slot token counts sum to {summed} but there are {len(self.tokens)} tokens")

    def flatten(self):
        """The flat arrays that cross the C ABI."""
        tokens = np.ascontiguousarray(self.tokens, dtype=np.uint32)
        positions = np.ascontiguousarray(self.positions, dtype=np.uint32)
        counts = np.ascontiguousarray(self.slot_token_counts, dtype=np.uint64)
        ctx = np.ascontiguousarray(self.context_lens, dtype=np.uint64)
        tables = self.block_tables
        if isinstance(tables, np.ndarray) and tables.ndim == 2:  # equal-length tables kept as one array
            offsets = np.arange(tables.shape[0] + 1, dtype=np.uint64) * np.uint64(tables.shape[1])
            flat = np.append(np.ascontiguousarray(tables, dtype=np.uint32).ravel(), np.uint32(0))
            return tokens, positions, counts, ctx, flat, offsets
        lens = np.fromiter((len(t) for t in tables), dtype=np.uint64, count=len(tables))
        offsets = np.zeros(len(tables) + 1, np.uint64)
        np.cumsum(lens, out=offsets[1:])
        if len(tables):
            flat = np.concatenate([np.asarray(t, dtype=np.uint32).ravel() for t in tables]
                                  + [np.zeros(1, np.uint32)])
        else:
            flat = np.zeros(1, np.uint32)
        return tokens, positions, counts, ctx, np.ascontiguousarray(flat), offsets


@dataclass
class ForwardOutput:
    """traits.rs:271-290: row-major ``[num_sequences, vocab_size]`` last-position logits."""
    logits: np.ndarray
    vocab_size: int
    sequence_ids: Sequence[int]

    def row(self, i: int) -> Optional[np.ndarray]:
        if i < 0 or i >= len(self.sequence_ids):
            return None
        return self.logits.reshape(-1)[i * self.vocab_size:(i + 1) * self.vocab_size]

    def num_sequences(self) -> int:
        return len(self.sequence_ids)
