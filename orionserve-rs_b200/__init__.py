"""Host-side mirror of the reference interface for the forward path, over the C ABI.

Names, argument meaning and error behaviour follow the reference:
``Backend`` / ``LanguageModel`` / ``ForwardBatch`` / ``ForwardOutput`` / ``ModelMetadata``
(crates/orion-core/src/traits.rs), ``CudaBackend`` / ``Tolerance`` / ``validate``
(crates/orion-cuda/src/lib.rs), ``TransformerModel::{new, from_directory}``
(crates/orion-models/src/transformer.rs:148-205), ``Rank`` / ``ParallelLayout`` / ``Collective``
(crates/orion-distributed/src/lib.rs), and for the driver side ``KvCacheManager`` / ``Scheduler`` /
``Engine`` (crates/orion-kv-cache, crates/orion-scheduler, crates/orion-runtime/src/engine.rs).
All arithmetic and all bookkeeping run in ``liborion_cuda.so``.
"""
from .errors import (BackendError, CacheExhausted, ContextLengthExceeded, CudaUnavailable, EngineError,
                     InternalError, InvalidRequest, ModelError, QueueFull)
from .types import DType, Device, ForwardBatch, ForwardOutput, ModelMetadata
from .backend import CudaBackend, device_count, is_available
from .model import CudaTransformerModel, HfConfig, read_safetensors, write_safetensors
from .validate import Tolerance, ValidationReport, validate
from .distributed import (Collective, CommunicationEstimate, NcclCollective, NcclCollectiveId, ParallelLayout, Rank,
                          Shard, ShardStrategy, SingleRank, shard_dimension)
from . import engine, errors, ops
from .engine import Engine, KvCacheManager, SamplingParams, Scheduler, SchedulerConfig, hash_block
from .attn_bench import PagedAttentionBench

__all__ = [
    "BackendError", "CudaUnavailable", "EngineError", "InternalError", "InvalidRequest", "ModelError",
    "DType", "Device", "ForwardBatch", "ForwardOutput", "ModelMetadata", "CudaBackend",
    "device_count", "is_available", "CudaTransformerModel", "HfConfig", "read_safetensors",
    "write_safetensors", "Tolerance", "ValidationReport", "validate", "Collective",
    "CommunicationEstimate", "NcclCollective", "NcclCollectiveId", "ParallelLayout", "Rank", "Shard", "ShardStrategy",
    "SingleRank", "shard_dimension", "ops", "PagedAttentionBench", "CacheExhausted", "ContextLengthExceeded",
    "QueueFull", "engine", "errors", "Engine", "KvCacheManager", "SamplingParams", "Scheduler", "SchedulerConfig",
    "hash_block",
]
