"""Tensor-parallel calculus and collectives (crates/orion-distributed/src/lib.rs)."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

import numpy as np

from . import _ffi
from .errors import InternalError, InvalidRequest, check
from .types import ModelMetadata


class ShardStrategy(enum.Enum):
    """lib.rs:58-71."""
    ColumnParallel = "column"
    RowParallel = "row"
    Replicated = "replicated"


@dataclass(frozen=True)
class Rank:
    """lib.rs:74-113."""
    index: int
    world_size: int

    def __post_init__(self):
        if self.world_size == 0:
            raise InvalidRequest("world_size must be at least 1")
        if self.index >= self.world_size or self.index < 0:
            raise InvalidRequest(f"rank {self.index} is out of range for world size {self.world_size}")

    @staticmethod
    def single() -> "Rank":
        return Rank(0, 1)

    def is_distributed(self) -> bool:
        return self.world_size > 1

    def is_leader(self) -> bool:
        return self.index == 0


@dataclass(frozen=True)
class Shard:
    """lib.rs:116-130."""
    start: int
    len: int

    def end(self) -> int:
        return self.start + self.len

    def is_empty(self) -> bool:
        return self.len == 0


def shard_dimension(total: int, rank: Rank) -> Shard:
    """lib.rs:139-152: exact divisibility or an error."""
    if total % rank.world_size != 0:
        raise InvalidRequest(
            f"cannot split {total} evenly across {rank.world_size} ranks; tensor parallelism requires "
            "the dimension to be divisible by the world size")
    n = total // rank.world_size
    return Shard(rank.index * n, n)


@dataclass(frozen=True)
class ParallelLayout:
    """lib.rs:156-224."""
    rank: Rank
    query_heads: Shard
    kv_heads: Shard
    ffn: Shard

    @staticmethod
    def compute(meta: ModelMetadata, rank: Rank, ffn_dim: int) -> "ParallelLayout":
        if not rank.is_distributed():
            return ParallelLayout(rank, Shard(0, meta.num_attention_heads), Shard(0, meta.num_kv_heads),
                                  Shard(0, ffn_dim))
        if meta.num_kv_heads < rank.world_size:
            raise InvalidRequest(
                f"model has {meta.num_kv_heads} KV heads but world size is {rank.world_size}; tensor "
                "parallelism beyond the KV head count would require replicating them, which is not "
                "implemented")
        return ParallelLayout(rank, shard_dimension(meta.num_attention_heads, rank),
                              shard_dimension(meta.num_kv_heads, rank), shard_dimension(ffn_dim, rank))

    @staticmethod
    def compute_native(meta: ModelMetadata, rank: Rank, ffn_dim: int) -> "ParallelLayout":
        """The same arithmetic through the C ABI (the copy the device model uses)."""
        q, kv, f = (C.c_uint64 * 2)(), (C.c_uint64 * 2)(), (C.c_uint64 * 2)()
        check(_ffi.lib().orion_cuda_tp_layout(meta.num_attention_heads, meta.num_kv_heads, ffn_dim,
                                              rank.index, rank.world_size, q, kv, f))
        return ParallelLayout(rank, Shard(q[0], q[1]), Shard(kv[0], kv[1]), Shard(f[0], f[1]))

    def local_attention_dim(self, head_dim: int) -> int:
        return self.query_heads.len * head_dim

    def local_kv_bytes_per_token(self, meta: ModelMetadata) -> int:
        return meta.dtype.size_in_bytes(2 * meta.num_layers * self.kv_heads.len * meta.head_dim)


class Collective:
    """lib.rs:231-254: the collectives a tensor-parallel forward needs, over f32 buffers."""

    def rank(self) -> Rank:
        raise NotImplementedError

    def all_reduce_sum(self, buffer: np.ndarray) -> None:
        raise NotImplementedError

    def all_gather(self, local: np.ndarray, out: np.ndarray) -> None:
        raise NotImplementedError

    def reduce_scatter_sum(self, inp: np.ndarray, out: np.ndarray) -> None:
        raise NotImplementedError

    def barrier(self) -> None:
        raise NotImplementedError


class SingleRank(Collective):
    """lib.rs:263-302: the correct implementation for world_size == 1."""

    def rank(self) -> Rank:
        return Rank.single()

    def all_reduce_sum(self, buffer: np.ndarray) -> None:
        return None

    def all_gather(self, local: np.ndarray, out: np.ndarray) -> None:
        if local.size != out.size:
            raise InternalError(f"all_gather on a single rank expects equal sizes, got {local.size} and {out.size}")
        out[...] = local

    def reduce_scatter_sum(self, inp: np.ndarray, out: np.ndarray) -> None:
        if inp.size != out.size:
            raise InternalError(f"reduce_scatter on a single rank expects equal sizes, got {inp.size} and {out.size}")
        out[...] = inp

    def barrier(self) -> None:
        return None


class TorchCollective(Collective):
    """Host-side N-rank collective over a ``torch.distributed`` process group (gloo on CPU).
    Used by the multi-rank host tests; the device path uses NCCL inside the library."""

    def __init__(self, group=None):
        import torch.distributed as dist

        self._dist, self._group = dist, group
        self._rank = Rank(dist.get_rank(group), dist.get_world_size(group))

    def rank(self) -> Rank:
        return self._rank

    def all_reduce_sum(self, buffer: np.ndarray) -> None:
        import torch

        t = torch.from_numpy(buffer)
        self._dist.all_reduce(t, group=self._group)

    def all_gather(self, local: np.ndarray, out: np.ndarray) -> None:
        import torch

        if out.size != local.size * self._rank.world_size:
            raise InternalError("all_gather output must hold world_size slices")
        parts = [torch.empty(local.size, dtype=torch.float32) for _ in range(self._rank.world_size)]
        self._dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(local, np.float32)).reshape(-1),
                              group=self._group)
        out.reshape(-1)[...] = torch.cat(parts).numpy()

    def reduce_scatter_sum(self, inp: np.ndarray, out: np.ndarray) -> None:
        import torch

        if inp.size != out.size * self._rank.world_size:
            raise InternalError("reduce_scatter input must hold world_size slices")
        t = torch.from_numpy(np.ascontiguousarray(inp, np.float32).copy()).reshape(-1)
        self._dist.all_reduce(t, group=self._group)
        n = out.size
        out.reshape(-1)[...] = t.numpy()[self._rank.index * n:(self._rank.index + 1) * n]

    def barrier(self) -> None:
        self._dist.barrier(group=self._group)


class NcclCollective(Collective):
    """The Collective trait over NCCL and NVLink (``orion_cuda_collective_*``): one handle per rank,
    on the backend's device; host f32 arrays in and out like the trait's slices."""

    def __init__(self, backend, unique_id: bytes, rank: Rank):
        self._rank = rank
        self._h = C.c_void_p()
        idbuf = (C.c_uint8 * _ffi.NCCL_ID_BYTES)(*(unique_id or bytes(_ffi.NCCL_ID_BYTES)))
        check(_ffi.lib().orion_cuda_collective_create(backend._h, idbuf, rank.index, rank.world_size,
                                                      C.byref(self._h)))

    def __del__(self):
        if getattr(self, "_h", None):
            _ffi.lib().orion_cuda_collective_destroy(self._h)
            self._h = None

    def rank(self) -> Rank:
        return self._rank

    @staticmethod
    def _f32(a: np.ndarray, writable: bool) -> np.ndarray:
        if a.dtype != np.float32 or not a.flags.c_contiguous or (writable and not a.flags.writeable):
            raise InternalError("collective buffers are contiguous f32 arrays")
        return a

    def all_reduce_sum(self, buffer: np.ndarray) -> None:
        b = self._f32(buffer, True)
        check(_ffi.lib().orion_cuda_collective_all_reduce_sum(self._h, b.ctypes.data_as(C.POINTER(C.c_float)), b.size))

    def all_gather(self, local: np.ndarray, out: np.ndarray) -> None:
        if out.size != local.size * self._rank.world_size:
            raise InternalError("all_gather output must hold world_size slices")
        a, o = self._f32(local, False), self._f32(out, True)
        F = C.POINTER(C.c_float)
        check(_ffi.lib().orion_cuda_collective_all_gather(self._h, a.ctypes.data_as(F), a.size, o.ctypes.data_as(F)))

    def reduce_scatter_sum(self, inp: np.ndarray, out: np.ndarray) -> None:
        if inp.size != out.size * self._rank.world_size:
            raise InternalError("reduce_scatter input must hold world_size slices")
        a, o = self._f32(inp, False), self._f32(out, True)
        F = C.POINTER(C.c_float)
        check(_ffi.lib().orion_cuda_collective_reduce_scatter_sum(self._h, a.ctypes.data_as(F), o.size, o.ctypes.data_as(F)))

    def barrier(self) -> None:
        check(_ffi.lib().orion_cuda_collective_barrier(self._h))


class NcclCollectiveId:
    """The 128-byte ``ncclUniqueId`` rank 0 creates and every rank passes to its model."""

    @staticmethod
    def create() -> bytes:
        buf = (C.c_uint8 * _ffi.NCCL_ID_BYTES)()
        check(_ffi.lib().orion_cuda_tp_unique_id(buf))
        return bytes(buf)


@dataclass(frozen=True)
class CommunicationEstimate:
    """lib.rs:311-336: two all-reduces per layer, ring factor 2(N-1)/N."""
    all_reduce_count: int
    bytes_per_token: int

    @staticmethod
    def for_model(meta: ModelMetadata, world_size: int) -> "CommunicationEstimate":
        if world_size <= 1:
            return CommunicationEstimate(0, 0)
        count = meta.num_layers * 2
        buffer = meta.dtype.size_in_bytes(meta.hidden_size)
        factor = 2.0 * (world_size - 1) / world_size
        return CommunicationEstimate(count, int(count * buffer * factor))
