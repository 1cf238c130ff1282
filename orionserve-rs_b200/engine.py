"""Host-side driver over the C ABI of ``include/orion_driver.h``: the KV-cache manager, the
continuous-batching scheduler and the engine step, with the reference's names and semantics
(crates/orion-kv-cache/src/manager.rs, crates/orion-scheduler/src/scheduler.rs,
crates/orion-runtime/src/engine.rs). All bookkeeping runs in ``liborion_cuda.so``; this file only
marshals arguments."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import numpy as np

from . import _ffi
from .errors import EngineError, check


class FinishReason(enum.IntEnum):
    """``FinishReason`` (crates/orion-core/src/sequence.rs:73-87)."""
    STOP = 1
    LENGTH = 2
    CANCELLED = 3
    TIMEOUT = 4
    ERROR = 5


class SequenceState(enum.IntEnum):
    """``SequenceState`` (sequence.rs:26-37)."""
    WAITING = 0
    PREFILLING = 1
    DECODING = 2
    FINISHED = 3


@dataclass
class SamplingParams:
    """``SamplingParams`` (crates/orion-core/src/sampling.rs:25-70): the fields the driver reads."""
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = 0
    repetition_penalty: float = 1.0
    max_tokens: int = 16
    min_tokens: int = 0
    stop_token_ids: List[int] = field(default_factory=list)

    def _c(self):
        stops = (C.c_uint32 * max(1, len(self.stop_token_ids)))(*self.stop_token_ids)
        p = _ffi.OrionSamplingParams(self.temperature, self.top_p, self.repetition_penalty, self.top_k,
                                     self.max_tokens, self.min_tokens, stops, len(self.stop_token_ids))
        return p, stops


@dataclass
class SchedulerConfig:
    """``SchedulerConfig`` with the reference's defaults (crates/orion-core/src/config.rs:143-155)."""
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: Optional[int] = None
    enable_chunked_prefill: bool = True
    max_waiting_requests: int = 1024
    request_timeout_secs: Optional[int] = 300
    prioritize_decode: bool = True
    #: not in the reference: start a new sequence's prefill after the tokens whose blocks came from
    #: the prefix cache (the reference shares those blocks but recomputes them)
    skip_cached_prefix: bool = False
    #: not in the reference: decode tokens at position total_len - 1 (their logical place) instead of
    #: total_len, so no cache slot is skipped and no step is refused
    logical_decode_positions: bool = False

    def _c(self):
        return _ffi.OrionSchedulerConfig(self.max_num_seqs, self.max_num_batched_tokens, self.max_model_len or 0,
                                         int(self.enable_chunked_prefill), self.max_waiting_requests,
                                         self.request_timeout_secs or 0, int(self.prioritize_decode),
                                         int(self.skip_cached_prefix), int(self.logical_decode_positions))


@dataclass(frozen=True)
class AllocationOutcome:
    allocated: int
    reused: int
    cached_tokens: int

    def had_cache_hit(self) -> bool:
        return self.reused > 0


@dataclass(frozen=True)
class ScheduledSequence:
    id: int
    num_tokens: int
    start_position: int
    is_prefill: bool


@dataclass
class SchedulerOutput:
    scheduled: List[ScheduledSequence]
    preempted: List[int]

    def is_empty(self) -> bool:
        return not self.scheduled

    def num_batched_tokens(self) -> int:
        return sum(s.num_tokens for s in self.scheduled)

    def num_sequences(self) -> int:
        return len(self.scheduled)

    def num_prefill_sequences(self) -> int:
        return sum(1 for s in self.scheduled if s.is_prefill)

    def num_decode_sequences(self) -> int:
        return sum(1 for s in self.scheduled if not s.is_prefill)

    def is_mixed(self) -> bool:
        return self.num_prefill_sequences() > 0 and self.num_decode_sequences() > 0


@dataclass(frozen=True)
class StreamEvent:
    """``StreamEvent`` (crates/orion-runtime/src/engine.rs:60-90): ``kind`` is "token" or "done"."""
    id: int
    kind: str
    token: int = 0
    index: int = 0
    reason: Optional[FinishReason] = None
    prompt_tokens: int = 0
    completion_tokens: int = 0


def _u32(values) -> "C.Array":
    arr = np.ascontiguousarray(values, dtype=np.uint32)
    return arr, arr.ctypes.data_as(C.POINTER(C.c_uint32))


def hash_block(parent: Optional[int], tokens: Sequence[int]) -> int:
    """``hash_block`` (crates/orion-kv-cache/src/table.rs:105-120)."""
    keep, ptr = _u32(tokens)
    return int(_ffi.lib().orion_hash_block(parent is not None, parent or 0, ptr, len(keep)))


def next_sequence_id() -> int:
    """The id the next submitted sequence will get (crates/orion-core/src/id.rs:52-55)."""
    return int(_ffi.lib().orion_sequence_id_peek())


class KvCacheManager:
    """``KvCacheManager`` (crates/orion-kv-cache/src/manager.rs:73-425)."""

    def __init__(self, num_blocks: int, block_size: int, prefix_caching_enabled: bool, *, _borrowed=None, _keep=None):
        # A borrowed view keeps its owner alive (`_keep`); owners never point back at their views,
        # so there is no reference cycle and handles are destroyed in dependency order.
        self._keep = _keep
        self._owned = _borrowed is None
        self._h = _borrowed or _ffi.lib().orion_kv_manager_create(num_blocks, block_size, int(prefix_caching_enabled))
        if not self._h:
            raise EngineError(_ffi.last_error())

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "_h", None):
            _ffi.lib().orion_kv_manager_destroy(self._h)
            self._h = None

    def allocate(self, seq: int, prompt: Sequence[int]) -> AllocationOutcome:
        keep, ptr = _u32(prompt)
        out = _ffi.OrionAllocationOutcome()
        check(_ffi.lib().orion_kv_manager_allocate(self._h, seq, ptr, len(keep), C.byref(out)))
        return AllocationOutcome(out.allocated, out.reused, out.cached_tokens)

    def commit_prefill(self, seq: int, prompt: Sequence[int]) -> None:
        keep, ptr = _u32(prompt)
        _ffi.lib().orion_kv_manager_commit_prefill(self._h, seq, ptr, len(keep))

    def append_token(self, seq: int) -> None:
        check(_ffi.lib().orion_kv_manager_append_token(self._h, seq))

    def free(self, seq: int) -> None:
        _ffi.lib().orion_kv_manager_free(self._h, seq)

    def preempt(self, seq: int) -> int:
        return int(_ffi.lib().orion_kv_manager_preempt(self._h, seq))

    def stats(self) -> dict:
        s = _ffi.OrionCacheStats()
        check(_ffi.lib().orion_kv_manager_stats(self._h, C.byref(s)))
        return {n: int(getattr(s, n)) for n, _ in s._fields_}

    def free_blocks(self) -> int:
        return self.stats()["free_blocks"]

    def total_blocks(self) -> int:
        return self.stats()["total_blocks"]

    def num_sequences(self) -> int:
        return self.stats()["num_sequences"]

    def can_allocate(self, num_tokens: int) -> bool:
        return bool(_ffi.lib().orion_kv_manager_can_allocate(self._h, num_tokens))

    def blocks_needed_for(self, num_tokens: int) -> int:
        return int(_ffi.lib().orion_kv_manager_blocks_needed_for(self._h, num_tokens))

    def evict_cached(self, count: int) -> int:
        return int(_ffi.lib().orion_kv_manager_evict_cached(self._h, count))

    def clear_prefix_cache(self) -> None:
        _ffi.lib().orion_kv_manager_clear_prefix_cache(self._h)

    def num_evictable(self) -> int:
        return int(_ffi.lib().orion_kv_manager_num_evictable(self._h))

    def is_allocated(self, seq: int) -> bool:
        return self.block_table(seq) is not None

    def block_table(self, seq: int):
        """``(blocks, num_tokens)`` of a sequence, or None (``raw_block_table``, manager.rs:379-381)."""
        nb, nt = C.c_uint64(), C.c_uint64()
        if not _ffi.lib().orion_kv_manager_block_table(self._h, seq, None, 0, C.byref(nb), C.byref(nt)):
            return None
        blocks = np.zeros(max(1, nb.value), np.uint32)
        _ffi.lib().orion_kv_manager_block_table(self._h, seq, blocks.ctypes.data_as(C.POINTER(C.c_uint32)), nb.value,
                                                C.byref(nb), C.byref(nt))
        return blocks[:nb.value].tolist(), int(nt.value)

    def block_info(self, block: int):
        """``(ref_count, num_tokens, hash or None)`` of a physical block, or None for an unknown id."""
        rc, nt, hh, h = C.c_uint32(), C.c_uint64(), C.c_int(), C.c_uint64()
        if not _ffi.lib().orion_kv_manager_block_info(self._h, block, C.byref(rc), C.byref(nt), C.byref(hh), C.byref(h)):
            return None
        return int(rc.value), int(nt.value), (int(h.value) if hh.value else None)

    def fail_next_append(self) -> None:
        _ffi.lib().orion_kv_manager_fail_next(self._h, 0)

    def fail_next_allocate(self) -> None:
        _ffi.lib().orion_kv_manager_fail_next(self._h, 1)


class Scheduler:
    """``Scheduler`` over its own ``KvCacheManager`` (crates/orion-scheduler/src/scheduler.rs:127-580)."""

    def __init__(self, config: SchedulerConfig, num_blocks: int, block_size: int, prefix_caching_enabled: bool = False,
                 *, _borrowed=None, _keep=None):
        self._owned = _borrowed is None
        self._keep = _keep
        if _borrowed is None:
            cfg = config._c()
            self._h = _ffi.lib().orion_scheduler_create(C.byref(cfg), num_blocks, block_size, int(prefix_caching_enabled))
        else:
            self._h = _borrowed
        if not self._h:
            raise EngineError(_ffi.last_error())

    def __del__(self):
        if getattr(self, "_owned", False) and getattr(self, "_h", None):
            _ffi.lib().orion_scheduler_destroy(self._h)
            self._h = None

    def cache(self) -> KvCacheManager:
        return KvCacheManager(0, 1, False, _borrowed=_ffi.lib().orion_scheduler_cache(self._h), _keep=self)

    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        keep, ptr = _u32(prompt)
        p, stops = (params or SamplingParams())._c()
        sid = C.c_uint64()
        check(_ffi.lib().orion_scheduler_add_request(self._h, ptr, len(keep), C.byref(p), C.byref(sid)))
        return int(sid.value)

    def cancel(self, seq: int) -> bool:
        return bool(_ffi.lib().orion_scheduler_cancel(self._h, seq))

    def schedule(self) -> SchedulerOutput:
        cap = 4096
        while True:
            sched = (_ffi.OrionScheduledSequence * cap)()
            pre = (C.c_uint64 * cap)()
            ns, npre = C.c_uint64(), C.c_uint64()
            check(_ffi.lib().orion_scheduler_schedule(self._h, sched, cap, C.byref(ns), pre, cap, C.byref(npre)))
            assert ns.value <= cap and npre.value <= cap, "scheduler output larger than the marshalling buffer"
            return SchedulerOutput([ScheduledSequence(int(x.id), int(x.num_tokens), int(x.start_position), bool(x.is_prefill))
                                    for x in sched[:ns.value]], [int(x) for x in pre[:npre.value]])

    def on_token(self, seq: int, token: int, eos_ids: Sequence[int] = ()) -> Optional[FinishReason]:
        keep, ptr = _u32(list(eos_ids))
        r = _ffi.lib().orion_scheduler_on_token(self._h, seq, token, ptr, len(keep))
        return FinishReason(r) if r else None

    def reap_finished(self) -> List[int]:
        ids = (C.c_uint64 * 4096)()
        n = _ffi.lib().orion_scheduler_reap_finished(self._h, ids, 4096)
        return [int(x) for x in ids[:min(n, 4096)]]

    def commit_prefill(self, seq: int) -> None:
        _ffi.lib().orion_scheduler_commit_prefill(self._h, seq)

    def num_waiting(self) -> int:
        return int(_ffi.lib().orion_scheduler_num_waiting(self._h))

    def num_running(self) -> int:
        return int(_ffi.lib().orion_scheduler_num_running(self._h))

    def has_work(self) -> bool:
        return self.num_waiting() > 0 or self.num_running() > 0

    def stats(self) -> dict:
        s = _ffi.OrionSchedulerStats()
        check(_ffi.lib().orion_scheduler_stats(self._h, C.byref(s)))
        return {n: int(getattr(s, n)) for n, _ in s._fields_}

    def running_sequence(self, seq: int):
        """``(state, computed_prefix_len, output_len)`` of a running sequence, or None."""
        st, cp, ol = C.c_int(), C.c_uint64(), C.c_uint64()
        if not _ffi.lib().orion_scheduler_running_sequence(self._h, seq, C.byref(st), C.byref(cp), C.byref(ol)):
            return None
        return SequenceState(st.value), int(cp.value), int(ol.value)


@dataclass
class HostBatch:
    """The batch one engine step built (``build_batch``, engine.rs:429-487)."""
    tokens: List[int]
    positions: List[int]
    sequence_ids: List[int]
    slot_token_counts: List[int]
    context_lens: List[int]
    block_tables: List[List[int]]
    has_prefill: bool


ForwardCallable = Callable[[HostBatch], Sequence[int]]


class Engine:
    """``Engine`` (crates/orion-runtime/src/engine.rs:186-487). ``model`` is a device model
    (greedy argmax on the GPU every step) or a Python callable ``HostBatch -> token ids`` (one per
    sequence) standing in for it; a callable may raise ``EngineError`` to fail the step."""

    def __init__(self, model, config: SchedulerConfig, num_blocks: int, block_size: int,
                 prefix_caching_enabled: bool = True, eos_ids: Sequence[int] = ()):
        self._model = model
        self._error: Optional[BaseException] = None
        cfg = config._c()
        keep, eos = _u32(list(eos_ids))
        if callable(model) and not hasattr(model, "_h"):
            self._cb = _ffi.FORWARD_FN(self._trampoline)
            handle = None
        else:
            self._cb = _ffi.FORWARD_FN()  # NULL: the library calls the device model itself
            handle = model._h
        self._h = _ffi.lib().orion_engine_create(handle, self._cb, None, C.byref(cfg), num_blocks, block_size,
                                                 int(prefix_caching_enabled), eos, len(keep))
        if not self._h:
            raise EngineError(_ffi.last_error())
        self._config = config

    def __del__(self):
        if getattr(self, "_h", None):
            _ffi.lib().orion_engine_destroy(self._h)
            self._h = None

    def _trampoline(self, _user, tokens, T, positions, seq_ids, counts, ctx, tables, offsets, S, has_prefill, out):
        try:
            offs = [int(offsets[i]) for i in range(S + 1)]
            batch = HostBatch([int(tokens[i]) for i in range(T)], [int(positions[i]) for i in range(T)],
                              [int(seq_ids[i]) for i in range(S)], [int(counts[i]) for i in range(S)],
                              [int(ctx[i]) for i in range(S)],
                              [[int(tables[j]) for j in range(offs[i], offs[i + 1])] for i in range(S)], bool(has_prefill))
            ids = self._model(batch)
            for i in range(S):
                out[i] = int(ids[i])
            return _ffi.ORION_OK
        except BaseException as e:  # never unwind through the C frames
            self._error = e
            return _ffi.ERR_INTERNAL

    def scheduler(self) -> Scheduler:
        return Scheduler(self._config, 0, 1, _borrowed=_ffi.lib().orion_engine_scheduler(self._h), _keep=self)

    def submit(self, prompt: Sequence[int], params: SamplingParams) -> int:
        keep, ptr = _u32(prompt)
        p, stops = params._c()
        sid = C.c_uint64()
        check(_ffi.lib().orion_engine_submit(self._h, ptr, len(keep), C.byref(p), C.byref(sid)))
        return int(sid.value)

    def cancel(self, seq: int) -> None:
        _ffi.lib().orion_engine_cancel(self._h, seq)

    def has_work(self) -> bool:
        return bool(_ffi.lib().orion_engine_has_work(self._h))

    def step(self) -> int:
        """One engine step; returns the number of sequences that ran. Raises the forward's error
        with scheduler and cache already advanced, like the reference (engine.rs:309-310)."""
        ran = C.c_uint64()
        self._error = None
        rc = _ffi.lib().orion_engine_step(self._h, C.byref(ran))
        if rc != _ffi.ORION_OK and self._error is not None:
            err, self._error = self._error, None
            raise err
        check(rc)
        return int(ran.value)

    def take_events(self) -> List[StreamEvent]:
        out: List[StreamEvent] = []
        buf = (_ffi.OrionEngineEvent * 1024)()
        while True:
            n = _ffi.lib().orion_engine_take_events(self._h, buf, 1024)
            for e in buf[:n]:
                if e.kind == 0:
                    out.append(StreamEvent(int(e.id), "token", token=int(e.token), index=int(e.index)))
                else:
                    out.append(StreamEvent(int(e.id), "done", reason=FinishReason(e.reason),
                                           prompt_tokens=int(e.prompt_tokens), completion_tokens=int(e.completion_tokens)))
            if n < 1024:
                return out

    def num_active(self) -> int:
        return int(_ffi.lib().orion_engine_num_active(self._h))

    def last_batch(self) -> HostBatch:
        u32p, u64p = C.POINTER(C.c_uint32), C.POINTER(C.c_uint64)
        tok, pos, tab = u32p(), u32p(), u32p()
        ids, cnt, ctx, off = u64p(), u64p(), u64p(), u64p()
        T, S, hp = C.c_uint64(), C.c_uint64(), C.c_int()
        check(_ffi.lib().orion_engine_last_batch(self._h, C.byref(tok), C.byref(T), C.byref(pos), C.byref(ids),
                                                 C.byref(cnt), C.byref(ctx), C.byref(tab), C.byref(off), C.byref(S),
                                                 C.byref(hp)))
        T, S = T.value, S.value
        offs = [int(off[i]) for i in range(S + 1)] if S else [0]
        return HostBatch([int(tok[i]) for i in range(T)], [int(pos[i]) for i in range(T)],
                         [int(ids[i]) for i in range(S)], [int(cnt[i]) for i in range(S)],
                         [int(ctx[i]) for i in range(S)],
                         [[int(tab[j]) for j in range(offs[i], offs[i + 1])] for i in range(S)], bool(hp.value))
