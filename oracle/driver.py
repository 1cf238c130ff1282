"""TEST INFRASTRUCTURE ONLY: a plain-Python restatement of the reference's driver side (block pool,
prefix cache, KV-cache manager, sequences, scheduler, engine step), used by tests as the checker
of the C++ driver. Nothing in the product path may import it.

It is written independently of the C++ driver, straight from the reference sources named on each
class, with Python lists and dicts only. Pinned against the reference's own unit tests, restated
as pytest cases in ``tests/test_driver.py`` (the reference cannot be compiled here: no Rust
toolchain), and then used as the oracle of randomised differential tests.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence as Seq

MASK64 = (1 << 64) - 1


class OracleError(Exception):
    """An ``EngineError`` of the reference; ``kind`` is the variant name."""

    def __init__(self, kind: str, message: str = ""):
        super().__init__(f"{kind}: {message}")
        self.kind = kind


def _mix(state: int, value: int) -> int:  # table.rs:122-126
    rot = ((state << 5) | (state >> 59)) & MASK64
    return ((rot ^ value) * 0x517CC1B727220A95) & MASK64


def hash_block(parent: Optional[int], tokens: Seq[int]) -> int:  # table.rs:105-120
    state = 0xCBF29CE484222325 if parent is None else parent
    state = _mix(state, len(tokens))
    for t in tokens:
        state = _mix(state, t)
    return state


class IdCounter:
    """``SequenceId::next`` (crates/orion-core/src/id.rs:52-55); tests set ``next`` to follow the
    process-wide counter of the library under test."""
    next = 1

    @classmethod
    def take(cls) -> int:
        v = cls.next
        cls.next += 1
        return v


class BlockPool:  # block.rs:93-275
    def __init__(self, num_blocks: int, block_size: int):
        self.ref = [0] * num_blocks
        self.ntok = [0] * num_blocks
        self.hash: List[Optional[int]] = [None] * num_blocks
        self.free_list = deque(range(num_blocks))
        self.block_size = block_size

    def num_free(self) -> int:
        return len(self.free_list)

    def allocate(self):  # block.rs:153-166
        if not self.free_list:
            raise OracleError("CacheExhausted", "needed 1, available 0")
        b = self.free_list.popleft()
        evicted = self.hash[b]
        self.ref[b], self.ntok[b], self.hash[b] = 1, 0, None
        return b, evicted

    def add_ref(self, b: int) -> None:  # block.rs:172-185
        if self.ref[b] == 0 and b in self.free_list:
            self.free_list.remove(b)
        self.ref[b] += 1

    def release(self, b: int) -> bool:  # block.rs:191-208
        if self.ref[b] == 0:
            raise OracleError("Internal", f"double release of blk-{b}")
        self.ref[b] -= 1
        if self.ref[b] == 0:
            self.free_list.append(b)
            return True
        return False

    def set_contents(self, b: int, n: int, h: Optional[int]) -> None:  # block.rs:211-230
        if n > self.block_size:
            raise OracleError("Internal", "block over capacity")
        self.ntok[b], self.hash[b] = n, h

    def evict_oldest_cached(self):  # block.rs:241-253
        for b in self.free_list:
            if self.hash[b] is not None:
                h = self.hash[b]
                self.hash[b], self.ntok[b] = None, 0
                return b, h
        return None

    def num_evictable(self) -> int:
        return sum(1 for b in self.free_list if self.hash[b] is not None)


class PrefixCache:  # prefix.rs:40-150
    def __init__(self):
        self.entries: Dict[int, tuple] = {}
        self.hits = self.misses = 0

    def lookup(self, h: int, tokens: Seq[int]) -> Optional[int]:
        e = self.entries.get(h)
        if e is not None and e[1] == list(tokens):
            self.hits += 1
            return e[0]
        self.misses += 1
        return None

    def insert(self, h: int, block: int, tokens: Seq[int]) -> None:
        self.entries.setdefault(h, (block, list(tokens)))

    def remove(self, h: int, block: int) -> None:
        e = self.entries.get(h)
        if e is not None and e[0] == block:
            del self.entries[h]


@dataclass
class Table:  # table.rs:13-22
    blocks: List[int] = field(default_factory=list)
    num_tokens: int = 0


def blocks_required(n: int, bs: int) -> int:
    return -(-n // bs)


class KvCacheManager:  # manager.rs:73-425
    def __init__(self, num_blocks: int, block_size: int, prefix_caching_enabled: bool):
        self.pool = BlockPool(num_blocks, block_size)
        self.tables: Dict[int, Table] = {}
        self.prefix = PrefixCache()
        self.enabled = prefix_caching_enabled
        self._fail_append = self._fail_allocate = False

    def free_blocks(self) -> int:
        return self.pool.num_free()

    def total_blocks(self) -> int:
        return len(self.pool.ref)

    def blocks_needed_for(self, n: int) -> int:
        return blocks_required(n, self.pool.block_size)

    def can_allocate(self, n: int) -> bool:
        return self.blocks_needed_for(n) <= self.pool.num_free()

    def allocate(self, seq: int, prompt: Seq[int]):  # manager.rs:163-250
        if self._fail_allocate:
            self._fail_allocate = False
            raise OracleError("CacheExhausted", "injected")
        if seq in self.tables:
            raise OracleError("Internal", f"seq-{seq} already has a block table")
        bs = self.pool.block_size
        needed = blocks_required(len(prompt), bs)
        if needed > self.pool.num_free():
            raise OracleError("CacheExhausted", f"needed {needed}, available {self.pool.num_free()}")
        table = Table()
        allocated = reused = cached = 0
        chain: Optional[int] = None
        matching = self.enabled
        for s in range(0, len(prompt), bs):
            chunk = list(prompt[s:s + bs])
            h = hash_block(chain, chunk) if (matching and len(chunk) == bs) else None
            blk = self.prefix.lookup(h, chunk) if h is not None else None
            if blk is not None:
                self.pool.add_ref(blk)
                table.blocks.append(blk)
                reused += 1
                cached += len(chunk)
                chain = h
            else:
                matching = False
                try:
                    blk, evicted = self.pool.allocate()
                except OracleError:
                    for b in table.blocks:
                        self.pool.release(b)
                    raise
                if evicted is not None:
                    self.prefix.remove(evicted, blk)
                table.blocks.append(blk)
                allocated += 1
                self.pool.set_contents(blk, len(chunk), None)
                chain = None
        table.num_tokens = len(prompt)
        self.tables[seq] = table
        return allocated, reused, cached

    def commit_prefill(self, seq: int, prompt: Seq[int]) -> None:  # manager.rs:258-283
        if not self.enabled or seq not in self.tables:
            return
        bs = self.pool.block_size
        table = self.tables[seq]
        chain: Optional[int] = None
        for i, s in enumerate(range(0, len(prompt), bs)):
            chunk = list(prompt[s:s + bs])
            if len(chunk) != bs or i >= len(table.blocks):
                break
            h = hash_block(chain, chunk)
            self.pool.set_contents(table.blocks[i], bs, h)
            self.prefix.insert(h, table.blocks[i], chunk)
            chain = h

    def append_token(self, seq: int) -> None:  # manager.rs:290-335
        if self._fail_append:
            self._fail_append = False
            raise OracleError("CacheExhausted", "injected")
        if seq not in self.tables:
            raise OracleError("Internal", f"seq-{seq} has no block table")
        bs = self.pool.block_size
        table = self.tables[seq]
        new_len = table.num_tokens + 1
        if blocks_required(new_len, bs) > len(table.blocks):
            blk, evicted = self.pool.allocate()
            if evicted is not None:
                self.prefix.remove(evicted, blk)
            table.blocks.append(blk)
        table.num_tokens = new_len
        if not table.blocks:
            raise OracleError("Internal", "empty block table")
        self.pool.set_contents(table.blocks[-1], new_len - (len(table.blocks) - 1) * bs, None)

    def free(self, seq: int) -> None:  # manager.rs:341-359
        table = self.tables.pop(seq, None)
        if table is not None:
            for b in table.blocks:
                self.pool.release(b)

    def preempt(self, seq: int) -> int:
        n = len(self.tables[seq].blocks) if seq in self.tables else 0
        self.free(seq)
        return n

    def evict_cached(self, count: int) -> int:  # manager.rs:397-409
        n = 0
        while n < count:
            hit = self.pool.evict_oldest_cached()
            if hit is None:
                break
            self.prefix.remove(hit[1], hit[0])
            n += 1
        return n

    def clear_prefix_cache(self) -> None:
        self.evict_cached(self.pool.num_evictable())
        self.prefix.entries.clear()

    def fail_next_append(self) -> None:
        self._fail_append = True

    def fail_next_allocate(self) -> None:
        self._fail_allocate = True


WAITING, PREFILLING, DECODING, FINISHED = "waiting", "prefilling", "decoding", "finished"
_LEGAL = {(WAITING, PREFILLING), (WAITING, FINISHED), (PREFILLING, PREFILLING), (PREFILLING, DECODING),
          (PREFILLING, WAITING), (PREFILLING, FINISHED), (DECODING, DECODING), (DECODING, WAITING),
          (DECODING, FINISHED)}  # sequence.rs:41-55


@dataclass
class Params:  # sampling.rs:25-70
    temperature: float = 1.0
    max_tokens: int = 16
    min_tokens: int = 0
    stop_token_ids: List[int] = field(default_factory=list)
    repetition_penalty: float = 1.0


class Sequence:  # sequence.rs:158-330
    def __init__(self, prompt: Seq[int], params: Params):
        self.id = IdCounter.take()
        self.prompt = list(prompt)
        self.output: List[int] = []
        self.computed = 0
        self.state = WAITING
        self.reason: Optional[str] = None
        self.params = params

    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    def prefill_complete(self) -> bool:
        return self.computed >= len(self.prompt)

    def transition(self, nxt: str) -> bool:
        if (self.state, nxt) not in _LEGAL:
            return False
        self.state = nxt
        return True

    def advance(self, n: int) -> None:
        self.computed = min(self.computed + n, len(self.prompt))

    def finish(self, reason: str) -> None:
        if self.state != FINISHED:
            self.state, self.reason = FINISHED, reason

    def preempt(self) -> bool:
        if (self.state, WAITING) not in _LEGAL:
            return False
        self.state, self.computed = WAITING, 0
        return True


@dataclass
class Config:  # config.rs:107-156
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: Optional[int] = None
    enable_chunked_prefill: bool = True
    max_waiting_requests: int = 1024
    prioritize_decode: bool = True
    skip_cached_prefix: bool = False  # not in the reference: prefill starts after the adopted cached tokens
    logical_decode_positions: bool = False  # not in the reference: decode at total_len - 1 instead of total_len


@dataclass(frozen=True)
class Scheduled:  # scheduler.rs:36-50
    id: int
    num_tokens: int
    start_position: int
    is_prefill: bool


class Scheduler:  # scheduler.rs:127-580
    def __init__(self, config: Config, cache: KvCacheManager):
        self.config, self.cache = config, cache
        self.waiting: deque = deque()
        self.running: List[Sequence] = []
        self.stats = dict(total_steps=0, total_admitted=0, total_finished=0, total_preempted=0, total_rejected=0,
                          total_batched_tokens=0, total_prefill_tokens=0, total_decode_tokens=0,
                          total_skipped_prefill_tokens=0)
        # only with skip_cached_prefix: sequences one of whose prefill chunks was in a step whose
        # forward failed (nothing written to the device cache although progress was recorded)
        self.unwritten_prefill: set = set()

    def has_work(self) -> bool:
        return bool(self.waiting) or bool(self.running)

    def add_request(self, seq: Sequence) -> int:  # scheduler.rs:174-214
        c = self.config
        if len(self.waiting) >= c.max_waiting_requests:
            self.stats["total_rejected"] += 1
            raise OracleError("QueueFull")
        max_len = c.max_model_len if c.max_model_len is not None else MASK64
        if len(seq.prompt) + seq.params.max_tokens > max_len:
            self.stats["total_rejected"] += 1
            raise OracleError("ContextLengthExceeded")
        if self.cache.blocks_needed_for(len(seq.prompt)) > self.cache.total_blocks():
            self.stats["total_rejected"] += 1
            raise OracleError("CacheExhausted")
        self.waiting.append(seq)
        self.stats["total_admitted"] += 1
        return seq.id

    def get(self, sid: int) -> Optional[Sequence]:
        return next((s for s in self.running if s.id == sid), None)

    def cancel(self, sid: int) -> bool:  # scheduler.rs:226-236
        for s in self.waiting:
            if s.id == sid:
                self.waiting.remove(s)
                return True
        s = self.get(sid)
        if s is not None:
            self.running.remove(s)
            self.cache.free(sid)
            self.unwritten_prefill.discard(sid)
            return True
        return False

    def schedule(self):  # scheduler.rs:239-263
        sched: List[Scheduled] = []
        preempted: List[int] = []
        used = [0]
        budget = self.config.max_num_batched_tokens
        order = (self._decodes, self._prefills) if self.config.prioritize_decode else (self._prefills, self._decodes)
        for phase in order:
            phase(sched, preempted, budget, used)
        self.stats["total_steps"] += 1
        self.stats["total_batched_tokens"] += sum(s.num_tokens for s in sched)
        for s in sched:
            self.stats["total_prefill_tokens" if s.is_prefill else "total_decode_tokens"] += s.num_tokens
        return sched, preempted

    def _try_append(self, sid: int) -> bool:
        try:
            self.cache.append_token(sid)
            return True
        except OracleError:
            return False

    def _decodes(self, sched, preempted, budget, used) -> None:  # scheduler.rs:267-313
        shift = 1 if self.config.logical_decode_positions else 0
        for sid, total in [(s.id, max(0, s.total_len() - shift)) for s in self.running if s.state == DECODING]:
            if used[0] >= budget:
                break
            if self._try_append(sid):
                sched.append(Scheduled(sid, 1, total, False))
                used[0] += 1
            else:
                if not self._preempt_one(preempted):
                    break
                if self._try_append(sid):
                    sched.append(Scheduled(sid, 1, total, False))
                    used[0] += 1

    def _preempt_one(self, preempted) -> bool:  # scheduler.rs:317-330
        if not self.running:
            return False
        victim = self.running.pop()
        self.cache.free(victim.id)
        victim.preempt()
        self.unwritten_prefill.discard(victim.id)
        self.waiting.appendleft(victim)
        preempted.append(victim.id)
        self.stats["total_preempted"] += 1
        return True

    def _chunk(self, remaining: int, room: int) -> Optional[int]:
        if self.config.enable_chunked_prefill:
            return min(remaining, room)
        return remaining if remaining <= room else None

    def _prefills(self, sched, preempted, budget, used) -> None:  # scheduler.rs:343-470
        for sid, already, remaining in [(s.id, s.computed, len(s.prompt) - s.computed) for s in self.running
                                        if s.state == PREFILLING and not s.prefill_complete()]:
            if used[0] >= budget:
                break
            chunk = self._chunk(remaining, budget - used[0])
            if not chunk:
                continue
            s = self.get(sid)
            if s is None:
                continue
            s.advance(chunk)
            if s.prefill_complete():
                s.transition(DECODING)
            sched.append(Scheduled(sid, chunk, already, True))
            used[0] += chunk
        while True:
            if len(self.running) >= self.config.max_num_seqs or used[0] >= budget or not self.waiting:
                break
            nxt = self.waiting[0]
            prompt_len, already = len(nxt.prompt), nxt.computed
            chunk = self._chunk(prompt_len - already, budget - used[0])
            if chunk is None or chunk == 0:
                break
            first = already == 0
            if first and not self.cache.can_allocate(prompt_len):
                if not self._preempt_one(preempted):
                    break
                continue
            seq = self.waiting.popleft()
            if first:
                try:
                    _, _, cached = self.cache.allocate(seq.id, seq.prompt)
                except OracleError:
                    seq.preempt()
                    self.waiting.appendleft(seq)
                    break
                if self.config.skip_cached_prefix and cached > 0:
                    skip = min(cached, prompt_len - 1)  # the last prompt token is always computed
                    seq.advance(skip)
                    self.stats["total_skipped_prefill_tokens"] += skip
                    already = skip
                    chunk = min(chunk, prompt_len - skip)
            seq.advance(chunk)
            if seq.state == WAITING:
                seq.transition(PREFILLING)
            if seq.prefill_complete():
                seq.transition(DECODING)
            sched.append(Scheduled(seq.id, chunk, already, True))
            used[0] += chunk
            self.running.append(seq)

    def on_token(self, sid: int, token: int, eos_ids: Seq[int]) -> Optional[str]:  # scheduler.rs:476-507
        s = self.get(sid)
        if s is None:
            return None
        s.output.append(token)
        reason = None
        if (token in eos_ids or token in s.params.stop_token_ids) and len(s.output) >= s.params.min_tokens:
            reason = "stop"
        elif len(s.output) >= s.params.max_tokens:
            reason = "length"
        if reason:
            s.finish(reason)
        return reason

    def reap_finished(self) -> List[Sequence]:  # scheduler.rs:513-520
        done = [s for s in self.running if s.state == FINISHED]
        self.running = [s for s in self.running if s.state != FINISHED]
        for s in done:
            self.cache.free(s.id)
            self.unwritten_prefill.discard(s.id)
        self.stats["total_finished"] += len(done)
        return done

    def commit_prefill(self, sid: int) -> None:  # scheduler.rs:557-564
        s = self.get(sid)
        if self.config.skip_cached_prefix and sid in self.unwritten_prefill:
            return
        if s is not None and s.prefill_complete():
            self.cache.commit_prefill(sid, s.prompt)

    def note_failed_step(self, sched) -> None:
        if self.config.skip_cached_prefix:
            self.unwritten_prefill.update(x.id for x in sched if x.is_prefill)


@dataclass
class Batch:  # traits.rs:193-210
    tokens: List[int] = field(default_factory=list)
    positions: List[int] = field(default_factory=list)
    sequence_ids: List[int] = field(default_factory=list)
    slot_token_counts: List[int] = field(default_factory=list)
    context_lens: List[int] = field(default_factory=list)
    block_tables: List[List[int]] = field(default_factory=list)
    has_prefill: bool = False


class Engine:  # engine.rs:186-487
    def __init__(self, scheduler: Scheduler, forward: Callable[[Batch], Seq[int]], eos_ids: Seq[int] = ()):
        self.scheduler, self.forward, self.eos = scheduler, forward, list(eos_ids)
        self.active: Dict[int, int] = {}
        self.events: List[tuple] = []
        self.batch = Batch()
        self.last = ([], [])

    def submit(self, prompt: Seq[int], params: Params) -> int:  # engine.rs:235-268
        if params.max_tokens == 0 or params.min_tokens > params.max_tokens or params.temperature < 0:
            raise OracleError("InvalidRequest")
        sid = self.scheduler.add_request(Sequence(prompt, params))
        self.active[sid] = len(prompt)
        return sid

    def has_work(self) -> bool:  # engine.rs:284-286
        return self.scheduler.has_work()

    def cancel(self, sid: int) -> None:  # engine.rs:271-281
        if self.scheduler.cancel(sid) and sid in self.active:
            self.events.append(("done", sid, "cancelled", self.active.pop(sid), 0))

    def step(self) -> int:  # engine.rs:293-342
        sched, preempted = self.scheduler.schedule()
        self.last = (sched, preempted)
        if not sched:
            self.batch = Batch()
            self._reap()
            return 0
        self.batch = self._build(sched)
        try:
            ids = self.forward(self.batch) if self.batch.sequence_ids else []
        except Exception:
            self.scheduler.note_failed_step(sched)
            raise
        for row, sid in enumerate(self.batch.sequence_ids):
            s = self.scheduler.get(sid)
            if s is not None and not s.prefill_complete():
                continue
            self._emit(sid, int(ids[row]))
        for x in sched:
            if x.is_prefill:
                self.scheduler.commit_prefill(x.id)
        self._reap()
        return len(self.batch.sequence_ids)

    def _emit(self, sid: int, token: int) -> None:  # engine.rs:345-386
        s = self.scheduler.get(sid)
        if s is None or sid not in self.active:
            return
        index = max(0, s.total_len() - self.active[sid])
        reason = self.scheduler.on_token(sid, token, self.eos)
        self.events.append(("token", sid, token, index))
        if reason:
            self._finish(sid, reason)

    def _finish(self, sid: int, reason: str) -> None:  # engine.rs:395-410
        s = self.scheduler.get(sid)
        if sid in self.active:
            self.events.append(("done", sid, reason, self.active.pop(sid), len(s.output) if s else 0))

    def _reap(self) -> None:  # engine.rs:414-426
        for s in self.scheduler.reap_finished():
            if s.id in self.active:
                self.events.append(("done", s.id, s.reason or "stop", self.active.pop(s.id), len(s.output)))

    def _build(self, sched) -> Batch:  # engine.rs:429-487
        b = Batch()
        for x in sched:
            s = self.scheduler.get(x.id)
            if s is None:
                continue
            table = self.scheduler.cache.tables.get(x.id)
            if table is None:
                raise OracleError("Internal", "scheduled without a block table")
            if x.is_prefill:
                toks = s.prompt[x.start_position:min(x.start_position + x.num_tokens, len(s.prompt))]
            elif s.output:
                toks = [s.output[-1]]
            else:
                toks = s.prompt[-1:]
            if not toks:
                continue
            b.positions += list(range(x.start_position, x.start_position + len(toks)))
            b.tokens += toks
            b.sequence_ids.append(x.id)
            b.slot_token_counts.append(len(toks))
            b.context_lens.append(x.start_position + len(toks))
            b.block_tables.append(list(table.blocks))
            b.has_prefill = b.has_prefill or x.is_prefill
        return b
