"""One small interface over the two driver implementations, so that every reference test restated in
``test_driver.py`` runs unchanged against the Python oracle (``oracle/driver.py``) and against the
C++ driver behind the C ABI (``orionserve_rs_b200.engine``)."""
from __future__ import annotations

import __graft_entry__ as ge
from oracle import driver as od


class DriverErr(Exception):
    def __init__(self, kind: str):
        super().__init__(kind)
        self.kind = kind


def _native_kind(pkg, e: Exception) -> str:
    from_cls = {pkg.errors.CacheExhausted: "CacheExhausted", pkg.errors.QueueFull: "QueueFull",
                pkg.errors.ContextLengthExceeded: "ContextLengthExceeded", pkg.errors.InternalError: "Internal",
                pkg.errors.InvalidRequest: "InvalidRequest"}
    for cls, kind in from_cls.items():
        if isinstance(e, cls):
            return kind
    raise e


class _Wrap:
    """Turns either implementation's exceptions into DriverErr(kind)."""

    def _call(self, fn, *a):
        try:
            return fn(*a)
        except od.OracleError as e:
            raise DriverErr(e.kind) from None
        except Exception as e:  # noqa: BLE001 - native errors are mapped, anything else re-raised
            if self.native:
                raise DriverErr(_native_kind(self.pkg, e)) from None
            raise


class Manager(_Wrap):
    def __init__(self, impl: str, num_blocks: int, block_size: int, prefix: bool, *, _inner=None):
        self.native = impl == "native"
        self.pkg = ge.load_package() if self.native else None
        if _inner is not None:
            self.m = _inner
        elif self.native:
            self.m = self.pkg.engine.KvCacheManager(num_blocks, block_size, prefix)
        else:
            self.m = od.KvCacheManager(num_blocks, block_size, prefix)

    def allocate(self, seq, prompt):
        out = self._call(self.m.allocate, seq, list(prompt))
        return (out.allocated, out.reused, out.cached_tokens) if self.native else out

    def append_token(self, seq):
        self._call(self.m.append_token, seq)

    def commit_prefill(self, seq, prompt):
        self.m.commit_prefill(seq, list(prompt))

    def free(self, seq):
        self.m.free(seq)

    def preempt(self, seq):
        return self.m.preempt(seq)

    def free_blocks(self):
        return self.m.free_blocks()

    def table(self, seq):
        if self.native:
            return self.m.block_table(seq)
        t = self.m.tables.get(seq)
        return None if t is None else (list(t.blocks), t.num_tokens)

    def is_allocated(self, seq):
        return self.table(seq) is not None

    def entries(self):
        return self.m.stats()["prefix_cache_entries"] if self.native else len(self.m.prefix.entries)

    def hits(self):
        return self.m.stats()["prefix_cache_hits"] if self.native else self.m.prefix.hits

    def misses(self):
        return self.m.stats()["prefix_cache_misses"] if self.native else self.m.prefix.misses

    def num_sequences(self):
        return self.m.num_sequences() if self.native else len(self.m.tables)

    def used_blocks(self):
        return self.m.stats()["used_blocks"] if self.native else self.m.total_blocks() - self.m.free_blocks()

    def num_evictable(self):
        return self.m.num_evictable() if self.native else self.m.pool.num_evictable()

    def evict_cached(self, n):
        return self.m.evict_cached(n)

    def clear_prefix_cache(self):
        self.m.clear_prefix_cache()

    def can_allocate(self, n):
        return self.m.can_allocate(n)

    def blocks_needed_for(self, n):
        return self.m.blocks_needed_for(n)

    def block_info(self, b):
        if self.native:
            return self.m.block_info(b)
        return self.m.pool.ref[b], self.m.pool.ntok[b], self.m.pool.hash[b]

    def fail_next_append(self):
        self.m.fail_next_append()


_REASON = {1: "stop", 2: "length", 3: "cancelled", 4: "timeout", 5: "error"}


class Sched(_Wrap):
    def __init__(self, impl: str, blocks: int, block_size: int = 4, prefix: bool = False, *, _inner=None, **cfg):
        self.native = impl == "native"
        self.pkg = ge.load_package() if self.native else None
        cfg.setdefault("request_timeout_secs", None)
        if _inner is not None:
            self.s = _inner
        elif self.native:
            self.s = self.pkg.engine.Scheduler(self.pkg.engine.SchedulerConfig(**cfg), blocks, block_size, prefix)
        else:
            cfg.pop("request_timeout_secs")
            self.s = od.Scheduler(od.Config(**cfg), od.KvCacheManager(blocks, block_size, prefix))
        self.cache = Manager(impl, 0, 1, False, _inner=self.s.cache() if self.native else self.s.cache)

    def add(self, prompt, max_tokens=16, min_tokens=0, stop_token_ids=()):
        prompt = [1] * prompt if isinstance(prompt, int) else list(prompt)
        if self.native:
            p = self.pkg.engine.SamplingParams(max_tokens=max_tokens, min_tokens=min_tokens,
                                               stop_token_ids=list(stop_token_ids))
            return self._call(self.s.add_request, prompt, p)
        p = od.Params(max_tokens=max_tokens, min_tokens=min_tokens, stop_token_ids=list(stop_token_ids))
        # the sequence takes its id on construction, admitted or not, like Sequence::new
        return self._call(self.s.add_request, od.Sequence(prompt, p))

    def schedule(self):
        if self.native:
            out = self.s.schedule()
            return [(x.id, x.num_tokens, x.start_position, x.is_prefill) for x in out.scheduled], list(out.preempted)
        sched, pre = self.s.schedule()
        return [(x.id, x.num_tokens, x.start_position, x.is_prefill) for x in sched], list(pre)

    def on_token(self, sid, token, eos=()):
        r = self.s.on_token(sid, token, list(eos))
        if self.native:
            return None if r is None else _REASON[int(r)]
        return r

    def reap(self):
        return self.s.reap_finished() if self.native else [s.id for s in self.s.reap_finished()]

    def cancel(self, sid):
        return self.s.cancel(sid)

    def commit_prefill(self, sid):
        self.s.commit_prefill(sid)

    def num_running(self):
        return self.s.num_running() if self.native else len(self.s.running)

    def num_waiting(self):
        return self.s.num_waiting() if self.native else len(self.s.waiting)

    def has_work(self):
        return self.s.has_work()

    def stats(self):
        return self.s.stats() if self.native else dict(self.s.stats)

    def running_ids(self):
        if self.native:
            raise NotImplementedError
        return [s.id for s in self.s.running]


class Eng(_Wrap):
    def __init__(self, impl: str, forward, blocks=64, block_size=4, prefix=True, eos=(), **cfg):
        self.native = impl == "native"
        self.pkg = ge.load_package() if self.native else None
        cfg.setdefault("request_timeout_secs", None)
        if self.native:
            E = self.pkg.engine
            self.e = E.Engine(forward, E.SchedulerConfig(**cfg), blocks, block_size, prefix, list(eos))
            self.sched = Sched(impl, 0, _inner=self.e.scheduler())
        else:
            cfg.pop("request_timeout_secs")
            s = od.Scheduler(od.Config(**cfg), od.KvCacheManager(blocks, block_size, prefix))
            self.e = od.Engine(s, forward, list(eos))
            self.sched = Sched(impl, 0, _inner=s)

    def submit(self, prompt, max_tokens, temperature=0.0, min_tokens=0, stop_token_ids=()):
        if self.native:
            p = self.pkg.engine.SamplingParams(temperature=temperature, max_tokens=max_tokens, min_tokens=min_tokens,
                                               stop_token_ids=list(stop_token_ids))
        else:
            p = od.Params(temperature=temperature, max_tokens=max_tokens, min_tokens=min_tokens,
                          stop_token_ids=list(stop_token_ids))
        return self._call(self.e.submit, list(prompt), p)

    def step(self):
        return self.e.step()

    def has_work(self):
        return self.e.has_work()

    def cancel(self, sid):
        self.e.cancel(sid)

    def events(self):
        if self.native:
            out = []
            for ev in self.e.take_events():
                if ev.kind == "token":
                    out.append(("token", ev.id, ev.token, ev.index))
                else:
                    out.append(("done", ev.id, _REASON[int(ev.reason)], ev.prompt_tokens, ev.completion_tokens))
            return out
        out, self.e.events = self.e.events, []
        return out

    def num_active(self):
        return self.e.num_active() if self.native else len(self.e.active)

    def batch(self):
        b = self.e.last_batch() if self.native else self.e.batch
        return dict(tokens=list(b.tokens), positions=list(b.positions), sequence_ids=list(b.sequence_ids),
                    slot_token_counts=list(b.slot_token_counts), context_lens=list(b.context_lens),
                    block_tables=[list(t) for t in b.block_tables], has_prefill=bool(b.has_prefill))
