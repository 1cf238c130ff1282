"""The reference's own unit tests of the driver side, restated case for case and run against BOTH
the Python oracle and the C++ driver behind the C ABI (host only, no GPU):

  crates/orion-kv-cache/src/table.rs:128-228      hash_block properties
  crates/orion-kv-cache/src/block.rs:277-483      pool behaviour (through the manager)
  crates/orion-kv-cache/src/manager.rs:470-839    KvCacheManager
  crates/orion-scheduler/src/scheduler.rs:566-1076 Scheduler
  crates/orion-runtime/src/engine.rs:640-959      Engine with the mock model

This is what pins the oracle: the reference holds no golden files for this path, its tests are
behavioural, and the Rust sources cannot be compiled here."""
import pytest

from driver_adapters import DriverErr, Eng, Manager, Sched
from oracle import driver as od

IMPLS = ["oracle", "native"]


@pytest.fixture(params=IMPLS)
def impl(request, pkg):
    return request.param


# ---- table.rs: hash_block ---------------------------------------------------------------------

def _hashers(pkg):
    return [od.hash_block, pkg.engine.hash_block]


def test_hash_block_properties_and_agreement(pkg):
    for h in _hashers(pkg):
        a, b = h(None, [1, 2, 3]), h(None, [1, 2, 3])
        assert a == b and h(a, [4, 5]) == h(b, [4, 5])  # identical_prefixes_hash_identically
        assert h(None, [1, 2, 3]) != h(None, [1, 2, 4]) and h(None, [1, 2, 3]) != h(None, [3, 2, 1])
        assert h(h(None, [10, 11]), [1, 2]) != h(h(None, [20, 21]), [1, 2])  # different prefix
        assert h(None, [1, 2]) != h(0, [1, 2])  # a_root_block_differs_from_the_same_tokens_mid_sequence
        assert h(None, [1, 2]) != h(None, [1, 2, 0])  # length_is_mixed_in
    # the recipe itself, by hand: rotate-left 5, xor, wrapping multiply (table.rs:105-126)
    mask, seed = (1 << 64) - 1, 0x517CC1B727220A95
    st = 0xCBF29CE484222325
    for v in (2, 7, 9):  # length 2, then the tokens
        st = ((((st << 5) | (st >> 59)) & mask) ^ v) * seed & mask
    assert od.hash_block(None, [7, 9]) == st == pkg.engine.hash_block(None, [7, 9])
    chain = None
    for i in range(50):  # bit-exact agreement on a long chain with large token ids
        toks = [(i * 2654435761 + j * 40503) % (1 << 32) for j in range(16)]
        x, y = od.hash_block(chain, toks), pkg.engine.hash_block(chain, toks)
        assert x == y
        chain = x


# ---- block.rs through the manager -----------------------------------------------------------------

def test_free_blocks_are_recycled_oldest_first(impl):
    m = Manager(impl, 3, 4, False)
    for s in (1, 2, 3):
        m.allocate(s, [1] * 4)
    assert [m.table(s)[0] for s in (1, 2, 3)] == [[0], [1], [2]], "a new pool hands out ascending ids"
    for s in (3, 1, 2):
        m.free(s)
    for s, expect in ((4, 2), (5, 0), (6, 1)):
        m.allocate(s, [1] * 4)
        assert m.table(s)[0] == [expect]


def test_a_freed_block_keeps_its_contents_until_reallocated_and_revival_leaves_the_free_list(impl):
    m = Manager(impl, 4, 4, True)
    prompt = [5, 6, 7, 8]
    m.allocate(1, prompt)
    m.commit_prefill(1, prompt)
    blk = m.table(1)[0][0]
    m.free(1)
    ref, ntok, h = m.block_info(blk)
    assert (ref, ntok) == (0, 4) and h == od.hash_block(None, prompt)
    assert m.free_blocks() == 4 and m.num_evictable() == 1
    assert m.allocate(2, prompt) == (0, 1, 4)  # revived by hash
    assert m.free_blocks() == 3 and m.block_info(blk)[0] == 1 and m.block_info(blk)[2] == h


# ---- manager.rs -----------------------------------------------------------------------------------

def test_allocation_reserves_the_right_number_of_blocks(impl):
    m = Manager(impl, 16, 4, True)
    assert m.allocate(1, [1] * 10)[:2] == (3, 0)
    assert m.free_blocks() == 13 and m.table(1)[1] == 10


def test_allocating_the_same_sequence_twice_is_an_internal_error(impl):
    m = Manager(impl, 16, 4, True)
    m.allocate(1, [1] * 4)
    with pytest.raises(DriverErr) as e:
        m.allocate(1, [1] * 4)
    assert e.value.kind == "Internal"


def test_allocation_beyond_capacity_is_refused_before_taking_blocks(impl):
    m = Manager(impl, 2, 4, True)
    with pytest.raises(DriverErr) as e:
        m.allocate(1, [1] * 100)
    assert e.value.kind == "CacheExhausted" and m.free_blocks() == 2 and not m.is_allocated(1)


def test_freeing_returns_every_block_and_unknown_sequences_are_a_no_op(impl):
    m = Manager(impl, 8, 4, True)
    m.allocate(1, [1] * 12)
    assert m.free_blocks() == 5
    m.free(1)
    assert m.free_blocks() == 8 and not m.is_allocated(1)
    m.free(42)
    assert m.free_blocks() == 8


def test_appending_reuses_the_final_block_until_it_fills(impl):
    m = Manager(impl, 8, 4, True)
    m.allocate(1, [1] * 4)
    assert len(m.table(1)[0]) == 1 and m.free_blocks() == 7
    m.append_token(1)
    assert len(m.table(1)[0]) == 2 and m.free_blocks() == 6
    for _ in range(3):
        m.append_token(1)
    assert len(m.table(1)[0]) == 2 and m.table(1)[1] == 8 and m.free_blocks() == 6


def test_append_fails_cleanly_when_the_pool_is_exhausted(impl):
    m = Manager(impl, 1, 4, False)
    m.allocate(1, [1] * 4)
    with pytest.raises(DriverErr) as e:
        m.append_token(1)
    assert e.value.kind == "CacheExhausted" and m.table(1) == ([0], 4)
    with pytest.raises(DriverErr) as e:
        m.append_token(9)
    assert e.value.kind == "Internal"


def test_a_shared_prefix_is_reused_by_a_second_sequence(impl):
    m = Manager(impl, 32, 4, True)
    prompt = list(range(12))
    assert m.allocate(1, prompt) == (3, 0, 0)
    m.commit_prefill(1, prompt)
    assert m.allocate(2, prompt) == (0, 3, 12)
    assert m.free_blocks() == 29 and m.table(1)[0] == m.table(2)[0]


def test_shared_blocks_survive_until_the_last_sequence_releases_them(impl):
    m = Manager(impl, 32, 4, True)
    prompt = list(range(8))
    m.allocate(1, prompt)
    m.commit_prefill(1, prompt)
    m.allocate(2, prompt)
    assert m.free_blocks() == 30
    m.free(1)
    assert m.free_blocks() == 30
    m.free(2)
    assert m.free_blocks() == 32


def test_a_divergent_prompt_shares_only_its_common_prefix(impl):
    m = Manager(impl, 32, 4, True)
    a = [1, 2, 3, 4, 5, 6, 7, 8]
    m.allocate(1, a)
    m.commit_prefill(1, a)
    assert m.allocate(2, [1, 2, 3, 4, 9, 9, 9, 9]) == (1, 1, 4)


def test_partial_uncommitted_and_disabled_prefixes_are_not_shared(impl):
    m = Manager(impl, 32, 4, True)
    p6 = list(range(6))
    m.allocate(1, p6)
    m.commit_prefill(1, p6)
    assert m.allocate(2, p6)[:2] == (1, 1)  # a_partial_trailing_block_is_never_shared
    m = Manager(impl, 32, 4, True)
    p8 = list(range(8))
    m.allocate(1, p8)
    assert m.allocate(2, p8)[:2] == (2, 0)  # uncommitted_prefill_is_not_shared
    m = Manager(impl, 32, 4, False)
    m.allocate(1, p8)
    m.commit_prefill(1, p8)
    assert m.allocate(2, p8)[:2] == (2, 0)  # prefix_caching_can_be_disabled


def test_preemption_reclaims_blocks_and_reports_the_count(impl):
    m = Manager(impl, 8, 4, True)
    m.allocate(1, [1] * 12)
    assert m.preempt(1) == 3 and m.free_blocks() == 8 and not m.is_allocated(1)


def test_eviction_drops_index_entries_and_stops_once_nothing_is_cached(impl):
    m = Manager(impl, 4, 4, True)
    prompt = list(range(8))
    m.allocate(1, prompt)
    m.commit_prefill(1, prompt)
    m.free(1)
    assert (m.entries(), m.num_evictable(), m.free_blocks()) == (2, 2, 4)
    assert m.evict_cached(100) == 2 and m.evict_cached(1) == 0
    assert m.entries() == 0 and m.free_blocks() == 4
    assert m.allocate(2, prompt)[1] == 0


def test_clearing_the_prefix_cache_leaves_blocks_allocatable(impl):
    m = Manager(impl, 4, 4, True)
    prompt = list(range(8))
    m.allocate(1, prompt)
    m.commit_prefill(1, prompt)
    m.free(1)
    m.clear_prefix_cache()
    assert m.entries() == 0 and m.free_blocks() == 4
    m.allocate(2, prompt)
    assert m.free_blocks() == 2


def test_recycling_a_cached_block_invalidates_its_index_entry(impl):
    m = Manager(impl, 2, 4, True)
    original = [1, 2, 3, 4, 5, 6, 7, 8]
    m.allocate(1, original)
    m.commit_prefill(1, original)
    m.free(1)
    assert m.entries() == 2 and m.num_evictable() == 2
    assert m.allocate(2, [9] * 8)[:2] == (2, 0)  # cached_blocks_are_recycled_under_pressure
    assert m.entries() == 0 and m.free_blocks() == 0
    m.free(2)
    assert m.allocate(3, original)[:2] == (2, 0)


def test_stats_admission_checks_and_empty_prompts(impl):
    m = Manager(impl, 10, 4, True)
    m.allocate(1, [1] * 8)
    assert (m.used_blocks(), m.free_blocks(), m.num_sequences()) == (2, 8, 1)
    m = Manager(impl, 3, 4, True)
    assert m.can_allocate(12) and not m.can_allocate(13) and m.blocks_needed_for(13) == 4
    m = Manager(impl, 4, 4, True)
    assert m.allocate(1, [])[0] == 0 and m.free_blocks() == 4


def test_many_sequences_allocate_and_free_without_leaking(impl):
    m = Manager(impl, 64, 4, True)
    for rnd in range(10):
        ids = [rnd * 100 + i for i in range(8)]
        for s in ids:
            m.allocate(s, [1] * 16)
        assert m.free_blocks() == 64 - 32
        for s in ids:
            m.free(s)
        assert m.free_blocks() == 64 and m.num_sequences() == 0


# ---- scheduler.rs ---------------------------------------------------------------------------------

CFG = dict(max_num_seqs=4, max_num_batched_tokens=32, max_model_len=1024, enable_chunked_prefill=True,
           max_waiting_requests=8, prioritize_decode=True)


def sched(impl, blocks, **over):
    return Sched(impl, blocks, 4, False, **{**CFG, **over})


def test_a_single_request_is_prefilled_then_decodes(impl):
    s = sched(impl, 16)
    assert s.schedule() == ([], []) and not s.has_work()
    sid = s.add(8, 4)
    assert s.schedule()[0] == [(sid, 8, 0, True)]
    s.on_token(sid, 100)
    assert s.schedule()[0] == [(sid, 1, 9, False)], "8 prompt + 1 generated: the reference's decode position"


def test_batching_budget_and_running_set_bounds(impl):
    s = sched(impl, 64)
    for _ in range(3):
        s.add(8, 4)
    out = s.schedule()[0]
    assert len(out) == 3 and sum(x[1] for x in out) == 24
    s = sched(impl, 64)
    for _ in range(3):
        s.add(16, 4)
    assert sum(x[1] for x in s.schedule()[0]) <= 32
    s = sched(impl, 256)
    for _ in range(8):
        s.add(1, 4)
    s.schedule()
    assert s.num_running() == 4 and s.num_waiting() == 4


def test_chunked_prefill_splits_a_long_prompt_across_steps(impl):
    s = sched(impl, 64)
    sid = s.add(100, 4)
    consumed = steps = 0
    while True:
        x = s.schedule()[0][0]
        assert x[0] == sid
        if not x[3]:
            break
        assert x[2] == consumed and x[1] <= 32
        consumed += x[1]
        steps += 1
        assert steps < 10
    assert consumed == 100 and steps == 4


def test_a_partially_prefilled_sequence_is_never_stranded(impl):
    s = sched(impl, 64)
    sid = s.add(100, 4)
    first = s.schedule()[0]
    assert first[0][3] and first[0][1] < 100 and s.num_running() == 1 and s.num_waiting() == 0
    second = s.schedule()[0]
    assert second and second[0][0] == sid and second[0][1] > 0


def test_every_admitted_request_eventually_finishes(impl):
    s = sched(impl, 128, max_waiting_requests=64)
    ids = [s.add(n, 5) for n in (4, 60, 8, 100, 16)]
    completed = 0
    for step in range(500):
        for x in s.schedule()[0]:
            if not x[3]:
                s.on_token(x[0], 42)
        completed += len(s.reap())
        if not s.has_work():
            break
        assert step < 499
    assert completed == len(ids) and s.num_running() == 0 and s.num_waiting() == 0


def test_chunked_prefill_interleaves_with_running_decodes(impl):
    s = sched(impl, 128)
    short = s.add(4, 100)
    s.schedule()
    s.on_token(short, 1)
    s.add(200, 4)
    out = s.schedule()[0]
    assert any(x[3] for x in out) and sum(1 for x in out if not x[3]) == 1
    assert any(x[0] == short and not x[3] for x in out) and sum(x[1] for x in out) <= 32


def test_unchunked_prefill_waits_for_a_prompt_that_fits(impl):
    s = sched(impl, 128, enable_chunked_prefill=False)
    a = s.add(30, 100)
    s.schedule()
    s.on_token(a, 1)
    s.add(32, 4)
    assert not any(x[3] for x in s.schedule()[0]) and s.num_waiting() == 1


def test_stop_rules(impl):
    s = sched(impl, 16)
    sid = s.add(8, 100)
    s.schedule()
    assert s.cache.free_blocks() < 16
    assert s.on_token(sid, 2, [2]) == "stop"  # stop_token_finishes_a_sequence_and_frees_its_blocks
    assert len(s.reap()) == 1 and s.cache.free_blocks() == 16 and s.num_running() == 0
    s = sched(impl, 32)
    sid = s.add(4, 3)
    s.schedule()
    assert [s.on_token(sid, t) for t in (10, 11, 12)] == [None, None, "length"]  # max_tokens_terminates_generation
    s = sched(impl, 32)
    sid = s.add([1] * 4, 10, min_tokens=3)
    s.schedule()
    assert [s.on_token(sid, 2, [2]) for _ in range(3)] == [None, None, "stop"]  # min_tokens_suppresses_an_early_eos
    s = sched(impl, 32)
    sid = s.add(4, 10, stop_token_ids=[7])
    s.schedule()
    assert s.on_token(sid, 7) == "stop"


def test_admission_limits(impl):
    s = sched(impl, 1024)
    for _ in range(8):
        s.add(1, 1)
    with pytest.raises(DriverErr) as e:
        s.add(1, 1)
    assert e.value.kind == "QueueFull" and s.stats()["total_rejected"] == 1
    with pytest.raises(DriverErr) as e:
        sched(impl, 1024).add(1000, 100)
    assert e.value.kind == "ContextLengthExceeded"
    s = sched(impl, 4)
    with pytest.raises(DriverErr) as e:
        s.add(100, 4)
    assert e.value.kind == "CacheExhausted" and s.num_waiting() == 0


def test_cancellation(impl):
    s = sched(impl, 32)
    sid = s.add(4, 4)
    assert s.cancel(sid) and s.num_waiting() == 0 and not s.cancel(sid)
    sid = s.add(8, 100)
    s.schedule()
    assert s.cache.free_blocks() < 32
    assert s.cancel(sid) and s.cache.free_blocks() == 32 and s.num_running() == 0


def test_preemption_evicts_the_newest_and_it_keeps_its_tokens(impl):
    s = sched(impl, 4, max_num_seqs=8, max_num_batched_tokens=64)
    a, b = s.add(4, 100), s.add(4, 100)
    s.schedule()
    assert s.num_running() == 2
    preempted = []
    for _ in range(8):
        s.on_token(a, 1)
        s.on_token(b, 1)
        preempted += s.schedule()[1]
    assert preempted and preempted[0] == b and s.stats()["total_preempted"] > 0


def test_a_preempted_sequence_is_rescheduled_before_new_arrivals(impl):
    s = sched(impl, 3, max_num_seqs=2, max_num_batched_tokens=64)
    a, b = s.add(4, 100), s.add(4, 100)
    s.schedule()
    for _ in range(6):
        s.on_token(a, 1)
        s.on_token(b, 1)
        pre = s.schedule()[1]
        if pre:
            nxt = s.schedule()[0]
            assert any(x[0] == pre[0] for x in nxt) or s.cache.free_blocks() == 0
            return
    pytest.fail("cache pressure never caused a preemption")


def test_cache_exhaustion_during_decode_does_not_lose_sequences(impl):
    s = sched(impl, 6, max_num_seqs=8, max_num_batched_tokens=64)
    ids = [s.add(4, 50) for _ in range(4)]
    s.schedule()
    for _ in range(10):
        for sid in ids:
            s.on_token(sid, 1)
        s.reap()
        s.schedule()
        assert s.num_running() + s.num_waiting() + s.stats()["total_finished"] == 4


def test_stats_and_inverted_priority(impl):
    s = sched(impl, 64)
    sid = s.add(8, 4)
    s.schedule()
    assert (s.stats()["total_prefill_tokens"], s.stats()["total_decode_tokens"]) == (8, 0)
    s.on_token(sid, 1)
    s.schedule()
    assert s.stats()["total_decode_tokens"] == 1 and s.stats()["total_admitted"] == 1
    s = sched(impl, 128, prioritize_decode=False, max_num_batched_tokens=8)
    running = s.add(4, 100)
    s.schedule()
    s.on_token(running, 1)
    s.add(8, 4)
    out = s.schedule()[0]
    assert sum(1 for x in out if x[3]) == 1 and sum(1 for x in out if not x[3]) == 0


def test_an_injected_append_failure_is_handled(impl):
    s = sched(impl, 2)
    a, b = s.add(4, 10), s.add(4, 10)
    s.schedule()
    s.cache.fail_next_append()
    for sid in (a, b):
        s.on_token(sid, 1)
    s.schedule()
    assert s.num_running() + s.num_waiting() == 2


def test_prefix_hits_do_not_skip_compute_unless_asked(impl):
    """The reference shares cached blocks but always prefills from position 0 (scheduler.rs:397-399,
    manager.rs:449-451). The opt-in extension starts after the adopted tokens and always computes at
    least the last prompt token."""
    prompt = list(range(100, 112))  # three full blocks of four
    for skip, expect_second, expect_full in ((False, (12, 0), (12, 0)), (True, (4, 8), (1, 11))):
        s = Sched(impl, 32, 4, True, **{**CFG, "skip_cached_prefix": skip})
        a = s.add(prompt[:8] + [7, 7, 7, 7], 4)
        s.schedule()
        s.commit_prefill(a)
        b = s.add(prompt, 4)  # shares the first two blocks with a
        assert s.schedule()[0][-1] == (b, expect_second[0], expect_second[1], True)
        s.commit_prefill(b)
        c = s.add(prompt, 4)  # every block cached: only the last token is computed when skipping
        assert s.schedule()[0][-1] == (c, expect_full[0], expect_full[1], True)
        assert s.stats()["total_skipped_prefill_tokens"] == (8 + 11 if skip else 0)
        assert s.cache.table(b)[0][:3] == s.cache.table(c)[0], "the prompt blocks are shared either way"


def test_decode_positions_follow_the_reference_unless_asked(impl):
    """scheduler.rs:283 feeds the decode token at total_len (pinned by its own test at :621); the
    opt-in alternative uses the token's logical position total_len - 1."""
    for logical, first, second in ((False, 9, 10), (True, 8, 9)):
        s = sched(impl, 16, logical_decode_positions=logical)
        sid = s.add(8, 4)
        s.schedule()
        s.on_token(sid, 100)
        assert s.schedule()[0] == [(sid, 1, first, False)]
        s.on_token(sid, 101)
        assert s.schedule()[0] == [(sid, 1, second, False)]


# ---- engine.rs with the mock model ------------------------------------------------------------------

def mock(favoured):
    """MockModel (engine.rs:563-636): the argmax always lands on ``favoured``."""
    return lambda batch: [favoured] * len(batch.sequence_ids)


def engine(impl, favoured):
    return Eng(impl, mock(favoured), 64, 4, True, eos=[15], max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256)


def run(e, limit):
    steps = 0
    while e.has_work() and steps < limit:
        e.step()
        steps += 1
    return steps


def test_a_request_generates_until_max_tokens(impl):
    e = engine(impl, 5)
    sid = e.submit([1, 2, 3], 4)
    run(e, 20)
    ev = e.events()
    assert [x[2] for x in ev if x[0] == "token"] == [5, 5, 5, 5]
    assert [x[3] for x in ev if x[0] == "token"] == [0, 1, 2, 3]
    assert ev[-1] == ("done", sid, "length", 3, 4)


def test_an_eos_token_stops_generation_early(impl):
    e = engine(impl, 15)
    sid = e.submit([1, 2], 100)
    run(e, 10)
    done = [x for x in e.events() if x[0] == "done"]
    assert done == [("done", sid, "stop", 2, 1)]


def test_several_requests_are_served_concurrently_and_blocks_are_released(impl):
    e = engine(impl, 5)
    free_before = e.sched.cache.free_blocks()
    ids = [e.submit([1, 2], 3) for _ in range(4)]
    run(e, 50)
    ev = e.events()
    for sid in ids:
        mine = [x for x in ev if x[1] == sid]
        assert sum(1 for x in mine if x[0] == "token") == 3 and mine[-1][0] == "done"
    assert e.sched.cache.free_blocks() == free_before and e.num_active() == 0


def test_submission_errors(impl):
    e = engine(impl, 5)
    with pytest.raises(DriverErr) as err:
        e.submit([1], 16, temperature=-1.0)
    assert err.value.kind == "InvalidRequest" and e.sched.num_waiting() == 0
    with pytest.raises(DriverErr) as err:
        e.submit([1] * 300, 10)
    assert err.value.kind == "ContextLengthExceeded"


def test_cancelling_frees_blocks_and_notifies_the_caller(impl):
    e = engine(impl, 5)
    sid = e.submit([1] * 8, 100)
    e.step()
    assert e.sched.cache.free_blocks() < 64
    e.cancel(sid)
    assert e.sched.cache.free_blocks() == 64
    assert ("done", sid, "cancelled", 8, 0) in e.events()
    e.cancel(9999)
    assert e.sched.num_running() == 0
    assert e.step() == 0  # an_empty_step_is_not_an_error


def test_a_long_prompt_is_prefilled_in_chunks_then_decodes(impl):
    e = engine(impl, 5)
    e.submit([1] * 100, 2)
    steps = run(e, 50)
    assert sum(1 for x in e.events() if x[0] == "token") == 2 and steps > 2


def test_the_prefix_cache_serves_a_repeated_prompt(impl):
    e = engine(impl, 5)
    for _ in range(2):
        e.submit(list(range(16)), 1)
        run(e, 20)
    assert e.sched.cache.hits() > 0


def test_a_prompt_with_a_chunk_lost_to_a_failed_step_is_not_offered_for_skipping(impl):
    """Prefill progress is recorded at schedule time and a failed forward rolls nothing back
    (engine.rs:310). With skip_cached_prefix a prompt one of whose chunks was in a failed step must
    not be published: a later request with the same prefix would adopt blocks that hold no keys and
    values and skip computing them. Without the flag the reference's behaviour stays: published, and
    recomputed by whoever adopts it."""
    prompt = list(range(200, 224))  # six blocks of four, three chunks of eight
    for skip in (True, False):
        fail = {"on": False}

        def forward(batch):
            if fail["on"]:
                raise RuntimeError("device refused the step")
            return [3] * len(batch.sequence_ids)

        e = Eng(impl, forward, 64, 4, True, eos=[15], max_num_seqs=4, max_num_batched_tokens=8, max_model_len=256,
                skip_cached_prefix=skip)
        a = e.submit(prompt, 1)
        assert e.step() == 1                      # chunk [0, 8)
        fail["on"] = True
        with pytest.raises(Exception):
            e.step()                              # chunk [8, 16) is scheduled, its forward fails
        fail["on"] = False
        assert e.batch()["positions"] == list(range(8, 16))
        assert e.step() == 1                      # chunk [16, 24) completes the prompt and samples
        assert e.batch()["positions"] == list(range(16, 24))
        assert ("done", a, "length", 24, 1) in e.events()
        assert (e.sched.cache.entries() == 0) == skip, "a prompt with an unwritten chunk is withheld only when skipping"
        b = e.submit(prompt, 1)
        e.step()
        first = e.batch()
        assert first["sequence_ids"] == [b] and first["positions"][0] == 0, "nothing to skip: prefill starts at 0"
        while e.has_work():
            e.step()
        assert e.sched.stats()["total_skipped_prefill_tokens"] == 0
        assert e.sched.cache.entries() == 6       # b ran every chunk, so its prompt is published
        c = e.submit(prompt, 1)
        e.step()
        assert e.batch()["positions"] == ([23] if skip else list(range(0, 8)))
