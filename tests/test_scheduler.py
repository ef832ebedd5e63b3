"""The scheduler's decisions, on the host only, with the step function replaced
by a stand-in that returns a fixed token (as the reference's tests do with
their fake runner, tests/scheduler_test.cc:42-50)."""
import pytest

from chibillm_b200.cache import CacheManager, GroupLayout
from chibillm_b200.engine.scheduler import (ADMITTED, DEFERRED, TOO_LARGE, Scheduler, SchedulerConfig,
                                            SchedulerError, Sequence)
from chibillm_b200.sampling import SamplingParams, uniform_for

EOS = 99


def make(pages=16, page_size=4, **cfg):
    cache = CacheManager([GroupLayout("full", 1, 8, None, page_size, pages, 1)], max_requests=8)
    return Scheduler(SchedulerConfig(**cfg), cache, EOS), cache


def seq(i, n, max_new=4, **kw):
    return Sequence(i, list(range(1, n + 1)), SamplingParams(max_new_tokens=max_new, **kw))


def run_step(s, token=42):
    b = s.schedule()
    return b, s.complete(b.batch_id, [token] * b.sample_count)


def test_whole_prompt_then_decode_until_length():
    s, cache = make(max_sequences=4, max_batch_tokens=64, prefill_chunk_tokens=8)
    assert s.try_add(seq("a", 10, max_new=3)) == ADMITTED
    b, ups = run_step(s)
    assert [(i.seq_id, i.first, i.count, i.sample) for i in b.items] == [("a", 0, 10, True)]
    assert ups[0].token == 42 and ups[0].finish_reason is None
    b, ups = run_step(s)
    assert [(i.first, i.count) for i in b.items] == [(10, 1)]       # the one-token gap
    b, ups = run_step(s)
    assert ups[0].finish_reason == "len_limit"
    assert not s.has_work() and cache.free_pages("full") == 16
    assert s.remove("a").completion == [42, 42, 42]


def test_eos_is_checked_before_length():
    s, _ = make()
    s.add(seq("a", 3, max_new=1))
    _, ups = run_step(s, token=EOS)
    assert ups[0].finish_reason == "eos"
    s.add(seq("b", 3, max_new=2, ignore_eos=True))
    _, ups = run_step(s, token=EOS)
    assert ups[0].finish_reason is None
    _, ups = run_step(s, token=EOS)
    assert ups[0].finish_reason == "len_limit"


def test_portions_under_contention_and_mixed_batches():
    s, _ = make(pages=64, max_sequences=4, max_batch_tokens=20, prefill_chunk_tokens=8)
    s.add(seq("a", 30, max_new=5))
    s.add(seq("b", 5, max_new=5))
    b, _ = run_step(s)
    # two waiting: portions of 8; a is cut, b fits whole and samples
    assert [(i.seq_id, i.count, i.sample) for i in b.items] == [("a", 8, False), ("b", 5, True)]
    b, _ = run_step(s)
    # b decodes first (one token), a's next portion rides in the same batch
    assert [(i.seq_id, i.first, i.count, i.sample) for i in b.items] == [("b", 5, 1, True), ("a", 8, 8, False)]
    b, _ = run_step(s)
    assert [(i.seq_id, i.first, i.count) for i in b.items] == [("b", 6, 1), ("a", 16, 8)]
    b, _ = run_step(s)
    assert [(i.seq_id, i.first, i.count, i.sample) for i in b.items] == [("b", 7, 1, True), ("a", 24, 6, True)]
    b, _ = run_step(s)
    assert sorted((i.seq_id, i.count) for i in b.items) == [("a", 1), ("b", 1)]
    s.check_invariants()


def test_token_budget_cuts_a_lone_prompt():
    s, _ = make(pages=64, max_sequences=2, max_batch_tokens=12, prefill_chunk_tokens=4)
    s.add(seq("a", 30))
    counts = []
    while s.sequences["a"].status == "waiting":
        b, _ = run_step(s)
        counts.append(b.items[0].count)
    assert counts == [12, 12, 6]                 # alone: the quantum is the whole budget


def test_admission_too_large_deferred_admitted():
    s, cache = make(pages=8, page_size=4, max_sequences=2, max_batch_tokens=64)
    assert s.try_add(seq("big", 30, max_new=4)) == TOO_LARGE         # 33 tokens -> 9 pages > 8
    assert s.try_add(seq("a", 13, max_new=4)) == ADMITTED            # 16 tokens -> 4 pages
    assert s.try_add(seq("b", 14, max_new=4)) == DEFERRED            # 17 tokens -> 5 pages, 4 left
    assert s.try_add(seq("c", 9, max_new=4)) == ADMITTED             # 12 tokens -> 3 pages
    assert s.try_add(seq("d", 1, max_new=1)) == DEFERRED             # two sequences are live
    with pytest.raises(SchedulerError) as e:
        s.add(seq("e", 1, max_new=1))
    assert e.value.code == "capacity_deferred"
    with pytest.raises(SchedulerError) as e:
        s.try_add(seq("a", 2))
    assert e.value.code == "duplicate_sequence_id"
    # pages never run out in the middle: run everything to the end
    while s.has_work():
        run_step(s)
        cache.check_invariants()
    assert cache.free_pages("full") == 8
    assert s.try_add(seq("b", 14, max_new=4)) == ADMITTED


def test_abort_keeps_pages_and_retry_is_identical():
    s, cache = make(max_batch_tokens=6, prefill_chunk_tokens=6)
    s.add(seq("a", 10))
    b1 = s.schedule()
    held = cache.free_pages("full")
    with pytest.raises(SchedulerError):
        s.schedule()                              # one batch at a time
    with pytest.raises(SchedulerError) as e:
        s.complete(b1.batch_id, [1, 2])           # wrong number of samples: nothing changes
    assert e.value.code == "result_count_mismatch"
    s.abort(b1.batch_id)
    assert cache.free_pages("full") == held and s.sequences["a"].scheduled == 0
    b2 = s.schedule()
    assert [(i.seq_id, i.first, i.count, i.sample) for i in b2.items] == \
           [(i.seq_id, i.first, i.count, i.sample) for i in b1.items]
    s.complete(b2.batch_id, [])
    s.check_invariants()


def test_cancel_frees_and_remove_needs_finished():
    s, cache = make()
    s.add(seq("a", 10))
    run_step(s)
    with pytest.raises(SchedulerError):
        s.remove("a")
    s.cancel("a")
    assert cache.free_pages("full") == 16 and s.sequences["a"].finish_reason == "cancelled"
    assert not s.has_work()
    s.remove("a")
    with pytest.raises(SchedulerError):
        s.cancel("a")


def test_bad_sequences_and_config():
    with pytest.raises(SchedulerError):
        Sequence(1, [], SamplingParams())
    with pytest.raises(SchedulerError):
        Sequence(1, [1], SamplingParams(max_new_tokens=0))
    with pytest.raises(SchedulerError):
        make(max_batch_tokens=0)
    s, _ = make()
    with pytest.raises(SchedulerError) as e:
        s.schedule()
    assert e.value.code == "no_runnable_sequences"


def test_uniforms_depend_on_their_arguments_only():
    a = uniform_for(1, 5, 0)
    assert a == uniform_for(1, 5, 0) and 0.0 <= a < 1.0
    assert len({uniform_for(1, 5, i) for i in range(100)}) == 100
    assert uniform_for(2, 5, 0) != a and uniform_for(1, 6, 0) != a
    vals = [uniform_for(7, k, i) for k in range(50) for i in range(50)]
    assert 0.45 < sum(vals) / len(vals) < 0.55 and max(vals) < 1.0
