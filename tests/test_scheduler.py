"""The scheduler's decisions on the host, with the cache manager and no model."""
import random

import pytest

from return_b200.cache.manager import CacheManager, GroupSpec, KVCapacityError
from return_b200.engine.request import Request
from return_b200.engine.scheduler import Scheduler


def _sched(pages=8, page=4, max_reside=3, chunk=8, max_len=64):
    m = CacheManager([GroupSpec("full", page, pages)], max_reside)
    return m, Scheduler(m, chunk, max_len)


def _run(s, m, tok=7, limit=500, stop_after=None):
    """Drives the scheduler with a model that always says ``tok``; returns the plans."""
    plans = []
    while s.has_unfinished():
        assert len(plans) < limit, "the scheduler does not make progress"
        p = s.schedule()
        plans.append(p)
        s.commit(p, {e.request.id: (tok, -1.0) for e in p.entries if e.sample})
        m.check()
    return plans


def test_budget_cuts_prompts_and_decodes_go_first():
    m, s = _sched(pages=16, chunk=8)
    a, b = Request("a", list(range(5)), max_new_tokens=3), Request("b", list(range(13)), max_new_tokens=2)
    s.add(a), s.add(b)
    p = s.schedule()
    assert [(e.request.id, len(e.tokens), e.start, e.sample) for e in p.entries] == [("a", 5, 0, True), ("b", 3, 0, False)]
    s.commit(p, {"a": (9, 0.0)})
    p = s.schedule()        # a decodes with one token of the budget, b takes the other seven
    assert [(e.request.id, len(e.tokens), e.start, e.sample) for e in p.entries] == [("a", 1, 5, True), ("b", 7, 3, False)]
    assert p.entries[0].tokens == [9]
    s.commit(p, {"a": (9, 0.0)})
    p = s.schedule()
    assert [(e.request.id, len(e.tokens), e.start, e.sample) for e in p.entries] == [("a", 1, 6, True), ("b", 3, 10, True)]
    done = s.commit(p, {"a": (9, 0.0), "b": (4, 0.0)})
    assert [r.id for r in done] == ["a"] and a.finish_reason == "length" and a.output == [9, 9, 9]
    assert "a" not in m
    p = s.schedule()
    assert [(e.request.id, e.tokens, e.start) for e in p.entries] == [("b", [4], 13)]
    done = s.commit(p, {"b": (4, 0.0)})
    assert done == [b] and not s.has_unfinished() and m.pages_used() == [0]


def test_admission_is_fifo_and_bounded_by_slots():
    m, s = _sched(pages=32, max_reside=2, chunk=64)
    reqs = [Request(i, [1, 2, 3], max_new_tokens=2) for i in range(4)]
    for r in reqs:
        s.add(r)
    p = s.schedule()
    assert [e.request.id for e in p.entries] == [0, 1] and len(s.waiting) == 2
    s.commit(p, {0: (5, 0.0), 1: (5, 0.0)})
    p = s.schedule()
    assert [e.request.id for e in p.entries] == [0, 1]
    s.commit(p, {0: (5, 0.0), 1: (5, 0.0)})                   # both finish, slots come back
    p = s.schedule()
    assert [e.request.id for e in p.entries] == [2, 3]


def test_stop_sequences_end_a_request_and_stay_in_the_output():
    m, s = _sched(pages=16, chunk=64)
    r = Request("r", [1, 2], max_new_tokens=10, stop_ids=[[7, 8], [3]])
    s.add(r)
    for tok in (7, 7, 8, 9):
        p = s.schedule()
        s.commit(p, {"r": (tok, 0.0)})
        if not s.has_unfinished():
            break
    assert r.output == [7, 7, 8] and r.finish_reason == "stop" and m.pages_used() == [0]


def test_out_of_pages_preempts_the_youngest_and_recomputes():
    # 8 pages of 4 = 32 tokens.  Three requests of 9 prompt tokens (3 pages each, 27 tokens) fit; they
    # cannot all grow to 14 tokens (4 pages each = 12 pages).
    m, s = _sched(pages=8, page=4, max_reside=3, chunk=32)
    reqs = [Request(i, list(range(9)), max_new_tokens=5) for i in range(3)]
    for r in reqs:
        s.add(r)
    plans = _run(s, m)
    assert all(r.finish_reason == "length" and r.output == [7] * 5 for r in reqs)
    preempted = [r.id for p in plans for r in p.preempted]
    assert preempted and set(preempted) <= {1, 2} and 0 not in preempted      # the oldest never gives way
    assert reqs[2].num_preemptions >= 1
    # after a preemption the request comes back with prompt + output as its prompt
    for p in plans:
        for e in p.entries:
            if e.request.num_preemptions and e.start == 0:
                assert e.tokens[:9] == list(range(9))[:len(e.tokens)]
    assert m.pages_used() == [0] and m.free_slots == 3


def test_decode_is_never_starved_by_new_prompts():
    m, s = _sched(pages=6, page=4, max_reside=3, chunk=16)
    a = Request("a", list(range(8)), max_new_tokens=12)
    s.add(a)
    p = s.schedule()
    s.commit(p, {"a": (1, 0.0)})
    s.add(Request("b", list(range(15)), max_new_tokens=2))       # wants 4 pages, 4 are free: fits for now
    steps = 0
    while a.finish_reason is None:
        p = s.schedule()
        assert any(e.request is a for e in p.entries), "the running decode was skipped"
        s.commit(p, {e.request.id: (1, 0.0) for e in p.entries if e.sample})
        m.check()
        steps += 1
        assert steps < 40
    assert len(a.output) == 12


def test_request_that_cannot_fit_alone_fails_with_capacity_error():
    m, s = _sched(pages=4, page=4, max_reside=2, chunk=64, max_len=64)
    with pytest.raises(KVCapacityError):
        s.add(Request("huge", list(range(17)), max_new_tokens=1))        # prompt > 16 token slots: at submit
    r = Request("grows", list(range(14)), max_new_tokens=10)               # fits now, outgrows the pool later
    s.add(r)
    plans = _run(s, m)
    assert r.finish_reason == "error" and isinstance(r.error, KVCapacityError)
    assert [q.id for p in plans for q in p.failed] == ["grows"]
    assert len(r.output) == 3 and m.pages_used() == [0] and m.free_slots == 2   # 14 + 3 tokens would need a 5th page
    with pytest.raises(ValueError):
        s.add(Request("empty", []))


@pytest.mark.parametrize("seed", range(6))
def test_random_load_finishes_everything_and_leaks_nothing(seed):
    rng = random.Random(seed)
    m = CacheManager([GroupSpec("full", 4, 24), GroupSpec("win", 4, 24, window=10)], 4)
    s = Scheduler(m, rng.choice([5, 16, 64]), 200)
    reqs = [Request(i, [rng.randrange(50) for _ in range(rng.randint(1, 40))], max_new_tokens=rng.randint(1, 25))
            for i in range(25)]
    pending = list(reqs)
    steps = 0
    while pending or s.has_unfinished():
        for _ in range(rng.randint(0, 2)):
            if pending:
                s.add(pending.pop(0))
        p = s.schedule()
        total = sum(len(e.tokens) for e in p.entries)
        assert total <= s.prefill_chunk
        assert len({e.request.id for e in p.entries}) == len(p.entries)
        for e in p.entries:
            assert e.tokens == e.request.all_ids[e.start:e.start + len(e.tokens)]
            assert m.length(e.request.id) == e.start + len(e.tokens)
        s.commit(p, {e.request.id: (rng.randrange(50), 0.0) for e in p.entries if e.sample})
        m.check()
        steps += 1
        assert steps < 5000
    assert all(r.finish_reason == "length" and len(r.output) == r.max_new_tokens for r in reqs)
    assert m.pages_used() == [0, 0] and m.free_slots == 4


def test_kept_session_resumes_behind_its_cache_and_is_released():
    m, s = _sched(pages=16, page=4, max_reside=2, chunk=32)
    a = Request("s", [1, 2, 3, 4, 5], max_new_tokens=3, keep=True)
    s.add(a)
    _run(s, m, tok=7)
    assert a.output == [7, 7, 7] and list(s.kept) == ["s"]
    assert s.kept["s"] == [1, 2, 3, 4, 5, 7, 7] and m.length("s") == 7        # the last sampled token was not fed
    assert m.pages_used() == [2] and m.free_slots == 1
    # the follow-up brings the whole conversation; only what is new runs
    b = Request("s", [1, 2, 3, 4, 5, 7, 7, 7, 9, 9], max_new_tokens=2)
    s.add(b)
    p = s.schedule()
    assert [(e.request.id, e.tokens, e.start, e.sample) for e in p.entries] == [("s", [7, 9, 9], 7, True)]
    s.commit(p, {"s": (8, 0.0)})
    _run(s, m, tok=8)
    assert b.output == [8, 8] and not s.kept and m.pages_used() == [0] and m.free_slots == 2     # b kept nothing
    # release of a kept session
    c = Request("t", [1, 2, 3], max_new_tokens=1, keep=True)
    s.add(c)
    _run(s, m)
    assert "t" in s.kept and s.release("t") and not s.kept and m.pages_used() == [0]
    assert not s.release("t")
    m.check()


def test_follow_up_that_does_not_continue_the_kept_tokens_starts_from_nothing():
    m, s = _sched(pages=16, page=4, chunk=32)
    s.add(Request("s", [1, 2, 3, 4], max_new_tokens=2, keep=True))
    _run(s, m, tok=7)
    b = Request("s", [1, 2, 9, 4, 7, 5], max_new_tokens=1)
    s.add(b)
    assert "s" not in m and b.num_computed == 0
    p = s.schedule()
    assert [(e.tokens, e.start) for e in p.entries] == [([1, 2, 9, 4, 7, 5], 0)]
    s.commit(p, {"s": (3, 0.0)})
    m.check()


def test_kept_sessions_give_way_before_running_requests_are_preempted():
    m, s = _sched(pages=6, page=4, max_reside=2, chunk=32)
    for name in ("k1", "k2"):
        s.add(Request(name, list(range(7)), max_new_tokens=2, keep=True))
    _run(s, m)
    assert list(s.kept) == ["k1", "k2"] and m.pages_used() == [4] and m.free_slots == 0
    # a new request needs a slot and more pages than are free: the session kept longest goes first
    n = Request("n", list(range(11)), max_new_tokens=2)
    s.add(n)
    p = s.schedule()
    assert [e.request.id for e in p.entries] == ["n"] and not p.preempted
    assert list(s.kept) == ["k2"]
    s.commit(p, {"n": (5, 0.0)})
    _run(s, m, tok=5)
    assert n.output == [5, 5]
    # k2 is still there for its follow-up
    f = Request("k2", list(range(7)) + [7, 7, 1], max_new_tokens=1)
    s.add(f)
    p = s.schedule()
    assert p.entries[0].start == 8 and p.entries[0].tokens == [7, 1]
    m.check()


def test_truncate_gives_pages_back():
    m = CacheManager([GroupSpec("full", 4, 8)], 2)
    m.add("a")
    m.append("a", 10)
    assert m.pages_used() == [3]
    m.truncate("a", 9)
    assert m.length("a") == 9 and m.pages_used() == [3]
    m.truncate("a", 4)
    assert m.pages_used() == [1] and m.append("a", 1) == 4
    m.truncatable = False
    with pytest.raises(ValueError, match="nothing can be taken back"):
        m.truncate("a", 2)
    m.check()
