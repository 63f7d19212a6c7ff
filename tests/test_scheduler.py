"""The scheduler's decisions, with the cache manager but without a GPU: a fake step
that only records what it was asked to run."""
import pytest

from airun_b200.cache import CacheManager
from airun_b200.engine.scheduler import FinishReason, Request, Scheduler
from airun_b200.parts.base import PagedKVSpec
from airun_b200.sampling.sampler import SamplingParams


def make(pages=16, page=4, budget=16, reqs=4, ctx=64):
    m = CacheManager([PagedKVSpec(1, 8, 0)], [None], page, pages, reqs)
    return m, Scheduler(m, budget, reqs, ctx)


def req(rid, n_prompt, max_new=4, eog=()):
    return Request(rid, list(range(1, n_prompt + 1)), SamplingParams.greedy(), max_new, tuple(eog))


def run(m, s, plan, token=7):
    """What the engine does around a step: reserve + commit pages, advance, accept tokens."""
    for e in plan.entries:
        m.reserve(e.request.rid, e.count)
    for e in plan.entries:
        m.commit(e.request.rid, e.count)
    s.advance(plan)
    done = []
    for e in plan.entries:
        if e.wants_logits:
            t = token(e.request) if callable(token) else token
            if s.accept(e.request, t) is not None:
                done.append(e.request)
    m.check_invariants()
    return done


def test_prompt_is_cut_under_the_budget_and_decodes_come_first():
    m, s = make(pages=32, budget=16)
    a, b = req("a", 5), req("b", 30)
    s.add(a)
    s.add(b)
    p = s.plan()
    assert [(e.request.rid, e.start, e.count, e.wants_logits) for e in p.entries] == \
        [("a", 0, 5, True), ("b", 0, 11, False)]
    run(m, s, p)
    p = s.plan()                       # a decodes one token, b gets the rest of the budget
    assert [(e.request.rid, e.start, e.count, e.wants_logits) for e in p.entries] == \
        [("a", 5, 1, True), ("b", 11, 15, False)]
    run(m, s, p)
    p = s.plan()
    assert [(e.request.rid, e.start, e.count, e.wants_logits) for e in p.entries] == \
        [("a", 6, 1, True), ("b", 26, 4, True)]
    run(m, s, p)
    p = s.plan()
    assert [(e.request.rid, e.count) for e in p.entries] == [("a", 1), ("b", 1)]


def test_portion_can_be_as_small_as_the_budget_leaves():
    m, s = make(pages=32, budget=8)
    for i in range(3):
        s.add(req(i, 3, max_new=50))
    run(m, s, s.plan())                # 3 + 3 + 2 tokens
    s.add(req("late", 20))
    p = s.plan()                       # two decode tokens, 1 prompt token of request 2, then "late"
    assert [(e.request.rid, e.count) for e in p.entries] == [(0, 1), (1, 1), (2, 1), ("late", 5)]


def test_finish_reasons_and_pages_come_back():
    m, s = make()
    a = req("a", 3, max_new=2)
    b = req("b", 3, max_new=10, eog=(99,))
    s.add(a)
    s.add(b)
    run(m, s, s.plan())
    assert a.output == [7] and b.output == [7]
    done = run(m, s, s.plan(), token=lambda r: 99 if r.rid == "b" else 8)
    assert {r.rid for r in done} == {"a", "b"}
    assert a.finished == FinishReason.MAX_TOKENS and a.output == [7, 8]
    assert b.finished == FinishReason.END_OF_GENERATION and b.output == [7]     # the end token is not emitted
    assert m.free_pages() == {0: 16} and not s.has_work()
    c = req("c", 4, max_new=100)
    c.cancelled = False
    s.add(c)
    run(m, s, s.plan())
    c.cancelled = True
    p = s.plan()
    assert c.finished == FinishReason.CANCELLED and c in p.finished and m.free_pages() == {0: 16}


def test_context_limit_ends_a_request():
    m, s = make(pages=32, ctx=8)
    a = req("a", 6, max_new=100)
    s.add(a)
    while s.has_work():
        run(m, s, s.plan())
    assert a.finished == FinishReason.CONTEXT_FULL and a.num_tokens == 8


def test_refused_at_submission():
    m, s = make(pages=4, page=4, ctx=64)        # the pool holds 16 tokens
    big = req("big", 16)
    s.add(big)
    assert big.finished == FinishReason.REFUSED and not s.has_work()
    empty = Request("e", [], SamplingParams.greedy(), 4)
    s.add(empty)
    assert empty.finished == FinishReason.REFUSED


def test_out_of_pages_preempts_the_newest_and_recomputes_it():
    m, s = make(pages=6, page=4, budget=32)      # 24 tokens in all
    a, b = req("a", 10, max_new=20), req("b", 9, max_new=20)
    s.add(a)
    s.add(b)
    run(m, s, s.plan())                          # a: 3 pages, b: 3 pages, pool full
    assert m.free_pages() == {0: 0}
    run(m, s, s.plan())                          # both decode inside their last page
    run(m, s, s.plan())
    assert a.num_tokens == 13 and b.num_tokens == 12
    p = s.plan()                                 # b needs a 4th page: none free, so the newest (b) goes
    assert p.preempted == [b] and [e.request.rid for e in p.entries] == ["a"]
    assert b.num_computed == 0 and b.preemptions == 1 and s.waiting[0] is b
    assert len(b.output) == 3                    # what it produced is kept and recomputed later
    run(m, s, p)
    while True:
        p = s.plan()
        if a.finished is not None:
            break
        assert all(e.request is a for e in p.entries)      # b cannot come back while a fills the pool
        run(m, s, p)
    # a filled the pool and ended (ContextFull); in the same plan b returns with prompt + its 3 tokens
    assert a.finished == FinishReason.CONTEXT_FULL and a in p.finished
    assert [(e.request.rid, e.start, e.count, e.wants_logits) for e in p.entries] == [("b", 0, 12, True)]
    run(m, s, p)
    while s.has_work():
        run(m, s, s.plan())
    assert b.finished in (FinishReason.MAX_TOKENS, FinishReason.CONTEXT_FULL)
    assert m.free_pages() == {0: 6}
    assert s.stats["preemptions"] >= 1


def test_a_request_alone_that_cannot_grow_ends_with_context_full():
    m, s = make(pages=3, page=4, budget=32, ctx=64)
    a = req("a", 11, max_new=50)
    s.add(a)
    while s.has_work():
        run(m, s, s.plan())
    assert a.finished == FinishReason.CONTEXT_FULL
    assert a.num_tokens == 13 and a.num_computed == 12     # 12 tokens fill the pool; the 13th was sampled, not run
    assert m.free_pages() == {0: 3}


def test_prefills_that_block_each_other_are_untangled():
    m, s = make(pages=8, page=4, budget=10, reqs=4)      # 32 tokens, two prompts of 20
    a, b = req("a", 20, max_new=2), req("b", 20, max_new=2)
    s.add(a)
    s.add(b)
    steps = 0
    while s.has_work() and steps < 100:
        run(m, s, s.plan())
        steps += 1
    assert a.finished == FinishReason.MAX_TOKENS and b.finished == FinishReason.MAX_TOKENS
    assert m.free_pages() == {0: 8}


def test_slots_limit_admission():
    m, s = make(pages=64, reqs=2, budget=64)
    rs = [req(i, 3, max_new=3) for i in range(5)]
    for r in rs:
        s.add(r)
    seen_running = 0
    while s.has_work():
        p = s.plan()
        seen_running = max(seen_running, len(s.running))
        run(m, s, p)
    assert seen_running == 2 and all(r.finished == FinishReason.MAX_TOKENS for r in rs)
