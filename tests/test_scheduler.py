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


# ----------------------------------------------------------------------------- kept caches of finished requests
class FakePages:
    """Stands in for the device: what token every (page, place) holds, the page copies the scheduler
    asks for, and a check that a request's block table names exactly its own tokens."""

    def __init__(self, m):
        self.m, self.cell, self.copies = m, {}, 0

    def run_copies(self, plan):
        ps = self.m.page_size
        for gid, src, dst in plan.pages:
            self.copies += 1
            for k in range(ps):
                self.cell[(dst, k)] = self.cell.get((src, k))

    def step(self, s, plan, token=7):
        ps = self.m.page_size
        for e in plan.entries:
            self.m.reserve(e.request.rid, e.count)
        for e in plan.entries:                       # the step writes its tokens' keys, then reads all of them
            bt = self.m.block_table(e.request.rid, 0)
            toks = e.request.tokens
            for pos in range(e.start, e.start + e.count):
                holders = [r for r in self.m.requests if bt[pos // ps] in self.m.block_table(r, 0)]
                assert holders == [e.request.rid], "a shared page is written"
                self.cell[(bt[pos // ps], pos % ps)] = toks[pos]
            for pos in range(e.start + e.count):
                assert self.cell.get((bt[pos // ps], pos % ps)) == toks[pos], (e.request.rid, pos)
        for e in plan.entries:
            self.m.commit(e.request.rid, e.count)
        s.advance(plan)
        done = []
        for e in plan.entries:
            if e.wants_logits:
                t = token(e.request) if callable(token) else token
                if s.accept(e.request, t) is not None:
                    done.append(e.request)
        self.m.check_invariants()
        return done


def make_kept(pages=16, page=4, budget=64, reqs=4, ctx=64):
    m = CacheManager([PagedKVSpec(1, 8, 0)], [None], page, pages, reqs)
    dev = FakePages(m)
    return m, Scheduler(m, budget, reqs, ctx, prefix_cache=True, run_copies=dev.run_copies), dev


def drain(s, dev, token=7):
    while s.has_work():
        dev.step(s, s.plan(), token)


def test_a_later_prompt_starts_from_the_kept_cache_of_an_earlier_one():
    m, s, dev = make_kept()
    a = Request("a", list(range(100, 114)), SamplingParams.greedy(), 3)          # 14 prompt tokens + 3 generated
    s.add(a)
    drain(s, dev)
    assert a.finished == FinishReason.MAX_TOKENS and len(s.kept) == 1 and len(m.requests) == 1
    kept_tokens = next(iter(s.kept.values()))
    assert kept_tokens == a.tokens[:16]                                           # the last token was never fed
    # same first 10 tokens: two whole pages are shared, the cut falls into the third (copied)
    b = Request("b", list(range(100, 110)) + [500, 501, 502], SamplingParams.greedy(), 2)
    s.add(b)
    p = s.plan()
    assert [(e.request.rid, e.start, e.count, e.wants_logits) for e in p.entries] == [("b", 10, 3, True)]
    assert s.stats["prefix_hits"] == 1 and s.stats["prefix_tokens"] == 10 and dev.copies == 1
    kept_name = next(iter(s.kept))
    assert m.block_table("b", 0)[:2] == m.block_table(kept_name, 0)[:2] and \
        m.block_table("b", 0)[2] != m.block_table(kept_name, 0)[2]
    dev.step(s, p)
    drain(s, dev)
    assert b.finished == FinishReason.MAX_TOKENS and len(s.kept) == 2
    # an identical prompt: everything but its last token is reused, which is computed for the logits
    c = Request("c", list(range(100, 114)), SamplingParams.greedy(), 1)
    s.add(c)
    p = s.plan()
    assert [(e.start, e.count, e.wants_logits) for e in p.entries] == [(13, 1, True)]
    dev.step(s, p)
    # less than a page in common: computed from the start
    d = Request("d", [100, 101, 9, 9, 9, 9], SamplingParams.greedy(), 1)
    s.add(d)
    p = s.plan()
    assert [(e.start, e.count) for e in p.entries] == [(0, 6)]
    dev.step(s, p)
    m.check_invariants()


def test_kept_caches_go_before_anybody_is_preempted_oldest_first():
    m, s, dev = make_kept(pages=8, page=4, reqs=3)
    for name, first in (("a", 100), ("b", 200)):                # two kept caches of 3 pages each (10 + 2 tokens)
        s.add(Request(name, list(range(first, first + 10)), SamplingParams.greedy(), 3))
        drain(s, dev)
    assert len(s.kept) == 2 and m.free_pages()[0] == 2
    first_kept, second_kept = list(s.kept)
    c = Request("c", list(range(300, 318)), SamplingParams.greedy(), 2)      # needs 5 pages: the oldest kept cache goes
    s.add(c)
    p = s.plan()
    assert [(e.start, e.count) for e in p.entries] == [(0, 18)] and not p.preempted
    assert list(s.kept) == [second_kept] and s.stats["prefix_evictions"] == 1
    dev.step(s, p)
    drain(s, dev)                                                 # c decodes past 20 tokens: needs page 6 of 8
    assert c.finished == FinishReason.MAX_TOKENS and s.stats["preemptions"] == 0
    # request slots: 3 in all; kept caches hold them until a new request needs one
    m.check_invariants()
    for i in range(4):
        s.add(Request(("e", i), [700 + i, 1, 2, 3, 4], SamplingParams.greedy(), 1))
    drain(s, dev)
    assert s.stats["preemptions"] == 0 and len(m.requests) <= 3


def test_using_a_kept_cache_makes_it_the_last_to_go_and_forks_evict_too():
    m, s, dev = make_kept(pages=12, page=4, reqs=4)
    for name, first in (("a", 100), ("b", 200)):
        s.add(Request(name, list(range(first, first + 8)), SamplingParams.greedy(), 1))
        drain(s, dev)
    ka, kb = list(s.kept)
    s.add(Request("a2", list(range(100, 108)) + [1], SamplingParams.greedy(), 4))    # uses a's cache
    p = s.plan()
    assert p.entries[0].start == 8 and list(s.kept) == [kb, ka]
    dev.step(s, p)
    live = s.running[0]
    child = Request("a3", list(live.tokens), SamplingParams.greedy(), 2)
    dev.run_copies(s.fork(live, child))
    drain(s, dev)
    m.check_invariants()


def test_models_that_cannot_be_cut_back_keep_nothing():
    m = CacheManager([PagedKVSpec(1, 8, 6)], [None], 4, 16, 4)                   # a window of 6 keys
    s = Scheduler(m, 64, 4, 64, prefix_cache=True)
    assert not s.prefix_cache
    s.add(req("a", 9, max_new=2))
    while s.has_work():
        run(m, s, s.plan())
    assert not s.kept and not m.requests


def test_random_traffic_with_kept_caches_never_reads_a_wrong_token():
    import random
    rnd = random.Random(5)
    m, s, dev = make_kept(pages=24, page=4, budget=24, reqs=4, ctx=48)
    stems = [[rnd.randrange(50, 60) for _ in range(20)] for _ in range(3)]
    done = 0
    for i in range(60):
        stem = rnd.choice(stems)
        prompt = stem[:rnd.randrange(1, 20)] + [rnd.randrange(1000, 1010) for _ in range(rnd.randrange(0, 6))]
        s.add(Request(("r", i), prompt, SamplingParams.greedy(), rnd.randrange(1, 6)))
        for _ in range(rnd.randrange(0, 4)):
            if s.has_work():
                done += len(dev.step(s, s.plan(), token=lambda r: rnd.randrange(50, 60)))
    while s.has_work():
        done += len(dev.step(s, s.plan(), token=lambda r: rnd.randrange(50, 60)))
    assert done == 60 and s.stats["prefix_hits"] > 5
    while s._drop_kept():
        pass
    assert not m.requests and m.free_pages()[0] == 24
    m.check_invariants()


@pytest.mark.parametrize("ps,pages", [(16, 10), (8, 17)])
def test_turns_of_a_conversation_in_a_pool_that_is_almost_full(ps, pages):
    """A first prompt, then the prompt + its answer + more, the same again, and a prompt that leaves the
    others inside a page, in a pool so small that reuse itself finds no free page until another kept
    cache has gone."""
    import random
    m = CacheManager([PagedKVSpec(1, 8, 0)], [None], ps, pages, 4, max_blocks=(128 + ps - 1) // ps)
    dev = FakePages(m)
    s = Scheduler(m, 32, 4, 128, prefix_cache=True, run_copies=dev.run_copies)
    rnd = random.Random(1)

    def ids(n):
        return [rnd.randrange(200, 250) for _ in range(n)]

    def generate(prompts, n):
        rs = [Request(("g", rnd.random()), list(p), SamplingParams.greedy(), n) for p in prompts]
        for r in rs:
            s.add(r)
        drain(s, dev, token=lambda r: sum(r.tokens) % 97 + 3)         # a "model": the next token follows from the sequence
        return [r.output for r in rs]

    turn1 = ids(3 * ps + 5)
    out1 = generate([turn1], 9)[0]
    turn2 = turn1 + out1 + ids(11)
    res = generate([turn2, ids(2 * ps + 3)], 7)
    st = s.stats
    assert st["prefix_hits"] == 1 and st["prefix_tokens"] == len(turn1) + len(out1) - 1
    assert generate([turn2], 7)[0] == res[0]
    assert st["prefix_hits"] == 2 and st["prefix_tokens"] == len(turn1) + len(out1) - 1 + len(turn2) - 1
    generate([turn2[:2 * ps + 3] + ids(40)], 6)
    assert st["prefix_hits"] == 3 and st["prefix_evictions"] >= 1 and st["preemptions"] == 0
    while s._drop_kept():
        pass
    assert not m.requests and m.free_pages()[0] == pages


# ----------------------------------------------------------------------------- the product's tile plan (host arithmetic)
def test_product_plan_takes_every_shape_and_stays_within_the_kernel_limits():
    """``plan_gemm`` decides (swapped, tile width, K slices) on the host; whatever the sizes, its answer
    must be one the kernel's entry point accepts: a tile width it is built for, at least one slice and
    no more than there are 64-wide K blocks, and for split products few enough CTAs to be resident at once."""
    import random
    from airun_b200.kernels.fast import SPLIT_CTAS, STREAM_CTAS, plan_gemm
    rnd = random.Random(0)
    shapes = [(1, 4096, 4096), (8, 6144, 4096), (8, 24576, 4096), (8, 4096, 12288), (64, 4096, 12288), (17, 4096, 4096),
              (2048, 6144, 4096), (2048, 24576, 4096), (129, 256, 64), (300, 100, 8), (1, 151936, 4096), (128, 151936, 4096)]
    shapes += [(rnd.randrange(1, 3000), rnd.randrange(1, 40000), 8 * rnd.randrange(1, 2000)) for _ in range(2000)]
    for M, N, K in shapes:
        swap, bn, ks = plan_gemm(M, N, K)
        kb = (K + 63) // 64
        assert ks >= 1 and ks <= max(kb, 1), (M, N, K, ks)
        if swap:
            assert M <= 128 and bn in (16, 32, 64, 128) and bn >= min(M, 128)
            tiles = (N + 127) // 128
            if ks > 1:
                assert tiles * ks <= (STREAM_CTAS if M <= 16 else SPLIT_CTAS) and (M <= 16 or ks <= 8)
        else:
            assert (M > 128 and bn in (128, 256)) or (64 < M <= 128 and bn == 256 and ks == 1 and (N + 255) // 256 >= 96)
            if ks > 1:
                assert ((M + 127) // 128) * ((N + bn - 1) // bn) * ks <= 148
    assert plan_gemm(8, 24576, 4096) == (True, 16, 1) and plan_gemm(2048, 24576, 4096) == (False, 256, 1)
    # the widest products read fewer activation bytes per weight byte as 128 x 256 tiles from 65 tokens on
    assert plan_gemm(64, 24576, 4096) == (True, 64, 1) and plan_gemm(65, 24576, 4096) == (False, 256, 1)
    assert plan_gemm(128, 151936, 4096) == (False, 256, 1) and plan_gemm(128, 4096, 12288)[0] is True
    # a GPU with another SM count gets plans sized for it, not for 148 SMs
    from airun_b200.kernels.fast import Machine
    small = Machine(66)
    assert small.stream_ctas == 132 and small.split_ctas <= 2 * 66 and small.decode_slots == 198
    for M, N, K in shapes[:200]:
        swap, bn, ks = plan_gemm(M, N, K, small)
        if swap and ks > 1:
            assert ((N + 127) // 128) * ks <= (small.stream_ctas if M <= 16 else small.split_ctas)
        if not swap and ks > 1:
            assert ((M + 127) // 128) * ((N + bn - 1) // bn) * ks <= 66


def test_a_second_request_under_a_live_id_is_refused_and_the_queue_moves_on():
    m, s = make(pages=16, page=4, budget=16)
    a = req("a", 5)
    s.add(a)
    again = req("a", 3)
    s.add(again)                                 # while the first one waits
    assert again.finished == FinishReason.REFUSED
    run(m, s, s.plan())
    running_again = req("a", 3)
    s.add(running_again)                         # while the first one runs
    assert running_again.finished == FinishReason.REFUSED
    b = req("b", 4)
    s.add(b)
    while s.has_work():
        run(m, s, s.plan())
    assert a.finished == FinishReason.MAX_TOKENS and b.finished == FinishReason.MAX_TOKENS
    later = req("a", 3)                          # the id is free again once its request has ended
    s.add(later)
    assert later.finished is None
    while s.has_work():
        run(m, s, s.plan())
    assert later.finished == FinishReason.MAX_TOKENS and m.free_pages() == {0: 16}


def test_a_request_that_ended_while_it_waited_is_not_run_again():
    m, s = make(pages=6, page=4, budget=32)
    a, b = req("a", 10, max_new=20), req("b", 9, max_new=20)
    s.add(a)
    s.add(b)
    for _ in range(3):
        run(m, s, s.plan())
    p = s.plan()
    assert p.preempted == [b] and s.waiting[0] is b
    b.finished = FinishReason.MAX_TOKENS         # as a token accepted for the step planned ahead would end it
    run(m, s, p)
    while s.has_work():
        p = s.plan()
        assert all(e.request is not b for e in p.entries)
        run(m, s, p)
    assert b not in s.running and "b" not in m.requests and m.free_pages() == {0: 6}


def test_a_misuse_of_fork_does_not_cost_the_kept_caches():
    m, s, dev = make_kept(pages=12, page=4, reqs=4)
    s.add(Request("a", list(range(100, 108)), SamplingParams.greedy(), 1))
    drain(s, dev)
    assert len(s.kept) == 1
    s.add(Request("live", list(range(300, 305)), SamplingParams.greedy(), 6))
    dev.step(s, s.plan())
    live = s.running[0]
    with pytest.raises(ValueError):
        s.fork(live, Request("live", list(live.tokens), SamplingParams.greedy(), 2))   # the child's id is in use
    assert len(s.kept) == 1 and s.stats["prefix_evictions"] == 0
    drain(s, dev)


def test_a_plan_made_while_a_request_samples_its_last_token_leaves_it_out():
    """The entry point plans the next step while the GPU still runs the current one; a request whose
    token on its way is certainly its last is marked ``ending`` meanwhile: it gets no entry, keeps its
    pages and slot, and nothing else about the plan changes (steady decoding and the general planner)."""
    m, s = make(pages=32, budget=16)
    a, b, c = req("a", 3, max_new=2), req("b", 4, max_new=8), req("c", 20, max_new=8)
    s.add(a)
    s.add(b)
    run(m, s, s.plan())                                  # both prompts whole, one token each
    a.ending = True                                      # a's second token is its last
    p = s.plan()                                         # nobody waits: the steady-decode plan
    assert [(e.request.rid, e.count) for e in p.entries] == [("b", 1)]
    assert a in s.running and "a" in m.requests          # a keeps what it holds until its token is read
    s.add(c)
    p = s.plan()                                         # somebody waits: the general planner
    assert [(e.request.rid, e.start, e.count) for e in p.entries] == [("b", 4, 1), ("c", 0, 15)]
    a.ending = False
    m.check_invariants()
