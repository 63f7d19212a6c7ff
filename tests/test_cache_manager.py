"""The cache manager without a GPU: no page lost, held twice or freed twice, under
random orders of requests; groups with a window give pages back; state slots."""
import random

import pytest
import torch

from airun_b200.cache import CacheError, CacheManager, CacheStorage, OutOfPages, PageAllocator
from airun_b200.parts.base import PagedKVSpec, StateSpec

FULL = PagedKVSpec(2, 16, 0)
WIN = PagedKVSpec(2, 16, 24)


def manager(specs=(FULL, FULL), cache_from=None, page=8, pages=12, reqs=4):
    return CacheManager(list(specs), list(cache_from or [None] * len(specs)), page, pages, reqs)


def test_allocator_hands_out_a_freed_page_next():
    a = PageAllocator(4)
    p = a.take(3)
    assert p == [0, 1, 2] and a.num_free == 1
    a.give_back(1)
    assert a.take(1) == [1]
    with pytest.raises(OutOfPages):
        a.take(2)
    a.give_back(0)
    with pytest.raises(CacheError):
        a.give_back(0)                       # freed twice
    with pytest.raises(CacheError):
        a.give_back(9)


def test_groups_by_equal_spec_and_sharing_entries():
    m = manager([FULL, WIN, FULL, WIN, None, StateSpec((3, 5))], [None] * 6)
    assert [g.spec for g in m.paged] == [FULL, WIN]
    assert m.paged[0].owners == [0, 2] and m.paged[1].owners == [1, 3]
    assert m.bindings[2].gid == 0 and m.bindings[2].index == 1
    assert m.bindings[4].kind == "none" and m.bindings[5].kind == "state"
    m2 = manager([FULL, FULL, FULL], [None, None, 0])
    assert m2.bindings[2].shared and m2.bindings[2].index == 0 and m2.paged[0].owners == [0, 1]
    with pytest.raises(ValueError):
        manager([FULL, WIN], [None, 0])      # cannot read a cache of another shape
    with pytest.raises(ValueError):
        manager([FULL, FULL, FULL], [None, 0, 1])   # must read an owner


def test_pages_follow_the_tokens():
    m = manager(page=8, pages=6)
    m.add_request("a")
    assert m.pages_needed("a", 9) == {0: 2}
    m.reserve("a", 9)
    m.commit("a", 9)
    assert m.block_table("a", 0) == [0, 1]
    m.reserve("a", 7)                        # tokens 9..15 fit the second page
    assert m.block_table("a", 0) == [0, 1]
    m.commit("a", 7)
    m.reserve("a", 1)
    assert m.block_table("a", 0) == [0, 1, 2]
    with pytest.raises(CacheError):
        m.commit("a", 9)                     # beyond what was reserved
    m.commit("a", 1)
    m.add_request("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 8 * 4)                # only 3 pages are free; nothing is taken
    assert m.free_pages() == {0: 3} and m.block_table("b", 0) == []
    m.free_request("a")
    assert m.free_pages() == {0: 6}
    with pytest.raises(CacheError):
        m.free_request("a")
    m.check_invariants()


def test_window_group_gives_pages_back_as_the_window_passes():
    m = manager([FULL, WIN], page=8, pages=16)
    m.add_request("a")
    m.reserve("a", 40)
    assert m.free_pages() == {0: 11, 1: 11}
    m.commit("a", 40)
    # the next query sits at 40 and sees keys 17..40: blocks 0 and 1 (keys 0..15) are behind the window
    assert m.block_table("a", 1)[:2] == [-1, -1] and m.block_table("a", 1)[2] >= 0
    assert m.free_pages() == {0: 11, 1: 13}
    for _ in range(30):
        m.reserve("a", 1)
        m.commit("a", 1)
    live = [p for p in m.block_table("a", 1) if p >= 0]
    assert len(live) <= 24 // 8 + 2           # never more than the window needs
    assert all(p >= 0 for p in m.block_table("a", 0))
    m.check_invariants()
    m.free_request("a")
    assert m.free_pages() == {0: 16, 1: 16}


def test_window_edge_is_exact():
    """A page is given back only when its LAST key is behind the window of the next query."""
    m = manager([WIN], page=8, pages=8)
    m.add_request("a")
    m.reserve("a", 31)
    m.commit("a", 31)                         # next query at 31 sees keys 8..31: key 7 is dead, block 0 goes
    assert m.block_table("a", 0)[0] == -1
    m2 = manager([WIN], page=8, pages=8)
    m2.add_request("a")
    m2.reserve("a", 30)
    m2.commit("a", 30)                        # next query at 30 sees keys 7..30: block 0 still holds key 7
    assert m2.block_table("a", 0)[0] >= 0


def test_state_slots():
    m = manager([StateSpec((4,)), FULL], page=8, pages=4, reqs=2)
    a = m.add_request("a")
    b = m.add_request("b")
    assert {a.slot, b.slot} == {0, 1}
    assert not m.has_free_slot()
    with pytest.raises(CacheError):
        m.add_request("c")
    with pytest.raises(CacheError):
        m.add_request("a")
    m.free_request("a")
    assert m.add_request("c").slot == a.slot
    st = CacheStorage(m, torch.float32, "cpu")
    assert st.state[0].shape == (1, 2, 4) and st.paged[0].shape == (1, 4, 2, 2, 8, 16)
    st.state[0].fill_(3.0)
    st.zero_state_slot(1)
    assert float(st.state[0][0, 1].abs().sum()) == 0 and float(st.state[0][0, 0].sum()) == 12


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    m = manager([FULL, WIN, FULL], page=4, pages=40, reqs=6)
    live = {}
    next_id = 0
    for step in range(600):
        r = rng.random()
        if r < 0.25 and m.has_free_slot():
            m.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif r < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 13])
            if m.can_reserve(rid, n):
                m.reserve(rid, n)
                m.commit(rid, n)
                live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
        elif live:
            rid = rng.choice(list(live))
            m.free_request(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            assert m.get(rid).num_tokens == n
            full = m.block_table(rid, 0)
            assert len(full) == (n + 3) // 4 and all(p >= 0 for p in full)
            # every key the next query can see in the window group still has its page
            win = m.block_table(rid, 1)
            for j in range(max(0, n - 24 + 1), n):
                assert win[j // 4] >= 0
    for rid in list(live):
        m.free_request(rid)
    assert m.free_pages() == {0: 40, 1: 40}
    m.check_invariants()


def test_fork_shares_whole_pages_and_copies_the_partial_one():
    m = manager([FULL], page=8, pages=6)
    m.add_request("a")
    m.reserve("a", 19)
    m.commit("a", 19)                         # pages 0, 1 whole, page 2 holds 3 tokens
    plan = m.fork("a", "b")
    assert m.block_table("b", 0)[:2] == [0, 1] and m.block_table("b", 0)[2] == 3
    assert plan.pages == [(0, 2, 3)] and plan.state is None
    assert m.paged[0].allocator.holders(0) == 2 and m.paged[0].allocator.holders(2) == 1
    assert m.get("b").num_tokens == 19
    m.check_invariants()
    m.free_request("a")                       # the shared pages stay with b
    assert m.free_pages() == {0: 3}
    m.reserve("b", 6)
    m.commit("b", 6)
    m.check_invariants()
    m.free_request("b")
    assert m.free_pages() == {0: 6}
    # at a page's edge nothing is copied
    m.add_request("c")
    m.reserve("c", 16)
    m.commit("c", 16)
    assert m.fork("c", "d").pages == []
    # short of pages or slots: nothing is taken
    m2 = manager([FULL], page=8, pages=1, reqs=2)
    m2.add_request("a")
    m2.reserve("a", 3)
    m2.commit("a", 3)
    with pytest.raises(OutOfPages):
        m2.fork("a", "b")
    assert "b" not in m2.requests and m2.has_free_slot()
    m2.check_invariants()


def test_truncate_gives_pages_back_and_never_writes_a_shared_page():
    m = manager([FULL], page=8, pages=8)
    m.add_request("a")
    m.reserve("a", 30)
    m.commit("a", 30)
    assert m.truncate("a", 30).pages == []
    m.fork("a", "b")                          # pages 0..2 shared, page 3 copied
    plan = m.truncate("b", 12)                # the end falls inside shared page 1
    assert len(m.block_table("b", 0)) == 2 and m.block_table("b", 0)[0] == 0
    assert plan.pages and plan.pages[0][1] == 1 and plan.pages[0][2] == m.block_table("b", 0)[1] != 1
    assert m.paged[0].allocator.holders(1) == 1 and m.paged[0].allocator.holders(2) == 1
    m.check_invariants()
    assert m.truncate("a", 16).pages == []    # at a page's edge: pages 2 and 3 go back
    assert len(m.block_table("a", 0)) == 2
    with pytest.raises(CacheError):
        m.truncate("a", 17)
    m.check_invariants()
    ms = manager([StateSpec((4,)), FULL], page=8, pages=4)
    ms.add_request("a")
    ms.reserve("a", 5)
    ms.commit("a", 5)
    assert ms.fork("a", "b").state == (ms.get("a").slot, ms.get("b").slot)
    with pytest.raises(CacheError):
        ms.truncate("a", 2)                   # fixed-size state cannot be moved back
    mw = manager([WIN], page=8, pages=8)
    mw.add_request("a")
    mw.reserve("a", 60)
    mw.commit("a", 60)
    with pytest.raises(CacheError):
        mw.truncate("a", 20)                  # the window's pages before 20 are gone
    assert mw.truncate("a", 58).pages == []


@pytest.mark.parametrize("seed", range(6))
def test_random_forks_and_cuts_every_request_reads_its_own_history(seed):
    """Pages carry what was written to them (a shadow of the device); through its block table
    every request must find its own tokens, whatever was shared, copied, cut or freed."""
    rng = random.Random(100 + seed)
    P = 4
    m = manager([FULL, WIN], page=P, pages=48, reqs=6)
    content = [[[None] * P for _ in range(48)] for _ in m.paged]
    history = {}
    next_id, stamp = 0, 0

    def write(rid, start, values):
        for g in m.paged:
            bt = m.block_table(rid, g.gid)
            for i, v in enumerate(values):
                pos = start + i
                assert m.paged[g.gid].allocator.holders(bt[pos // P]) == 1, "a shared page is written"
                content[g.gid][bt[pos // P]][pos % P] = v

    def run(plan):
        for gid, src, dst in plan.pages:
            content[gid][dst] = list(content[gid][src])

    for step in range(500):
        r = rng.random()
        if r < 0.15 and m.has_free_slot():
            m.add_request(next_id)
            history[next_id] = []
            next_id += 1
        elif r < 0.65 and history:
            rid = rng.choice(list(history))
            n = rng.choice([1, 1, 2, 3, 7])
            if m.can_reserve(rid, n):
                m.reserve(rid, n)
                vals = list(range(stamp, stamp + n))
                stamp += n
                write(rid, len(history[rid]), vals)
                m.commit(rid, n)
                history[rid] += vals
        elif r < 0.78 and history and m.has_free_slot():
            rid = rng.choice(list(history))
            try:
                run(m.fork(rid, next_id))
                history[next_id] = list(history[rid])
                next_id += 1
            except OutOfPages:
                pass
        elif r < 0.88 and history:
            rid = rng.choice(list(history))
            n = rng.randint(max(0, len(history[rid]) - 6), len(history[rid]))
            try:
                run(m.truncate(rid, n))
                del history[rid][n:]
            except (OutOfPages, CacheError):
                pass
        elif history:
            rid = rng.choice(list(history))
            m.free_request(rid)
            del history[rid]
        m.check_invariants()
        for rid, h in history.items():
            assert m.get(rid).num_tokens == len(h)
            for g in m.paged:
                bt = m.block_table(rid, g.gid)
                lo = 0 if g.window == 0 else max(0, len(h) - g.window + 1)
                for pos in range(lo, len(h)):
                    assert content[g.gid][bt[pos // P]][pos % P] == h[pos], (rid, g.gid, pos)
    for rid in list(history):
        m.free_request(rid)
    assert m.free_pages() == {0: 48, 1: 48}


def test_rename_keeps_slot_tokens_and_pages_and_refuses_a_live_name():
    m = manager()
    a = m.add_request("a")
    m.reserve("a", 11)
    m.commit("a", 11)
    blocks, slot = m.block_table("a", 0), a.slot
    m.add_request("b")
    with pytest.raises(CacheError):
        m.rename("a", "b")                   # "b" is live
    with pytest.raises(CacheError):
        m.rename("nobody", "x")
    m.rename("a", ("kept", 0))
    assert "a" not in m.requests and m.get(("kept", 0)).slot == slot and m.get(("kept", 0)).rid == ("kept", 0)
    assert m.get(("kept", 0)).num_tokens == 11 and m.block_table(("kept", 0), 0) == blocks
    m.add_request("a")                       # the old name is free for a new request
    m.check_invariants()
    m.free_request(("kept", 0))
    m.free_request("a")
    m.free_request("b")
    assert m.free_pages() == {0: 12}


def test_can_rewind_only_without_windows_and_state():
    assert manager([FULL, FULL]).can_rewind
    assert not manager([FULL, WIN]).can_rewind
    assert not manager([FULL, StateSpec((3,))]).can_rewind


@pytest.mark.parametrize("seed", [0, 1, 2, 3])
def test_batch_layout_of_random_steps(seed):
    """The native core lays a step's batch into the staging buffer (tokens, positions, owner of every
    row, wanted rows, row offsets, context lengths, slots, one block table per group, the shared
    prefix); every word is checked against the plain meaning of the batch, with and without padding."""
    import ctypes
    import numpy as np
    rnd = random.Random(seed)
    page, R_max, T_max, pages = 4, 6, 64, 60
    m = CacheManager([FULL, WIN, FULL], [None, None, None], page, pages, R_max, max_blocks=24)
    n_groups = len(m.paged)
    sizes = [T_max, T_max, T_max, T_max, R_max + 1, R_max, R_max] + [R_max * m.max_blocks] * n_groups + [1] * n_groups
    offs, total = [], 0
    for n in sizes:
        offs.append(total)
        total += (n + 63) // 64 * 64
    buf = np.full(total, -777, dtype=np.int32)
    c_offs = (ctypes.c_longlong * len(offs))(*offs)
    held = {}                                               # rid -> tokens so far
    for step in range(60):
        # a few requests come, go, or are forked; then a batch of some of the live ones
        if len(held) < R_max and (not held or rnd.random() < 0.4):
            rid = ("r", step)
            m.add_request(rid)
            held[rid] = 0
        if held and rnd.random() < 0.15:
            rid = rnd.choice(list(held))
            m.free_request(rid)
            del held[rid]
            continue
        forked = None
        if held and len(held) < R_max and rnd.random() < 0.3:
            par = rnd.choice(list(held))
            try:
                m.fork(par, ("f", step))
                held[("f", step)] = held[par]
                forked = [par, ("f", step)]
            except OutOfPages:
                pass
        rids = forked if forked and rnd.random() < 0.7 else rnd.sample(list(held), rnd.randrange(1, len(held) + 1))
        decode = rnd.random() < 0.5 or rids is forked
        qlens = [1 if decode else rnd.randrange(1, 9) for _ in rids]
        qlens = [min(q, 90 - held[r]) for q, r in zip(qlens, rids)]
        rids, qlens = [r for r, q in zip(rids, qlens) if q > 0], [q for q in qlens if q > 0]
        if not rids or sum(qlens) > T_max:
            continue
        try:
            m.reserve_many(rids, qlens)
        except OutOfPages:
            continue
        toks = np.array([rnd.randrange(1000) for _ in range(sum(qlens))], dtype=np.int32)
        wants = [sorted(rnd.sample(range(q), rnd.randrange(0, q + 1))) for q in qlens]
        pad_to = rnd.choice([0, 0, T_max]) if sum(qlens) <= T_max else 0
        n_want = sum(len(w) for w in wants)
        pad_want = n_want + rnd.randrange(0, 3) if pad_to else 0
        buf[:] = -777
        t, nw, max_ctx, max_q, slots, shared = m.build_batch(
            rids, qlens, toks, [len(w) for w in wants], [x for w in wants for x in w], buf.ctypes.data, c_offs,
            R_max, m.max_blocks, pad_to, pad_want)
        T = sum(qlens)
        assert (t, nw, max_q) == (T, n_want, max(qlens)) and max_ctx == max(held[r] + q for r, q in zip(rids, qlens))
        assert slots == [m.get(r).slot for r in rids]
        tok, pos, owner, wr, cu, cl, sl = (buf[o:o + n] for o, n in zip(offs[:7], sizes[:7]))
        assert tok[:T].tolist() == toks.tolist()
        row = 0
        for i, (r, q) in enumerate(zip(rids, qlens)):
            assert cu[i] == row and cl[i] == held[r] + q and sl[i] == slots[i]
            assert pos[row:row + q].tolist() == list(range(held[r], held[r] + q)) and set(owner[row:row + q]) == {i}
            row += q
        assert cu[len(rids)] == T
        assert wr[:n_want].tolist() == [c + x for c, w in zip(np.cumsum([0] + qlens[:-1]).tolist(), wants) for x in w]
        if pad_to:
            assert set(pos[T:pad_to].tolist()) <= {-1} and set(owner[T:pad_to].tolist()) <= {-1}
            assert set(cu[len(rids):R_max + 1].tolist()) == {T} and set(wr[n_want:pad_want].tolist()) <= {0}
        for g in m.paged:
            bt = buf[offs[7 + g.gid]:offs[7 + g.gid] + R_max * m.max_blocks].reshape(R_max, m.max_blocks)
            for i, (r, q) in enumerate(zip(rids, qlens)):
                blocks = m.block_table(r, g.gid)
                need = -(-(held[r] + q) // page)
                assert bt[i, :need].tolist() == blocks[:need]
                first_key = max(0, held[r] + q - 1 - (g.window - 1)) if g.window else 0     # oldest key the newest token sees
                assert all(b >= 0 for b in blocks[first_key // page:need])
            # the shared prefix: whole pages at the start that every request of a decode batch holds alike
            want_shared = 0
            if len(rids) >= 2 and max(qlens) == 1 and g.window == 0:
                tables = [m.block_table(r, g.gid) for r in rids]
                limit = min(held[r] // page for r in rids)
                while want_shared < limit and len({tb[want_shared] for tb in tables}) == 1:
                    want_shared += 1
                want_shared *= page
            assert shared[g.gid] == want_shared == buf[offs[7 + n_groups + g.gid]]
        m.commit_many(rids, qlens)
        for r, q in zip(rids, qlens):
            held[r] += q
        m.check_invariants()


def test_fixed_size_state_is_taken_off_the_memory_the_pages_get(monkeypatch):
    """The cache size worked out from free memory leaves room for the state slots of every request."""
    import torch
    from airun_b200.engine.engine import Engine, EngineOptions
    from airun_b200.parts.base import PagedKVSpec, StateSpec
    monkeypatch.setattr(torch.cuda, "mem_get_info", lambda dev=None: (1 << 30, 1 << 31))
    o = EngineOptions(dtype="bfloat16", memory_fraction=0.5, max_requests=16, page_size=16)
    kv = PagedKVSpec(2, 64, 0)
    per_token = 2 * 2 * 64 * 2
    plain = Engine._tokens_that_fit([kv], [None], o)
    assert plain == (1 << 29) // per_token
    state = StateSpec((1024, 256), torch.float32)                      # 1 MiB per request and owner layer
    with_state = Engine._tokens_that_fit([kv, state, state], [None, None, 1], o)     # the second reads the first's
    assert with_state == ((1 << 29) - 16 * (1 << 20)) // per_token
