"""The cache manager's bookkeeping (CPU): no page lost, held twice or freed twice, under random orders."""
import random

import pytest

from cppvllm_b200.cache.manager import CacheError, CacheManager, GroupConfig, OutOfPages


def test_reserve_release_reuse():
    m = CacheManager([GroupConfig(8)], page_size=16, num_state_slots=4)
    m.admit("a")
    m.reserve("a", 33)
    assert m.block_table("a", 0) == [0, 1, 2] and m.num_free_pages() == 5
    assert m.slots_for("a", 0, 15, 3) == [15, 16, 17]
    m.reserve("a", 33)                                      # idempotent
    assert m.num_free_pages() == 5
    m.admit("b")
    with pytest.raises(OutOfPages):
        m.reserve("b", 16 * 6)                               # all or nothing
    assert m.block_table("b", 0) == [] and m.num_free_pages() == 5
    m.reserve("b", 16 * 5)
    assert m.num_free_pages() == 0 and not m.can_reserve("a", 49)
    m.release("a")
    m.check_invariants()
    # least recently freed first; a's pages were given back last page first
    m.admit("c")
    m.reserve("c", 17)
    assert m.block_table("c", 0) == [2, 1]
    m.check_invariants()


def test_misuse_is_refused():
    m = CacheManager([GroupConfig(4)], 16, 2)
    m.admit(1)
    with pytest.raises(CacheError, match="already admitted"):
        m.admit(1)
    with pytest.raises(CacheError, match="not admitted"):
        m.reserve(2, 5)
    m.release(1)
    with pytest.raises(CacheError, match="not admitted"):
        m.release(1)
    with pytest.raises(CacheError):
        m.pools[0].give_back(0)                              # double free
    m.admit(1); m.admit(2)
    with pytest.raises(CacheError, match="no free state slot"):
        m.admit(3)
    m.reserve(1, 10)
    with pytest.raises(CacheError, match="no page"):
        m.slots_for(1, 0, 16, 1)
    with pytest.raises(CacheError, match="shrink"):
        m.advance(1, 5) or m.advance(1, 3)


def test_state_slots_are_fresh_once():
    m = CacheManager([GroupConfig(4)], 16, 3)
    a = m.admit("a").state_slot
    b = m.admit("b").state_slot
    assert {a, b} == {0, 1} and sorted(m.take_fresh_slots()) == [0, 1] and m.take_fresh_slots() == []
    m.release("a")
    assert m.admit("c").state_slot == a and m.take_fresh_slots() == [a]


def test_window_group_gives_pages_back_as_the_window_passes():
    # group 0 keeps everything, group 1 only looks back 20 positions; page 16
    m = CacheManager([GroupConfig(16), GroupConfig(16, window=20)], 16, 2)
    m.admit("a")
    m.reserve("a", 40)
    assert m.block_table("a", 1) == [0, 1, 2]
    m.advance("a", 40)            # next token at 40 reads 21..40 -> page 0 (positions 0..15) is passed
    assert m.block_table("a", 1) == [-1, 1, 2] and m.block_table("a", 0) == [0, 1, 2]
    assert m.num_free_pages(1) == 14 and m.num_free_pages(0) == 13
    m.reserve("a", 41)
    m.advance("a", 41)
    m.reserve("a", 100)           # a long portion: pages for 41..99; positions 22.. are still needed
    assert m.block_table("a", 1)[:3] == [-1, 1, 2]
    m.advance("a", 100)           # next reads 81..100 -> pages 0..4 passed
    assert m.block_table("a", 1)[:5] == [-1] * 5 and all(p >= 0 for p in m.block_table("a", 1)[5:])
    m.check_invariants()
    # a request admitted late never takes pages for positions the window has passed
    m.admit("b")
    m.leases["b"].computed = 64
    m.reserve("b", 70)
    assert m.block_table("b", 1)[:2] == [-1, -1] and m.block_table("b", 1)[2] >= 0
    m.release("a"); m.release("b")
    m.check_invariants()
    assert m.num_free_pages(0) == 16 and m.num_free_pages(1) == 16


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    windows = [0, 24] if seed % 2 else [0]
    m = CacheManager([GroupConfig(24, w) for w in windows], 8, 5)
    live = {}
    nxt = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            m.admit(nxt)
            live[nxt] = 0
            nxt += 1
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 13, 30])
            if m.can_reserve(rid, live[rid] + n):
                m.reserve(rid, live[rid] + n)
                m.slots_for(rid, 0, live[rid], n)            # every token of the step has a page
                live[rid] += n
                m.advance(rid, live[rid])
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, live[rid] + n)
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        for g, w in enumerate(windows):                      # what the next token reads is held
            for rid, n in live.items():
                lo = max(0, n - w + 1) if w else 0
                tab = m.block_table(rid, g)
                assert all(tab[i] >= 0 for i in range(lo // 8, len(tab)))
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert all(p.num_free == p.num_pages for p in m.pools) and m.slots.num_free == 5


def test_prefix_cache_shares_registered_pages_and_forgets_reused_ones():
    m = CacheManager([GroupConfig(6)], 4, 4, prefix_caching=True)
    toks = list(range(100, 111))                               # 11 tokens: two full pages and a partial one
    a = m.admit("a", toks)
    assert a.computed == 0
    m.reserve("a", len(toks))
    m.advance("a", 11)
    m.commit("a", toks)
    assert a.registered == 2
    b = m.admit("b", toks[:8] + [1, 2])                         # same first two pages
    assert b.computed == 8 and b.tables[0] == a.tables[0][:2]
    assert [m.pools[0].refs(p) for p in a.tables[0]] == [2, 2, 1]
    m.reserve("b", 10)
    m.check_invariants()
    m.release("a")
    assert [m.pools[0].refs(p) for p in b.tables[0]] == [1, 1, 1]
    m.check_invariants()
    m.release("b")
    assert m.num_free_pages() == 6
    # the pages keep their keys while they are free: a third request finds them again, taking them off the free list
    assert m.can_admit(toks, 11)
    c = m.admit("c", toks)
    assert c.computed == 8 and m.num_free_pages() == 4
    m.release("c")
    # fresh contents for all six pages: the keys are forgotten
    m.admit("d")
    m.reserve("d", 24)
    assert m.admit("e", toks).computed == 0
    m.release("d")
    m.release("e")
    m.check_invariants()
    # tokens that are not known yet (negative placeholders) are never registered or looked up
    f = m.admit("f", [5, 6, 7, 8, -1])
    m.reserve("f", 5)
    m.advance("f", 5)
    m.commit("f", [5, 6, 7, 8, -1])
    assert f.registered == 1
    g = m.admit("g", [5, 6, 7, -1, 9])
    assert g.computed == 0
    with pytest.raises(ValueError):
        CacheManager([GroupConfig(4), GroupConfig(4, window=8)], 4, 2, prefix_caching=True)


def test_prefix_cache_under_random_orders():
    """Random admissions with shared prefixes, growth, commits and releases: reference counts and the free list stay
    consistent, and a request never gets a page whose registered tokens differ from its own."""
    rng = random.Random(7)
    m = CacheManager([GroupConfig(40)], 4, 16, prefix_caching=True)
    stems = [[rng.randrange(50) for _ in range(24)] for _ in range(3)]
    live = {}
    for step in range(600):
        if live and rng.random() < 0.35:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        elif len(live) < 10:
            stem = rng.choice(stems)
            toks = stem[:rng.randrange(1, 25)] + [rng.randrange(50, 60) for _ in range(rng.randrange(0, 6))]
            if m.can_admit(toks, len(toks)):
                lease = m.admit(step, toks)
                assert lease.computed % 4 == 0 and lease.computed < len(toks)
                for i, p in enumerate(lease.tables[0]):
                    assert m.pools[0]._tokens[p] == tuple(toks[4 * i:4 * i + 4])
                m.reserve(step, len(toks))
                m.advance(step, len(toks))
                m.commit(step, toks)
                live[step] = toks
        m.check_invariants()
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert m.num_free_pages() == 40 and m.prefix_hits > 0
