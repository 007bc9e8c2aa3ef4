"""The cache manager in C++ against its plain twin in Python (CPU): the same calls in the same random orders must
give the same pages in the same tables, the same counts, the same answers and the same refusals."""
import random

import numpy as np
import pytest

from cppvllm_b200.cache.manager import CacheError, CacheManager, GroupConfig, OutOfPages
from cppvllm_b200.cache.native import NativeCacheManager


def pair(groups, page_size, slots, width, prefix=False):
    return (CacheManager(groups, page_size, slots, prefix_caching=prefix),
            NativeCacheManager(groups, page_size, slots, width, prefix_caching=prefix))


def same_state(py, nat):
    assert set(py.leases) == set(nat.leases)
    for g in range(len(py.groups)):
        assert py.num_free_pages(g) == nat.num_free_pages(g)
        for p in range(py.groups[g].num_pages):
            assert py.pools[g].refs(p) == nat.pools[g].refs(p)
    for rid, lease in py.leases.items():
        other = nat.lease(rid)
        assert lease.state_slot == other.state_slot and lease.computed == other.computed
        assert lease.registered == other.registered
        for g in range(len(py.groups)):
            assert list(lease.tables[g]) == [int(x) for x in other.tables[g]]
            # beyond its length a row of the dense array holds nothing
            row = nat.tables[g][other.state_slot]
            assert (row[len(lease.tables[g]):] == -1).all()
    assert py.prefix_hits == nat.prefix_hits
    py.check_invariants()
    nat.check_invariants()


def both(py, nat, name, *args):
    """Call the method on both; the same result or the same kind of refusal."""
    out = []
    for m in (py, nat):
        try:
            r = getattr(m, name)(*args)
            out.append(("ok", r if not hasattr(r, "state_slot") else r.state_slot))
        except (CacheError, OutOfPages, ValueError) as e:
            out.append((type(e).__name__, None))
    assert out[0] == out[1], (name, args, out)
    return out[0]


def test_the_first_steps_by_hand():
    py, nat = pair([GroupConfig(8)], 16, 4, 8)
    for m in (py, nat):
        m.admit("a")
        assert m.reserve("a", 33) == 48
        assert m.block_table("a", 0) == [0, 1, 2] and m.num_free_pages() == 5
        assert m.slots_for("a", 0, 15, 3) == [15, 16, 17]
        m.admit("b")
        with pytest.raises(OutOfPages):
            m.reserve("b", 16 * 6)
        assert m.block_table("b", 0) == [] and m.num_free_pages() == 5
        m.reserve("b", 16 * 5)
        assert not m.can_reserve("a", 49) and m.covered("a", 48) and not m.covered("a", 49)
        m.release("a")
        m.admit("c")
        m.reserve("c", 17)
        assert m.block_table("c", 0) == [2, 1]               # least recently freed first, a's last page first
        with pytest.raises(CacheError):
            m.release("a")
        with pytest.raises(CacheError):
            m.admit("c")
        with pytest.raises(CacheError):
            m.advance("c", 5) or m.advance("c", 3)
        assert m.take_fresh_slots() == [1, 0] and m.take_fresh_slots() == []
    same_state(py, nat)
    with pytest.raises(OutOfPages):
        nat.reserve("c", 16 * 9)                             # more than the pool has: refused as the twin refuses it
    wide = NativeCacheManager([GroupConfig(20)], 16, 2, 4)
    wide.admit("w")
    with pytest.raises(ValueError):
        wide.reserve("w", 16 * 5)                            # the pool has the pages, the dense table has no column for them
    assert wide.num_free_pages() == 20 and wide.block_table("w", 0) == []
    with pytest.raises(ValueError):
        NativeCacheManager([GroupConfig(8), GroupConfig(8, window=32)], 16, 4, 8, prefix_caching=True)


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_give_the_same_tables(seed):
    rng = random.Random(seed)
    ps = rng.choice([4, 16, 32])
    groups = [GroupConfig(rng.randint(12, 40)), GroupConfig(rng.randint(8, 30), window=rng.choice([ps, 3 * ps + 1, 5 * ps]))]
    if seed % 3 == 0:
        groups = groups[:1]
    width = 24
    py, nat = pair(groups, ps, 5, width)
    length = {}
    for step in range(600):
        op = rng.random()
        live = list(length)
        if op < 0.2:
            rid = f"r{step}"
            if both(py, nat, "admit", rid)[0] == "ok":
                length[rid] = 0
        elif op < 0.65 and live:
            rid = rng.choice(live)
            upto = min(length[rid] + rng.randint(1, 3 * ps), width * ps)
            assert py.can_reserve(rid, upto) == nat.can_reserve(rid, upto)
            assert py.pages_missing(rid, upto) == nat.pages_missing(rid, upto)
            if both(py, nat, "reserve", rid, upto)[0] == "ok":
                assert py.covered(rid, upto) and nat.covered(rid, upto)
                both(py, nat, "advance", rid, upto)          # the tokens are computed: windows give pages back
                length[rid] = upto
        elif op < 0.8 and live:
            rid = rng.choice(live)
            both(py, nat, "release", rid)
            del length[rid]
        elif op < 0.9:
            both(py, nat, "release", f"nobody{step}")        # misuse is refused by both
            if live:
                both(py, nat, "advance", live[0], max(0, length[live[0]] - 1) if length[live[0]] else 0)
        else:
            assert py.take_fresh_slots() == nat.take_fresh_slots()
        if step % 20 == 0:
            same_state(py, nat)
    same_state(py, nat)
    for rid in list(length):
        both(py, nat, "release", rid)
    same_state(py, nat)
    assert all(nat.num_free_pages(g) == groups[g].num_pages for g in range(len(groups)))
    for g in range(len(groups)):
        assert (nat.tables[g] == -1).all()


@pytest.mark.parametrize("seed", range(6))
def test_prefix_cache_under_random_orders_gives_the_same_sharing(seed):
    rng = random.Random(100 + seed)
    ps = rng.choice([4, 8])
    py, nat = pair([GroupConfig(rng.randint(16, 40))], ps, 6, 32, prefix=True)
    stems = [[rng.randint(0, 50) for _ in range(rng.randint(2 * ps, 6 * ps))] for _ in range(3)]
    toks, done = {}, {}
    for step in range(500):
        op = rng.random()
        live = list(toks)
        if op < 0.3:
            rid = f"r{step}"
            t = list(rng.choice(stems))[:rng.randint(ps, 6 * ps)] + [rng.randint(0, 50) for _ in range(rng.randint(1, 2 * ps))]
            assert py.can_admit(t, len(t)) == nat.can_admit(t, len(t))
            if py.can_admit(t, len(t)):
                a = both(py, nat, "admit", rid, t)
                if a[0] == "ok":
                    assert py.lease(rid).computed == nat.lease(rid).computed
                    both(py, nat, "reserve", rid, len(t))
                    toks[rid], done[rid] = t, py.lease(rid).computed
        elif op < 0.7 and live:
            rid = rng.choice(live)
            t = toks[rid]
            if done[rid] < len(t):                           # a portion of the prompt is computed
                done[rid] = min(len(t), done[rid] + rng.randint(1, 2 * ps))
            elif len(t) < 30 * ps:                           # a decoded token, sometimes not yet known on the host
                t.append(rng.randint(0, 50))
                if both(py, nat, "reserve", rid, len(t))[0] != "ok":
                    t.pop()
                    continue
                done[rid] = len(t)
            both(py, nat, "advance", rid, done[rid])
            known = list(t)
            if rng.random() < 0.3:
                known[-1] = -1
            both(py, nat, "commit", rid, known)
        elif op < 0.9 and live:
            rid = rng.choice(live)
            both(py, nat, "commit", rid, toks[rid])
            both(py, nat, "release", rid)
            del toks[rid], done[rid]
        if step % 25 == 0:
            same_state(py, nat)
    same_state(py, nat)
    assert py.prefix_hits > 0                                 # the stems were shared at all


def test_advance_many_is_advance_for_each():
    py, nat = pair([GroupConfig(30), GroupConfig(20, window=9)], 4, 4, 16)
    for rid, n in (("a", 30), ("b", 11), ("c", 4)):
        for m in (py, nat):
            m.admit(rid)
            m.reserve(rid, n)
    for rid, n in (("a", 30), ("b", 11), ("c", 4)):
        py.advance(rid, n)
    nat.advance_many(["a", "b", "c"], [30, 11, 4])
    same_state(py, nat)
    with pytest.raises(CacheError):
        nat.advance_many(["a", "b"], [30, 5])                 # b would shrink; a's call before it stands
    with pytest.raises(CacheError):
        nat.advance_many(["nobody"], [1])
    same_state(py, nat)


def test_tables_are_read_in_place():
    """The dense arrays belong to the library and follow every call without being fetched again."""
    nat = NativeCacheManager([GroupConfig(10)], 8, 3, 6)
    tab = nat.tables[0]
    nat.admit("x")
    nat.reserve("x", 20)
    assert tab[0].tolist() == [0, 1, 2, -1, -1, -1] and isinstance(tab, np.ndarray) and tab.dtype == np.int32
    nat.release("x")
    assert (tab == -1).all()
