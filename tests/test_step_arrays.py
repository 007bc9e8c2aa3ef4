"""The step's index arrays (CPU): tokens, positions, slots, block tables, wanted rows as `ModelRunner._fill` stages them
must be the same, byte for byte, with the cache manager in C++ (whose dense tables it reads in place) and with the one in
Python (whose lists it mirrors): decoded tokens alone (filled whole), prompt portions beside them (filled entry by entry),
padding rows of a captured graph, one group and two with a window that gives pages back.  The runner here is a stub that
has only what `_fill` touches; no device is needed."""
import random

import numpy as np
import pytest
import torch

from cppvllm_b200.cache.manager import CacheManager, GroupConfig
from cppvllm_b200.cache.native import NativeCacheManager
from cppvllm_b200.engine import runner as R


class _Event:
    def record(self):
        pass

    def synchronize(self):
        pass


class _Spec:                                 # what _fill reads of a group's cache spec
    def __init__(self, window):
        self.window = window

def make(native, groups, ps, slots, W, max_tokens, max_seqs):
    r = object.__new__(R.ModelRunner)
    r.page_size, r.max_step_tokens, r.max_seqs, r.table_width = ps, max_tokens, max_seqs, W
    r.group_specs = [(_Spec(g.window), [0]) for g in groups]
    r.cache = NativeCacheManager(groups, ps, slots, W) if native else CacheManager(groups, ps, slots)
    G = len(groups)
    cap = (5 * R._align(max_tokens) + 3 * R._align(max_seqs + 1) + G * (R._align(max_tokens) + R._align(max_seqs * W)) + 64)
    r._stage_capacity = cap
    r._stage_host = [torch.zeros(cap, dtype=torch.int32) for _ in range(4)]
    r._stage_np = [t.numpy() for t in r._stage_host]
    r._stage_events = [None] * 4
    r._stage_turn = 0
    r._stage_dev = torch.zeros(cap, dtype=torch.int32)
    r.scratch_slot, r.scratch_page = slots, groups[0].num_pages
    r.num_pages = groups[0].num_pages
    if native:
        r._tab_mirror = list(r.cache.tables)
    else:
        r._tab_mirror = [np.full((slots + 1, W), -1, dtype=np.int32) for _ in groups]
        r._mirror_owner = [[None] * (slots + 1) for _ in groups]
        r._mirror_len = [[0] * (slots + 1) for _ in groups]
    r._feed = None
    return r


@pytest.mark.parametrize("seed", range(4))
def test_index_arrays_are_the_same_with_either_cache_manager(seed, monkeypatch):
    monkeypatch.setattr(torch.cuda, "Event", _Event)
    assert torch.arange(10)[np.int32(3)].item() == 3          # a table entry of the C++ manager indexes a tensor
    rng = random.Random(seed)
    for trial in range(10):
        ps = rng.choice([4, 16])
        groups = [GroupConfig(60), GroupConfig(40, window=rng.choice([ps, 3 * ps + 1]))][: rng.choice([1, 2])]
        W = 12
        a, b = make(False, groups, ps, 6, W, 256, 6), make(True, groups, ps, 6, W, 256, 6)
        pos = {}
        for step in range(60):
            live = list(pos)
            if len(live) < 5 and rng.random() < 0.3:
                rid = f"r{trial}_{step}"
                for r in (a, b): r.cache.admit(rid)
                pos[rid] = 0
                live.append(rid)
            if not live: continue
            chosen = rng.sample(live, rng.randint(1, len(live)))
            entries = []
            decode = rng.random() < 0.5
            for rid in chosen:
                n = 1 if decode or pos[rid] > 0 and rng.random() < 0.5 else rng.randint(1, 3 * ps)
                if pos[rid] + n > W * ps: continue
                for r in (a, b): r.cache.reserve(rid, pos[rid] + n)
                toks = [rng.randint(0, 99) for _ in range(n)]
                want = [n - 1] if decode or rng.random() < 0.7 else []
                entries.append(R.StepEntry(rid, toks, pos[rid], want))
            if not entries: continue
            T = sum(len(e.tokens) for e in entries); S = len(entries); Rr = sum(len(e.want) for e in entries)
            pad = rng.choice([0, 0, 8]) if T == S and Rr == S else 0
            Wuse = W if pad else max(len(a.cache.lease(e.request_id).tables[g]) for e in entries for g in range(len(groups)))
            la = a._fill(entries, T, S, Rr, Wuse, pad_to=pad); lb = b._fill(entries, T, S, Rr, Wuse, pad_to=pad)
            assert la[1:] == lb[1:] and la[0] == lb[0]
            end = la[0]["_end"][0]
            ia, ib = (a._stage_turn - 1) % 4, (b._stage_turn - 1) % 4
            assert ia == ib
            # compare only the regions the layout names (gaps between aligned regions keep old bytes)
            for name, (o, n) in la[0].items():
                if name == "_end": continue
                x, y = a._stage_np[ia][o:o + n], b._stage_np[ib][o:o + n]
                if name == "feed_src": continue
                assert (x == y).all(), (trial, step, name, x, y)
            for r in (a, b):
                r._advance(entries)                          # the runner's own step end: one call into the C++ manager
            for e in entries:
                assert a.cache.lease(e.request_id).computed == b.cache.lease(e.request_id).computed == e.start + len(e.tokens)
                pos[e.request_id] = e.start + len(e.tokens)
            if rng.random() < 0.15:
                rid = rng.choice(list(pos))
                for r in (a, b): r.cache.release(rid)
                del pos[rid]
