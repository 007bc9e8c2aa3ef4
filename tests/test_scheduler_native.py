"""The scheduler in C++ against its plain twin in Python (CPU): the same requests through the same engine loop (steps in
flight, tokens that travel on the device, preemption when pages run out, the prefix cache, end-of-sequence tokens) must
give the same batches, the same tokens to feed, the same preemptions and the same results; and the batches of the
reference's own scheduler (tests/golden) come out of it too."""
import json
import os
import random

import pytest

from cppvllm_b200.cache.manager import CacheManager, GroupConfig
from cppvllm_b200.cache.native import NativeCacheManager
from cppvllm_b200.engine.native_scheduler import NativeScheduler
from cppvllm_b200.engine.scheduler import FINISHED, PENDING, Scheduler, SchedulerConfig, Sequence
from cppvllm_b200.sampling.params import SamplingParams

from test_cache_native import same_state

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "scheduler_golden.json")
EOS = 13


def sample(rid: int, pos: int) -> int:
    """What the 'model' samples for request `rid` at position `pos`: any function of the two."""
    return (rid * 31 + pos * 7 + (pos * pos) % 11) % 50


def groups_of(blocks, window):
    """One group that keeps all keys; with a window, a second, smaller one that gives pages back as the window passes."""
    return [GroupConfig(blocks)] + ([GroupConfig(max(4, blocks // 2), window=window)] if window else [])


class PythonLoop:
    """The engine's loop (engine/llm_engine.py: step, _retire_oldest) around the scheduler in Python."""

    def __init__(self, cfg, blocks, page, slots, prefix, depth, window=0):
        self.cache = CacheManager(groups_of(blocks, window), page, slots, prefix_caching=prefix)
        self.sched = Scheduler(cfg, self.cache)
        self.depth, self.inflight, self.results, self.seqs = depth, [], {}, {}

    def add(self, rid, prompt, sp):
        s = Sequence(rid, prompt, sp)
        self.sched.add_request(s)
        self.seqs[rid] = s

    def finished(self):
        return not self.inflight and self.sched.is_finished()

    def retire(self):
        rec = self.inflight.pop(0)
        toks = [sample(s.seq_id, p) for s, f, p in zip(rec["batch"].seqs, rec["flags"], rec["batch"].sample_pos) if f]
        for s in self.sched.postprocess(rec["batch"], rec["flags"], toks):
            self.results[s.seq_id] = (list(s.token_ids), s.stopped_on_eos)

    def step(self):
        if self.sched.is_finished():
            while self.inflight:
                self.retire()
            return None
        b = self.sched.schedule(allow_preempt=not self.inflight)
        if not b.seqs:
            while self.inflight:
                self.retire()
            return ("empty", [s.seq_id for s in b.preempted], b.blocked)
        prev = self.inflight[-1] if self.inflight else None
        rows = []
        for s in b.seqs:
            c, n = s.num_cached_tokens, s.num_scheduled_tokens
            toks = s.token_ids[c:c + n]
            src = [-1] * n
            if toks[-1] == PENDING:
                toks = toks[:-1] + [0]
                src[-1] = prev["index"][s.seq_id]
            rows.append((s.seq_id, c, n, tuple(toks), tuple(src), s.samples_this_step()))
            self.cache.advance(s.seq_id, c + n)
        samplers = [s for s in b.seqs if s.samples_this_step()]
        flags = self.sched.on_launched(b)
        self.inflight.append({"batch": b, "flags": flags, "index": {s.seq_id: i for i, s in enumerate(samplers)}})
        if b.blocked:
            while self.inflight:
                self.retire()
        else:
            while len(self.inflight) >= self.depth:
                self.retire()
        return (rows, [s.seq_id for s in b.preempted], b.blocked)


class NativeLoop:
    """The same loop around the scheduler in C++."""

    def __init__(self, cfg, blocks, page, slots, prefix, depth, window=0):
        self.cache = NativeCacheManager(groups_of(blocks, window), page, slots, (cfg.max_model_len + page - 1) // page,
                                        prefix_caching=prefix)
        self.sched = NativeScheduler(cfg, self.cache)
        self.depth, self.inflight, self.results = depth, [], {}

    def add(self, rid, prompt, sp):
        self.sched.add_request(rid, prompt, sp, row_seed=rid)

    def finished(self):
        return not self.inflight and self.sched.is_finished()

    def retire(self):
        toks = self.inflight.pop(0)
        for rid in self.sched.postprocess(toks):
            self.results[rid] = (self.sched.tokens(rid), self.sched.info(rid)["stopped_on_eos"])
            assert self.sched.info(rid)["status"] == "finished"
            self.sched.forget(rid)

    def step(self):
        if self.sched.is_finished():
            while self.inflight:
                self.retire()
            return None
        b = self.sched.schedule(allow_preempt=not self.inflight)
        if not b.ids:
            while self.inflight:
                self.retire()
            return ("empty", b.preempted, b.blocked)
        rows, o, fake = [], 0, []
        for rid, c, n, smp in zip(b.ids, b.starts, b.counts, b.samples):
            rows.append((rid, c, n, tuple(b.tokens[o:o + n].tolist()), tuple(b.feed_src[o:o + n].tolist()), smp))
            assert self.cache.lease(rid).computed == c and self.cache.lease(rid).state_slot == self.sched.info(rid)["state_slot"]
            self.cache.advance(rid, c + n)
            if smp:
                fake.append(sample(rid, c + n))
            o += n
        assert o == b.total_tokens and len(fake) == len(b.temps) == len(b.generated)
        assert b.need_feed == any(x >= 0 for x in b.feed_src.tolist())
        assert self.sched.on_launched() == len(fake)
        self.inflight.append(fake)
        if b.blocked:
            while self.inflight:
                self.retire()
        else:
            while len(self.inflight) >= self.depth:
                self.retire()
        return (rows, b.preempted, b.blocked)


def run_both(cfg, blocks, page, slots, requests, prefix=False, depth=2, arrivals=None, max_steps=5000, window=0):
    loops = [PythonLoop(cfg, blocks, page, slots, prefix, depth, window), NativeLoop(cfg, blocks, page, slots, prefix, depth, window)]
    arrivals = arrivals or {}
    pending = list(enumerate(requests))
    steps = 0
    while True:
        due = [r for r in pending if arrivals.get(r[0], 0) <= steps]
        pending = [r for r in pending if arrivals.get(r[0], 0) > steps]
        for rid, (prompt, sp) in due:
            for lp in loops:
                lp.add(rid, prompt, sp)
        if not pending and all(lp.finished() for lp in loops):
            break
        a, b = loops[0].step(), loops[1].step()
        assert a == b, (steps, a, b)
        assert loops[0].sched.num_preemptions == loops[1].sched.num_preemptions
        assert [s.seq_id for s in loops[0].sched.running] == loops[1].sched.running
        assert [s.seq_id for s in loops[0].sched.waiting] == loops[1].sched.waiting
        if steps % 7 == 0:
            same_state(loops[0].cache, loops[1].cache)
        steps += 1
        assert steps < max_steps
    same_state(loops[0].cache, loops[1].cache)
    assert loops[0].results == loops[1].results and len(loops[0].results) == len(requests)
    assert loops[1].cache.num_free_pages() == blocks and not loops[1].cache.leases
    assert all(loops[1].cache.num_free_pages(g) == gc.num_pages for g, gc in enumerate(loops[1].cache.groups))
    return loops, steps


@pytest.mark.parametrize("depth", [1, 2])
@pytest.mark.parametrize("prefix", [False, True])
@pytest.mark.parametrize("seed", range(8))
def test_random_workloads_give_the_same_steps(seed, prefix, depth):
    rng = random.Random(1000 + seed)
    page = rng.choice([4, 8, 16])
    blocks = rng.randint(12, 40) if seed < 4 else rng.randint(8, 16)          # the small pools run out of pages
    cfg = SchedulerConfig(rng.choice([16, 48, 128]), rng.choice([2, 4, 8]), rng.choice([0, 8, 24]), blocks * page // 2, (EOS,))
    stems = [[rng.randint(0, 49) for _ in range(4 * page)] for _ in range(2)]
    requests, arrivals = [], {}
    for i in range(rng.randint(6, 14)):
        stem = rng.choice(stems)[:rng.randint(0, 4 * page)] if rng.random() < 0.6 else []
        prompt = stem + [rng.randint(0, 49) for _ in range(rng.randint(1, 3 * page))]
        room = cfg.max_model_len - len(prompt)
        if room < 1:
            prompt = prompt[:cfg.max_model_len - 4]
            room = 4
        sp = SamplingParams(temperature=rng.choice([0.0, 0.7]), max_tokens=rng.randint(1, min(room, 3 * page)),
                            ignore_eos=rng.random() < 0.5)
        requests.append((prompt, sp))
        arrivals[i] = rng.randint(0, 30)
    loops, steps = run_both(cfg, blocks, page, 8, requests, prefix=prefix, depth=depth, arrivals=arrivals)
    assert steps > 5


def test_pages_run_out_and_requests_are_preempted_in_both():
    cfg = SchedulerConfig(64, 4, 16, 96, ())
    requests = [([i + 1] * n, SamplingParams(max_tokens=40, ignore_eos=True)) for i, n in enumerate((30, 25, 20, 28))]
    loops, _ = run_both(cfg, blocks=10, page=16, slots=4, requests=requests, depth=2)
    assert loops[1].sched.num_preemptions > 0


@pytest.mark.parametrize("seed", range(4))
def test_two_groups_of_pages_one_with_a_window(seed):
    """A second group of cache units that looks back only `window` positions: it holds few pages per request and gives
    them back as decoding goes on, so the two groups run out at different times."""
    rng = random.Random(50 + seed)
    page, blocks = 8, rng.randint(14, 24)
    cfg = SchedulerConfig(48, 4, 16, blocks * page // 2, ())
    requests = [([rng.randint(0, 49) for _ in range(rng.randint(1, 5 * page))],
                 SamplingParams(max_tokens=rng.randint(1, 4 * page), ignore_eos=True)) for _ in range(8)]
    requests = [(p[:cfg.max_model_len - sp.max_tokens] or [1], sp) for p, sp in requests]
    loops, _ = run_both(cfg, blocks, page, 6, requests, depth=2, window=rng.choice([page, 2 * page + 3]),
                        arrivals={i: rng.randint(0, 12) for i in range(8)})


def test_requests_are_refused_as_the_twin_refuses_them():
    cfg = SchedulerConfig(64, 4, 16, 64, ())
    cache = NativeCacheManager([GroupConfig(3)], 16, 4, 4)
    s = NativeScheduler(cfg, cache)
    with pytest.raises(ValueError, match="max_model_len"):
        s.add_request(0, [1] * 60, SamplingParams(max_tokens=5), 0)
    with pytest.raises(ValueError, match="cache pages"):
        s.add_request(1, [1] * 50, SamplingParams(max_tokens=5), 0)
    with pytest.raises(ValueError, match="at least one"):
        s.add_request(2, [], SamplingParams(max_tokens=5), 0)
    s.add_request(3, [1, 2, 3], SamplingParams(max_tokens=2), 0)
    with pytest.raises(ValueError, match="in use"):
        s.add_request(3, [1], SamplingParams(max_tokens=2), 0)
    with pytest.raises(TypeError):
        NativeScheduler(cfg, CacheManager([GroupConfig(3)], 16, 4))


@pytest.mark.parametrize("case", json.load(open(GOLDEN)), ids=lambda c: f"blocks{c['blocks']}")
def test_same_batches_as_the_reference_scheduler(case):
    """The reference's scheduler and block manager, compiled and run on these workloads, wrote tests/golden: the
    scheduler in C++ schedules the same (request, tokens, samples) in every step, with the prefix cache on and pages of
    16 as there, and the driver's tokens (all distinct, counted up from 1000 in the driver's order)."""
    page = 16
    cfg = SchedulerConfig(case["budget"], case["max_seqs"], case["chunk"], 4096, ())
    cache = NativeCacheManager([GroupConfig(case["blocks"])], page, max(8, case["max_seqs"]), 4096 // page, prefix_caching=True)
    s = NativeScheduler(cfg, cache)
    nxt = 1000
    for i, n in enumerate(case["prompts"]):
        s.add_request(i, list(range(nxt, nxt + n)), SamplingParams(max_tokens=case["max_tokens"], ignore_eos=True), i)
        nxt += n
    steps = []
    while not s.is_finished():
        assert len(steps) < 2000
        b = s.schedule()
        cache.check_invariants()
        steps.append([[rid, n, int(smp)] for rid, n, smp in zip(b.ids, b.counts, b.samples)])
        for rid, c, n in zip(b.ids, b.starts, b.counts):
            cache.slots_for(rid, 0, c, n)
            cache.advance(rid, c + n)
        toks = []
        for smp in b.samples:                             # the driver draws a token for every scheduled request
            if smp:
                toks.append(nxt)
            nxt += 1
        assert s.on_launched() == len(toks)
        s.postprocess(toks)
    cache.check_invariants()
    assert steps == case["steps"]
    assert s.num_preemptions == case["preemptions"]
    assert (cache.prefix_hits > 0) == (case["preemptions"] > 0)
    assert cache.num_free_pages() == case["blocks"]
