"""The scheduler's decisions (CPU, no model): portions under a budget, admission, finishing, preemption.

`golden/scheduler_golden.json` was printed by the reference's own scheduler and block manager, compiled on the
CPU by `golden/scheduler_driver.cpp`; the same workloads must produce the same batches here."""
import json
import os

import pytest

from cppvllm_b200.cache.manager import CacheManager, GroupConfig
from cppvllm_b200.engine.scheduler import FINISHED, Scheduler, SchedulerConfig, Sequence
from cppvllm_b200.sampling.params import SamplingParams

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "scheduler_golden.json")


_KIND = "python"


@pytest.fixture(autouse=True, params=["python", "native"])
def manager_kind(request):
    """Every test of this file runs with the cache manager in Python and with the one in C++."""
    global _KIND
    _KIND = request.param
    yield
    _KIND = "python"


def make(blocks, budget, chunk, max_seqs, page=16, max_model_len=4096, eos=(), prefix_caching=False):
    if _KIND == "native":
        from cppvllm_b200.cache.native import NativeCacheManager
        cache = NativeCacheManager([GroupConfig(blocks)], page, max(8, max_seqs), (max_model_len + page - 1) // page,
                                   prefix_caching=prefix_caching)
    else:
        cache = CacheManager([GroupConfig(blocks)], page, max(8, max_seqs), prefix_caching=prefix_caching)
    return Scheduler(SchedulerConfig(budget, max_seqs, chunk, max_model_len, tuple(eos)), cache), cache


def run(sched, cache, seqs, token=lambda step, seq: 7, max_steps=2000):
    """Drive the scheduler with a model that 'samples' `token`; returns per step [(id, n, samples)]."""
    for s in seqs:
        sched.add_request(s)
    steps = []
    while not sched.is_finished():
        assert len(steps) < max_steps
        b = sched.schedule()
        cache.check_invariants()
        steps.append([(s.seq_id, s.num_scheduled_tokens, int(s.samples_this_step())) for s in b.seqs])
        for s in b.seqs:                                  # every scheduled token has a page
            cache.slots_for(s.seq_id, 0, s.num_cached_tokens, s.num_scheduled_tokens)
            cache.advance(s.seq_id, s.num_cached_tokens + s.num_scheduled_tokens)
        flags = sched.on_launched(b)
        toks = [token(len(steps), s) for s, f in zip(b.seqs, flags) if f]
        sched.postprocess(b, flags, toks)
    cache.check_invariants()
    return steps


@pytest.mark.parametrize("case", json.load(open(GOLDEN)), ids=lambda c: f"blocks{c['blocks']}")
def test_same_batches_as_the_reference_scheduler_with_the_prefix_cache(case):
    """With the prefix cache on (as in the reference, where it cannot be switched off) and the driver's tokens (every
    prompt token and every sampled token distinct, counted up from 1000 in the driver's order), every step of every
    case is the reference's, the re-admission of preempted requests behind their own surviving pages included."""
    sched, cache = make(case["blocks"], case["budget"], case["chunk"], case["max_seqs"], prefix_caching=True)
    nxt = [1000]

    def fresh(n):
        out = list(range(nxt[0], nxt[0] + n))
        nxt[0] += n
        return out

    seqs = [Sequence(i, fresh(n), SamplingParams(max_tokens=case["max_tokens"], ignore_eos=True))
            for i, n in enumerate(case["prompts"])]
    for s in seqs:
        sched.add_request(s)
    steps = []
    while not sched.is_finished():
        assert len(steps) < 2000
        b = sched.schedule()
        cache.check_invariants()
        steps.append([[s.seq_id, s.num_scheduled_tokens, int(s.samples_this_step())] for s in b.seqs])
        for s in b.seqs:
            cache.slots_for(s.seq_id, 0, s.num_cached_tokens, s.num_scheduled_tokens)
            cache.advance(s.seq_id, s.num_cached_tokens + s.num_scheduled_tokens)
        flags = sched.on_launched(b)
        toks = []
        for f in flags:                                   # the driver draws a token for every scheduled request
            if f:
                toks.append(nxt[0])
            nxt[0] += 1
        sched.postprocess(b, flags, toks)
    cache.check_invariants()
    assert steps == case["steps"]
    assert sched.num_preemptions == case["preemptions"]
    assert (cache.prefix_hits > 0) == (case["preemptions"] > 0)
    assert cache.num_free_pages() == case["blocks"]


@pytest.mark.parametrize("case", json.load(open(GOLDEN)), ids=lambda c: f"blocks{c['blocks']}")
def test_same_batches_as_the_reference_scheduler(case):
    sched, cache = make(case["blocks"], case["budget"], case["chunk"], case["max_seqs"])
    seqs = [Sequence(i, list(range(n)), SamplingParams(max_tokens=case["max_tokens"], ignore_eos=True))
            for i, n in enumerate(case["prompts"])]
    steps = [[list(x) for x in st] for st in run(sched, cache, seqs)]
    if case["preemptions"] == 0:
        assert steps == case["steps"]
    else:
        # Without the prefix cache a preempted request recomputes all of its tokens, where the reference finds its
        # first full blocks again (engine/block_manager.cpp:80-116) and recomputes fewer.  Up to the first
        # re-admission, victims included, the decisions are the same.
        gone = set()
        for n, (mine, ref) in enumerate(zip(steps, case["steps"])):
            back = [x[0] for x in ref if x[0] in gone]
            if back:
                break
            assert mine == ref, f"step {n}"
            if n + 1 < len(case["steps"]):
                nxt = {x[0] for x in case["steps"][n + 1]}
                gone |= {x[0] for x in ref if x[0] not in nxt and x[2] == 1 and
                         len([1 for st in case["steps"][:n + 1] for y in st if y[0] == x[0] and y[2]]) < case["max_tokens"]}
        assert n >= 19 and gone
    assert sched.num_preemptions == case["preemptions"]
    assert all(s.status == FINISHED and s.num_completion_tokens == case["max_tokens"] for s in seqs)
    assert cache.num_free_pages() == case["blocks"]


def test_requests_with_a_common_prefix_share_pages():
    """Three requests whose prompts begin with the same 40 tokens: the first computes everything; the later ones,
    admitted after the first one's pages were registered, start behind two shared pages of 16."""
    sched, cache = make(32, budget=64, chunk=0, max_seqs=4, prefix_caching=True)
    common = list(range(500, 540))
    a = Sequence(0, common + [1, 2, 3], SamplingParams(max_tokens=3, ignore_eos=True))
    steps = run(sched, cache, [a], token=lambda step, seq: 900 + step)
    assert steps[0] == [(0, 43, 1)]
    b = Sequence(1, common + [7, 8], SamplingParams(max_tokens=2, ignore_eos=True))
    c = Sequence(2, common[:33], SamplingParams(max_tokens=2, ignore_eos=True))
    steps = run(sched, cache, [b, c], token=lambda step, seq: 800 + step)
    assert steps[0] == [(1, 42 - 32, 1), (2, 33 - 32, 1)]   # both start at token 32: two full pages are shared
    assert cache.prefix_hits == 4
    cache.check_invariants()
    assert cache.num_free_pages() == 32
    # a prompt that IS two full pages still computes its last token (at least one token always runs)
    d = Sequence(3, common[:32], SamplingParams(max_tokens=1, ignore_eos=True))
    steps = run(sched, cache, [d], token=lambda step, seq: 700)
    assert steps[0] == [(3, 16, 1)]


def test_budget_and_chunk_cap_cut_prompts_into_portions():
    sched, cache = make(64, budget=50, chunk=20, max_seqs=8)
    a, b = Sequence(0, list(range(45)), SamplingParams(max_tokens=2)), Sequence(1, list(range(30)), SamplingParams(max_tokens=2))
    steps = run(sched, cache, [a, b])
    assert steps[0] == [(0, 20, 0), (1, 20, 0)]            # each capped at 20, 40 <= 50
    assert steps[1] == [(0, 20, 0), (1, 10, 1)]            # b ends its prompt and samples
    assert steps[2] == [(0, 5, 1), (1, 1, 1)]              # a's last portion beside b's decoded token
    assert steps[3] == [(0, 1, 1)]
    no_cap, c2 = make(64, budget=50, chunk=0, max_seqs=8)
    assert run(no_cap, c2, [Sequence(0, list(range(45)), SamplingParams(max_tokens=1))])[0] == [(0, 45, 1)]


def test_max_num_seqs_and_first_come_first_served():
    sched, cache = make(64, budget=100, chunk=0, max_seqs=2)
    seqs = [Sequence(i, [1, 2, 3], SamplingParams(max_tokens=2)) for i in range(4)]
    steps = run(sched, cache, seqs)
    assert steps[0] == [(0, 3, 1), (1, 3, 1)] and steps[1] == [(0, 1, 1), (1, 1, 1)]
    assert steps[2] == [(2, 3, 1), (3, 3, 1)]


def test_eos_finishes_unless_ignored_and_max_tokens_bounds():
    sched, cache = make(16, 64, 0, 4, eos=(99,))
    a = Sequence(0, [1, 2], SamplingParams(max_tokens=10))
    b = Sequence(1, [1, 2], SamplingParams(max_tokens=3, ignore_eos=True))
    run(sched, cache, [a, b], token=lambda step, s: 99 if step == 2 else 5)
    assert a.token_ids == [1, 2, 5, 99] and a.stopped_on_eos
    assert b.token_ids == [1, 2, 5, 99, 5] and not b.stopped_on_eos


def test_oversize_requests_are_refused_at_admission():
    sched, cache = make(4, 64, 0, 4, max_model_len=100)
    with pytest.raises(ValueError, match="cache pages"):
        sched.add_request(Sequence(0, list(range(60)), SamplingParams(max_tokens=10)))      # 5 pages > 4
    with pytest.raises(ValueError, match="max_model_len"):
        sched.add_request(Sequence(1, list(range(50)), SamplingParams(max_tokens=60)))
    with pytest.raises(ValueError, match="at least one"):
        Sequence(2, [], SamplingParams())


def test_pages_run_out_last_running_request_is_preempted_and_recomputed():
    # 4 pages of 16.  Two requests of 31 tokens fill them; when request 0 crosses into a third page, the last
    # running request (1) is preempted: it gives back everything, keeps its tokens and later runs them again.
    sched, cache = make(4, 64, 0, 4)
    a = Sequence(0, list(range(31)), SamplingParams(max_tokens=8, ignore_eos=True))
    b = Sequence(1, list(range(100, 131)), SamplingParams(max_tokens=8, ignore_eos=True))
    steps = run(sched, cache, [a, b])
    assert steps[0] == [(0, 31, 1), (1, 31, 1)] and steps[1] == [(0, 1, 1), (1, 1, 1)]
    assert steps[2] == [(0, 1, 1)]                          # 0 needs a third page -> 1 is preempted
    assert sched.num_preemptions >= 1 and b.num_preemptions >= 1
    readmit = next(st for st in steps[3:] if any(x[0] == 1 for x in st))
    n_again = [x for x in readmit if x[0] == 1][0][1]
    assert n_again > 31                                     # prompt plus what it had generated, as one portion
    assert a.num_completion_tokens == 8 and b.num_completion_tokens == 8
    assert b.token_ids[:31] == list(range(100, 131))


def test_a_request_alone_preempts_itself_only_if_it_cannot_fit():
    sched, cache = make(3, 64, 0, 4)
    a = Sequence(0, list(range(40)), SamplingParams(max_tokens=8, ignore_eos=True))       # 48 tokens = 3 pages: fits
    run(sched, cache, [a])
    assert sched.num_preemptions == 0 and a.num_completion_tokens == 8


def test_with_a_step_in_flight_nothing_is_preempted_and_the_batch_is_blocked():
    sched, cache = make(4, 64, 0, 4)
    a = Sequence(0, list(range(31)), SamplingParams(max_tokens=8, ignore_eos=True))
    b = Sequence(1, list(range(100, 131)), SamplingParams(max_tokens=8, ignore_eos=True))
    sched.add_request(a)
    sched.add_request(b)
    inflight = []
    for _ in range(2):                                        # two steps without reading anything back
        batch = sched.schedule(allow_preempt=not inflight)
        for s in batch.seqs:
            cache.advance(s.seq_id, s.num_cached_tokens + s.num_scheduled_tokens)
        inflight.append((batch, sched.on_launched(batch)))
    assert a.token_ids[-1] == -1 and len(a) == 33             # a placeholder stands for the token in flight
    blocked = sched.schedule(allow_preempt=False)             # both need a third page, none is free
    assert blocked.blocked and blocked.seqs == [] and sched.num_preemptions == 0
    for batch, flags in inflight:                             # the engine drains ...
        sched.postprocess(batch, flags, [7] * sum(flags))
    assert a.token_ids[-2:] == [7, 7] and -1 not in a.token_ids
    nxt = sched.schedule(allow_preempt=True)                  # ... and now the last running request gives way
    assert [s.seq_id for s in nxt.seqs] == [0] and sched.num_preemptions == 1 and not nxt.blocked


def test_a_request_that_finished_while_a_later_step_was_in_flight_drops_the_later_result():
    sched, cache = make(8, 64, 0, 4, eos=(99,))
    a = Sequence(0, [1, 2, 3], SamplingParams(max_tokens=10))
    sched.add_request(a)
    recs = []
    for _ in range(2):
        batch = sched.schedule(allow_preempt=not recs)
        for s in batch.seqs:
            cache.advance(s.seq_id, s.num_cached_tokens + s.num_scheduled_tokens)
        recs.append((batch, sched.on_launched(batch)))
    assert a.token_ids == [1, 2, 3, -1, -1]
    assert sched.postprocess(recs[0][0], recs[0][1], [99]) == [a]      # the first sample ends the request
    assert a.token_ids == [1, 2, 3, 99] and a.stopped_on_eos and cache.num_free_pages() == 8
    assert sched.postprocess(recs[1][0], recs[1][1], [5]) == []         # the second step's sample is dropped
    assert a.token_ids == [1, 2, 3, 99] and sched.is_finished()
    cache.check_invariants()


def test_max_tokens_counts_the_token_in_flight():
    sched, cache = make(8, 64, 0, 4)
    a = Sequence(0, [1, 2, 3], SamplingParams(max_tokens=1, ignore_eos=True))
    sched.add_request(a)
    batch = sched.schedule()
    rec = (batch, sched.on_launched(batch))
    assert sched.schedule(allow_preempt=False).seqs == []               # its only token is in flight already
    sched.postprocess(rec[0], rec[1], [4])
    assert a.token_ids == [1, 2, 3, 4] and sched.is_finished()
