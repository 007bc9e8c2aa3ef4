"""The engine's own loop (LLMEngine.add_request / step / generate) on the CPU, with stand-ins for the model runner and
the sampler: the runtime in C++ (cache manager and scheduler, the default) and its twins in Python must take the same
steps and return the same results, with one and two steps in flight, end-of-sequence tokens, temperatures and seeds that
reach the sampler, pools that run out, and the prefix cache."""
import random
import types

import pytest

from cppvllm_b200.cache.manager import CacheManager, GroupConfig
from cppvllm_b200.cache.native import NativeCacheManager
from cppvllm_b200.config.engine_config import EngineConfig
from cppvllm_b200.engine.llm_engine import LLMEngine
from cppvllm_b200.sampling.params import SamplingParams

EOS = 13
VOCAB = 50


def token_for(rid, pos: int) -> int:
    return (int(rid) * 17 + pos * 5 + (pos * pos) % 7) % VOCAB


class FakeRunner:
    """What the engine uses of a ModelRunner; a step returns, as its 'logits', which (request, position) it samples."""

    def __init__(self, native: bool, blocks: int, page: int, max_seqs: int, max_model_len: int, prefix: bool):
        groups = [GroupConfig(blocks)]
        width = (max_model_len + page - 1) // page
        self.cache = (NativeCacheManager(groups, page, max_seqs, width, prefix_caching=prefix) if native
                      else CacheManager(groups, page, max_seqs, prefix_caching=prefix))
        self.config = types.SimpleNamespace(eos_token_ids=(EOS,))
        self.device, self.vocab_size, self.max_model_len, self.num_pages = "cpu", VOCAB, max_model_len, blocks
        self.log = []

    def step(self, entries, feed=None):
        rows, fed, t = [], [], 0
        for e in entries:
            lease = self.cache.lease(e.request_id)
            assert lease.computed == e.start
            toks = [int(x) for x in e.tokens]
            assert self.cache.covered(e.request_id, e.start + len(toks))        # pages for every token of the step
            for w in e.want:
                rows.append((e.request_id, e.start + w + 1))
            if feed is not None:
                fed.append(tuple(int(x) for x in feed[1][t:t + len(toks)]))
            else:
                fed.append((-1,) * len(toks))
            t += len(toks)
            self.cache.advance(e.request_id, e.start + len(toks))
        self.log.append([(e.request_id, e.start, tuple(int(x) for x in e.tokens), tuple(e.want), f) for e, f in zip(entries, fed)])
        return rows

    def check_errors(self):
        pass


class FakeSampler:
    def __init__(self):
        self.pending, self.calls = {}, []

    def sample_async(self, logits, temps, seeds, positions, slot=0):
        assert len(logits) == len(temps) == len(seeds) == len(positions)
        self.calls.append([(rid, pos, round(float(t), 4), int(s), int(p)) for (rid, pos), t, s, p in zip(logits, temps, seeds, positions)])
        self.pending[slot] = [token_for(rid, pos) for rid, pos in logits]
        return ("device", slot)

    def collect(self, n, slot=0):
        out = self.pending.pop(slot)
        assert len(out) == n
        return out


def make_engine(native: bool, depth: int, blocks=24, page=8, max_seqs=4, budget=48, chunk=16, prefix=False):
    max_model_len = blocks * page // 2
    cfg = EngineConfig(model_path="", max_num_batched_tokens=budget, max_num_seqs=max_seqs, max_chunk_tokens=chunk,
                       max_model_len=max_model_len, block_size=16, pipeline_depth=depth, enable_prefix_caching=prefix,
                       native_cache_manager=native, native_scheduler=native, seed=5)
    return LLMEngine(cfg, runner=FakeRunner(native, blocks, page, max_seqs, max_model_len, prefix), sampler=FakeSampler())


def workload(rng, n, page, max_model_len):
    stems = [[rng.randint(0, VOCAB - 1) for _ in range(3 * page)] for _ in range(2)]
    reqs = []
    for i in range(n):
        prompt = (rng.choice(stems)[:rng.randint(0, 3 * page)] if rng.random() < 0.6 else []) + \
                 [rng.randint(0, VOCAB - 1) for _ in range(rng.randint(1, 2 * page))]
        room = max(1, max_model_len - len(prompt))
        sp = SamplingParams(temperature=rng.choice([0.0, 0.6, 1.0]), max_tokens=rng.randint(1, min(room, 3 * page)),
                            ignore_eos=rng.random() < 0.5, seed=rng.choice([None, 7, 123456789012345]))
        reqs.append((prompt, sp))
    return reqs


@pytest.mark.parametrize("depth", [1, 2])
@pytest.mark.parametrize("prefix", [False, True])
@pytest.mark.parametrize("seed", range(4))
def test_engines_with_the_runtime_in_cpp_and_in_python_take_the_same_steps(seed, prefix, depth):
    rng = random.Random(300 + seed)
    blocks = rng.choice([10, 16, 30])
    a, b = (make_engine(native, depth, blocks=blocks, prefix=prefix) for native in (True, False))
    assert a._native and not b._native
    reqs = workload(rng, rng.randint(5, 10), 8, a.runner.max_model_len)
    later = reqs[len(reqs) // 2:]
    for prompt, sp in reqs[:len(reqs) // 2]:
        assert a.add_request(prompt, sp) == b.add_request(prompt, sp)
    steps = 0
    while not (a.is_finished() and b.is_finished() and not later):
        if later and steps % 3 == 0:
            prompt, sp = later.pop(0)
            assert a.add_request(prompt, sp) == b.add_request(prompt, sp)
        ia, ib = a.step(), b.step()
        assert (ia.num_seqs, ia.num_tokens, ia.num_sampled, ia.num_finished) == (ib.num_seqs, ib.num_tokens, ib.num_sampled, ib.num_finished)
        assert a.stats().preemptions == b.stats().preemptions and a.stats().prefix_hit_pages == b.stats().prefix_hit_pages
        steps += 1
        assert steps < 3000
    a.sync()
    b.sync()
    assert a.runner.log == b.runner.log                       # the same entries, tokens, wanted rows and fed rows every step
    assert a.sampler.calls == b.sampler.calls                 # the same temperatures, seeds and output positions
    outs = [[(o.request_id, o.prompt_ids, o.token_ids, o.stopped_on_eos) for o in e.take_finished()] for e in (a, b)]
    assert outs[0] == outs[1] and len(outs[0]) == len(reqs)
    for (rid, prompt, toks, eos), (want_prompt, sp) in zip(outs[0], reqs):
        assert prompt == want_prompt and len(toks) <= sp.max_tokens
        assert toks == [token_for(rid, len(prompt) + i) for i in range(len(toks))] or eos
        if eos:
            assert not sp.ignore_eos and EOS not in toks and len(toks) < sp.max_tokens + 1
    for e in (a, b):
        e.runner.cache.check_invariants()
        assert e.runner.cache.num_free_pages() == blocks and not e.runner.cache.leases
    assert a.stats().tokens_generated == b.stats().tokens_generated


def test_generate_returns_the_requests_in_order_and_refuses_what_cannot_fit():
    for native in (True, False):
        e = make_engine(native, 2, blocks=6, page=8, max_seqs=2)
        outs = e.generate([[1, 2, 3], [4] * 10, [5]], SamplingParams(max_tokens=6, ignore_eos=True))
        assert [o.request_id for o in outs] == [0, 1, 2]
        assert [len(o.token_ids) for o in outs] == [6, 6, 6]
        assert outs[1].token_ids == [token_for(1, 10 + i) for i in range(6)]
        with pytest.raises(ValueError, match="max_model_len"):
            e.add_request([1] * 20, SamplingParams(max_tokens=10))
        with pytest.raises(ValueError, match="vocabulary"):
            e.add_request([VOCAB + 3], SamplingParams(max_tokens=1))
        assert e.stats().preemptions >= 0 and e.num_without_first_token() == 0
