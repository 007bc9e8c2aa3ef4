"""The engine's public face, in the reference's manner (engine/llm_engine.h:34-69, example.cpp, bench.cpp):

    engine = LLMEngine(EngineConfig(model_path=..., dtype="bfloat16"))
    outs = engine.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.6, max_tokens=64))

``add_request`` / ``step`` / ``is_finished`` / ``generate`` / ``take_finished`` / ``stats`` / ``num_kv_blocks`` keep the
reference's names and meanings.  Token ids go in and come out; there is no tokenizer.  ``LLM`` is the same class
under the name a Python user expects.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence as Seq, Union

import torch

from ..config.engine_config import EngineConfig
from ..sampling.params import SamplingParams
from ..sampling.sampler import Sampler, mix_seed
from .runner import ModelRunner, StepEntry
from .native_scheduler import NativeScheduler
from .scheduler import FINISHED, PENDING, ScheduledBatch, Scheduler, SchedulerConfig, Sequence


@dataclass
class GenerationOutput:
    request_id: int = 0
    prompt_ids: List[int] = field(default_factory=list)
    token_ids: List[int] = field(default_factory=list)
    stopped_on_eos: bool = False


@dataclass
class StepInfo:
    num_seqs: int = 0
    num_tokens: int = 0
    num_sampled: int = 0
    num_finished: int = 0


@dataclass
class EngineStats:
    steps: int = 0
    tokens_processed: int = 0
    tokens_generated: int = 0
    preemptions: int = 0
    prefix_hit_pages: int = 0            # cache pages that admissions took from the prefix cache
    seconds: float = 0.0

    def generated_per_second(self) -> float:
        return self.tokens_generated / self.seconds if self.seconds > 0 else 0.0


class LLMEngine:
    def __init__(self, config: Union[EngineConfig, str, None] = None, *, runner=None, sampler=None, **kwargs):
        """`runner` and `sampler`: objects to use instead of a ModelRunner and a Sampler built from the configuration (the
        tests of the engine's loop on the CPU hand in stand-ins that need no device)."""
        if isinstance(config, str):
            config = EngineConfig(model_path=config, **kwargs)
        elif config is None:
            config = EngineConfig(**kwargs)
        elif kwargs:
            raise TypeError("pass either an EngineConfig or keyword options, not both")
        self.config = config
        self.runner = runner if runner is not None else ModelRunner(
            config.model_path, dtype=config.dtype, device=config.device, page_size=config.block_size,
            num_pages=config.num_kv_blocks if config.num_kv_blocks > 0 else None,
            max_step_tokens=config.max_num_batched_tokens, max_seqs=config.max_num_seqs,
            max_model_len=config.max_model_len, gpu_memory_utilization=config.gpu_memory_utilization,
            enforce_eager=config.enforce_eager, enable_prefix_caching=config.enable_prefix_caching,
            use_ref_kernels=config.use_ref_kernels, native_cache_manager=config.native_cache_manager)
        eos = tuple(getattr(self.runner.config, "eos_token_ids", ()) or ())
        sched_cfg = SchedulerConfig(
            max_num_batched_tokens=config.max_num_batched_tokens, max_num_seqs=config.max_num_seqs,
            max_chunk_tokens=config.max_chunk_tokens, max_model_len=self.runner.max_model_len, eos_token_ids=eos)
        # the scheduler in C++ keeps the requests itself and works on the cache manager in C++; else the twins in Python
        self._native = bool(config.native_scheduler and getattr(self.runner.cache, "native", False))
        self.scheduler = NativeScheduler(sched_cfg, self.runner.cache) if self._native else Scheduler(sched_cfg, self.runner.cache)
        self.sampler = sampler if sampler is not None else Sampler(self.runner.device, config.max_num_seqs)
        self._live: Dict[int, Sequence] = {}
        self._finished: Dict[int, GenerationOutput] = {}
        self._next_id = 0
        self._stats = EngineStats()
        self._empty_steps = 0
        self._inflight: List[dict] = []
        self._forget_later: List[int] = []
        self._slot = 0

    # ---- requests ------------------------------------------------------------------------------------
    def add_request(self, prompt: Seq[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams()
        vocab = self.runner.vocab_size
        for t in prompt:
            if not (0 <= int(t) < vocab):
                raise ValueError(f"prompt token {t} lies outside the vocabulary of {vocab}")
        rid = self._next_id
        row_seed = mix_seed(self.config.seed, params.seed if params.seed is not None else rid)
        if self._native:
            self.scheduler.add_request(rid, prompt, params, row_seed)
            self._live[rid] = None
        else:
            seq = Sequence(rid, prompt, params)
            seq.row_seed = row_seed
            self.scheduler.add_request(seq)
            self._live[rid] = seq
        self._next_id += 1
        return rid

    def num_without_first_token(self) -> int:
        """Live requests that have not sampled their first token yet."""
        if self._native:
            n = 0
            for rid in self._live:
                d = self.scheduler.info(rid)
                n += 1 if d["num_tokens"] <= d["num_prompt_tokens"] else 0
            return n
        return sum(1 for s in self._live.values() if s.num_completion_tokens == 0)

    def is_finished(self) -> bool:
        return not self._inflight and self.scheduler.is_finished()

    @property
    def num_kv_blocks(self) -> int:
        return self.runner.num_pages

    def stats(self) -> EngineStats:
        return self._stats

    # ---- one step -------------------------------------------------------------------------------------
    def step(self) -> StepInfo:
        """Schedule and launch one step; with ``pipeline_depth`` 2 the previous step's samples are read back only
        after this one has been handed to the device (reference engine/llm_engine.cpp:70-113).  A token that is not
        known on the host yet travels from the previous step's samples to this step's inputs on the device."""
        info = StepInfo()
        t0 = time.perf_counter()
        if self.scheduler.is_finished():
            self.sync(info)
            return info
        if self._native:
            return self._step_native(info, t0)
        batch = self.scheduler.schedule(allow_preempt=not self._inflight)
        self._stats.preemptions = self.scheduler.num_preemptions
        self._stats.prefix_hit_pages = self.runner.cache.prefix_hits
        if not batch.seqs:
            if self._inflight:                                 # everything runnable waits for tokens in flight
                self.sync(info)
                self._account(info, t0)
                return info
            self._empty_steps += 1
            if self._empty_steps > 2:
                raise RuntimeError("the scheduler produced no work although requests are pending")
            return info
        self._empty_steps = 0

        prev = self._inflight[-1] if self._inflight else None
        entries, feed_src, need_feed = [], [], False
        for seq in batch.seqs:
            c, n = seq.num_cached_tokens, seq.num_scheduled_tokens
            toks = seq.token_ids[c:c + n]
            src = [-1] * n
            if toks[-1] == PENDING:                            # sampled by the step in flight: fed on the device
                toks = toks[:-1] + [0]
                src[-1] = prev["index"][seq.seq_id]
                need_feed = True
            entries.append(StepEntry(seq.seq_id, toks, c, (n - 1,) if seq.samples_this_step() else ()))
            feed_src.extend(src)
        feed = (prev["sampled"], feed_src) if need_feed else None
        logits = self.runner.step(entries, feed=feed)
        samplers = [s for s in batch.seqs if s.samples_this_step()]
        slot = self._slot
        self._slot ^= 1
        sampled_dev = self.sampler.sample_async(
            logits, [s.params.temperature for s in samplers], [s.row_seed for s in samplers],
            [s.num_completion_tokens for s in samplers], slot=slot) if samplers else None
        flags = self.scheduler.on_launched(batch)
        self._inflight.append({"batch": batch, "flags": flags, "slot": slot, "n": len(samplers), "sampled": sampled_dev,
                               "index": {s.seq_id: i for i, s in enumerate(samplers)}})
        info.num_seqs, info.num_tokens = len(batch.seqs), batch.total_tokens
        self._stats.steps += 1
        self._stats.tokens_processed += batch.total_tokens
        if batch.blocked:
            self.sync(info)                                    # drain, so that the next schedule may preempt
        else:
            while len(self._inflight) >= self.config.pipeline_depth:
                self._retire_oldest(info)
        self._account(info, t0)
        return info

    def _step_native(self, info: StepInfo, t0: float) -> StepInfo:
        """The same step with the scheduler in C++: it hands out the step as arrays (which requests, where their tokens
        start, the tokens, which rows of the step in flight feed them, the sampling rows' options)."""
        b = self.scheduler.schedule(allow_preempt=not self._inflight)
        self._stats.preemptions = self.scheduler.num_preemptions
        self._stats.prefix_hit_pages = self.runner.cache.prefix_hits
        if not b.ids:
            if self._inflight:
                self.sync(info)
                self._account(info, t0)
                return info
            self._empty_steps += 1
            if self._empty_steps > 2:
                raise RuntimeError("the scheduler produced no work although requests are pending")
            return info
        self._empty_steps = 0
        prev = self._inflight[-1] if self._inflight else None
        entries, o = [], 0
        for rid, c, n, smp in zip(b.ids, b.starts, b.counts, b.samples):
            entries.append(StepEntry(rid, b.tokens[o:o + n], c, (n - 1,) if smp else ()))
            o += n
        feed = (prev["sampled"], b.feed_src) if b.need_feed else None
        logits = self.runner.step(entries, feed=feed)
        slot = self._slot
        self._slot ^= 1
        rows = len(b.temps)
        sampled_dev = self.sampler.sample_async(logits, b.temps, b.seeds, b.generated, slot=slot) if rows else None
        if self.scheduler.on_launched() != rows:
            raise RuntimeError("the scheduler and the step disagree on the sampling rows")
        self._inflight.append({"slot": slot, "n": rows, "sampled": sampled_dev})
        info.num_seqs, info.num_tokens = len(b.ids), b.total_tokens
        self._stats.steps += 1
        self._stats.tokens_processed += b.total_tokens
        if b.blocked:
            self.sync(info)
        else:
            while len(self._inflight) >= self.config.pipeline_depth:
                self._retire_oldest(info)
        self._account(info, t0)
        return info

    def _account(self, info: StepInfo, t0: float) -> None:
        self._stats.tokens_generated += info.num_sampled
        self._stats.seconds += time.perf_counter() - t0

    def _retire_oldest(self, info: StepInfo) -> None:
        rec = self._inflight.pop(0)
        tokens = self.sampler.collect(rec["n"], slot=rec["slot"]) if rec["n"] else []
        if self._native:
            finished = self.scheduler.postprocess(tokens)
            for rid in finished:
                d = self.scheduler.info(rid)
                toks = self.scheduler.tokens(rid)
                out = GenerationOutput(rid, toks[:d["num_prompt_tokens"]], toks[d["num_prompt_tokens"]:], d["stopped_on_eos"])
                if out.stopped_on_eos and out.token_ids:
                    out.token_ids.pop()                      # the end-of-sequence token itself is not returned
                self._finished[rid] = out
                self._live.pop(rid, None)
            # the library keeps a finished request while a step in flight still names it
            self._forget_later = [r for r in self._forget_later + finished if not self.scheduler.forget(r)]
            info.num_sampled += len(tokens)
            info.num_finished += len(finished)
            return
        finished = self.scheduler.postprocess(rec["batch"], rec["flags"], tokens)
        for seq in finished:
            self._harvest(seq)
        info.num_sampled += len(tokens)
        info.num_finished += len(finished)

    def sync(self, info: Optional[StepInfo] = None) -> None:
        """Read back every step that is still in flight."""
        info = info if info is not None else StepInfo()
        while self._inflight:
            self._retire_oldest(info)

    def _harvest(self, seq: Sequence) -> None:
        out = GenerationOutput(seq.seq_id, seq.token_ids[:seq.num_prompt_tokens], seq.token_ids[seq.num_prompt_tokens:],
                               seq.stopped_on_eos)
        if out.stopped_on_eos and out.token_ids:
            out.token_ids.pop()                              # the end-of-sequence token itself is not returned
        self._finished[seq.seq_id] = out
        self._live.pop(seq.seq_id, None)

    def take_finished(self) -> List[GenerationOutput]:
        outs = [self._finished[k] for k in sorted(self._finished)]
        self._finished.clear()
        return outs

    # ---- whole requests ---------------------------------------------------------------------------------
    def generate(self, prompts: Seq[Seq[int]], params: Union[SamplingParams, Seq[SamplingParams], None] = None) -> List[GenerationOutput]:
        if params is None or isinstance(params, SamplingParams):
            plist = [params or SamplingParams()] * len(prompts)
        else:
            plist = list(params)
            if len(plist) != len(prompts):
                raise ValueError("one SamplingParams per prompt is needed")
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        while not self.is_finished():
            self.step()
        self.sync()
        self.runner.check_errors()
        outs = []
        for rid in ids:
            if rid not in self._finished:
                raise RuntimeError(f"generate: request {rid} never finished")
            outs.append(self._finished.pop(rid))
        return outs


LLM = LLMEngine
