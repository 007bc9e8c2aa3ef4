"""Continuous batching above the step function: admission, prompt portions under a token budget, decoding,
finishing and freeing, and what happens when pages run out.

Policy after the reference's ``Scheduler`` (engine/scheduler.cpp):

* a step has a token budget ``max_num_batched_tokens``; a request gets ``min(tokens not yet in the cache, budget
  left, max_chunk_tokens)`` tokens (:43-44,68,99); ``max_chunk_tokens = 0`` means no cap; a prompt longer than
  that runs as portions over several steps and samples only in the step that ends with its last known token
  (scheduler.h:29-31);
* running requests come first, in order, decodes being portions of one token (:55-90); then waiting requests
  are admitted first-come-first-served while budget, ``max_num_seqs`` and pages allow; admission stops at the
  first request that does not fit, and no admission happens in a step that preempted (:91-100);
* admission reserves pages for the whole current sequence; before each later step the reservation is topped up
  to the sequence's length (engine/block_manager.cpp:80-126);
* pages run out: the request that cannot grow preempts the LAST running request that this step has not looked
  at yet, or itself if there is none (:74-85).  A preempted request gives back all pages and its state slot,
  keeps the tokens it has generated, and goes to the FRONT of the waiting queue; on re-admission its whole
  sequence is run again as a prompt (:28-34; engine/sequence.h:82-89);
* a request whose prompt plus ``max_tokens`` can never fit the pool, or exceeds ``max_model_len``, is refused at
  ``add_request`` (:18-26);
* a request finishes on an end-of-sequence token (unless ``ignore_eos``) or at ``max_tokens`` new tokens, and
  its pages are freed at once (:123-155);
* with the cache manager's prefix cache on, admission shares the pages of the longest registered prefix and the
  request starts behind them; after every step the full pages of its requests are registered (:94-96,133-150;
  engine/block_manager.cpp:71-143);
* with a step still in flight (the engine overlaps the host's work on step n + 1 with the device's work on step n,
  engine/llm_engine.cpp:70-113) a request's newest token is a placeholder whose value is handed over on the device;
  nothing is preempted while a step is in flight: a request that cannot grow is left out, the batch is marked
  ``blocked`` and the engine drains its pipeline before it schedules again (:74-85, llm_engine.cpp:106-107); a request
  that already has ``max_tokens`` tokens counting the placeholder is not scheduled again (:62-66).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, List, Optional, Sequence as Seq

from ..cache.manager import CacheManager
from ..sampling.params import SamplingParams

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"
PENDING = -1        # placeholder for a token that was sampled on the device but has not been read back yet
                    # (reference engine/sequence.h:16, kPendingToken)


class Sequence:
    """One request: its tokens (prompt, then generated), how many are in the cache, and its options."""
    __slots__ = ("seq_id", "token_ids", "num_prompt_tokens", "num_cached_tokens", "num_scheduled_tokens",
                 "params", "status", "stopped_on_eos", "row_seed", "num_preemptions", "num_inflight", "capacity")

    def __init__(self, seq_id: int, prompt: Seq[int], params: Optional[SamplingParams] = None):
        if len(prompt) == 0:
            raise ValueError("a request needs at least one prompt token")
        self.seq_id = seq_id
        self.token_ids: List[int] = [int(t) for t in prompt]
        self.num_prompt_tokens = len(self.token_ids)
        self.num_cached_tokens = 0
        self.num_scheduled_tokens = 0
        self.params = params or SamplingParams()
        self.status = WAITING
        self.stopped_on_eos = False
        self.row_seed = 0
        self.num_preemptions = 0
        self.num_inflight = 0
        self.capacity = 0            # tokens that the pages reserved for it cover (the scheduler's copy of the cache's answer)

    def __len__(self) -> int:
        return len(self.token_ids)

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def num_uncached_tokens(self) -> int:
        return len(self.token_ids) - self.num_cached_tokens

    def samples_this_step(self) -> bool:
        return self.num_cached_tokens + self.num_scheduled_tokens == len(self.token_ids)


@dataclass
class SchedulerConfig:
    max_num_batched_tokens: int = 4096
    max_num_seqs: int = 256
    max_chunk_tokens: int = 1024
    max_model_len: int = 4096
    eos_token_ids: tuple = ()


@dataclass
class ScheduledBatch:
    seqs: List[Sequence] = field(default_factory=list)
    total_tokens: int = 0
    preempted: List[Sequence] = field(default_factory=list)
    blocked: bool = False                      # a request could not grow and nothing may be preempted right now
    sample_pos: List[int] = field(default_factory=list)   # per sequence: index in token_ids of its placeholder, or -1

    @property
    def all_single_token(self) -> bool:
        return bool(self.seqs) and all(s.num_scheduled_tokens == 1 for s in self.seqs)


class Scheduler:
    def __init__(self, config: SchedulerConfig, cache: CacheManager):
        self.cfg = config
        self.cache = cache
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.num_preemptions = 0

    # ---- queue ---------------------------------------------------------------------------------------
    def add_request(self, seq: Sequence) -> None:
        max_len = seq.num_prompt_tokens + max(seq.params.max_tokens, 0)
        if max_len > self.cfg.max_model_len:
            raise ValueError(f"request needs {max_len} tokens (prompt {seq.num_prompt_tokens} + max_tokens "
                             f"{seq.params.max_tokens}) but max_model_len is {self.cfg.max_model_len}")
        need = self.cache.num_pages_for(max_len)
        smallest = min(p.num_pages for p in self.cache.pools) if self.cache.pools else need
        if need > smallest:
            raise ValueError(f"request needs {need} cache pages but the pool only has {smallest}")
        seq.status = WAITING
        self.waiting.append(seq)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def _preempt(self, seq: Sequence) -> None:
        self.cache.release(seq.seq_id)
        seq.status = WAITING
        seq.num_cached_tokens = 0
        seq.num_scheduled_tokens = 0
        seq.num_preemptions += 1
        seq.capacity = 0
        self.waiting.appendleft(seq)
        self.num_preemptions += 1

    # ---- one step's decisions --------------------------------------------------------------------------
    # Two passes, as in csrc/scheduler_runtime.cpp.  Pass 1 sees the running list through a window [i, live): request i
    # is served from the front; when its pages cannot grow, the request at the far end of the window gives up what it
    # holds and waits again (request i itself, once the window has shrunk onto it).  Pass 2 admits waiting requests first
    # come first served, unless the step took somebody out or was blocked.  Policy of the reference's
    # engine/scheduler.cpp:36-106, held to it by the golden batches.
    def schedule(self, allow_preempt: bool = True) -> ScheduledBatch:
        out = ScheduledBatch()
        self._tokens_left = self.cfg.max_num_batched_tokens
        self._took_out = False
        self._serve_running(out, allow_preempt)
        self._admit_waiting(out)
        return out

    def _portion(self, seq: Sequence) -> int:
        """How many of its tokens the request would run now: what it has not computed, cut to the cap and to the budget."""
        cap = self.cfg.max_chunk_tokens if self.cfg.max_chunk_tokens > 0 else 1 << 62
        return min(len(seq.token_ids) - seq.num_cached_tokens, cap, self._tokens_left)

    def _take(self, out: ScheduledBatch, seq: Sequence, n: int) -> None:
        seq.num_scheduled_tokens = n
        out.seqs.append(seq)
        out.total_tokens += n
        self._tokens_left -= n

    def _make_room(self, out: ScheduledBatch, i: int, live: int, allow_preempt: bool):
        """Pages for all tokens of running[i].  Returns (outcome, live) with outcome 'has' | 'blocked' | 'gave_way'."""
        seq = self.running[i]
        n_tok = len(seq.token_ids)
        if n_tok <= seq.capacity:                                  # most decode steps need no new page
            return "has", live
        while not self.cache.can_reserve(seq.seq_id, n_tok):
            if not allow_preempt:
                return "blocked", live
            live -= 1                                              # live >= i: at worst the request itself
            last = self.running[live]
            self._preempt(last)
            out.preempted.append(last)
            self._took_out = True
            if live == i:
                return "gave_way", live
        seq.capacity = self.cache.reserve(seq.seq_id, n_tok)
        return "has", live

    def _serve_running(self, out: ScheduledBatch, allow_preempt: bool) -> None:
        live, i = len(self.running), 0
        while i < live:
            seq = self.running[i]
            generated = len(seq.token_ids) - seq.num_prompt_tokens
            n = 0 if (generated > 0 and generated >= seq.params.max_tokens) else self._portion(seq)   # complete but for a token in flight
            if n > 0 and len(out.seqs) < self.cfg.max_num_seqs:
                outcome, live = self._make_room(out, i, live, allow_preempt)
                if outcome == "blocked":
                    out.blocked = True
                elif outcome == "has":
                    self._take(out, seq, n)
            i += 1
        del self.running[live:]

    def _admit_waiting(self, out: ScheduledBatch) -> None:
        if self._took_out or out.blocked:
            return
        while (self.waiting and self._tokens_left > 0 and len(self.running) < self.cfg.max_num_seqs
               and len(out.seqs) < self.cfg.max_num_seqs):
            seq = self.waiting[0]
            if not self.cache.can_admit(seq.token_ids, len(seq)):
                return                                             # first come first served: nobody overtakes
            self.waiting.popleft()
            lease = self.cache.admit(seq.seq_id, seq.token_ids)    # with the prefix cache: shared pages count as computed
            seq.num_cached_tokens = lease.computed
            seq.capacity = self.cache.reserve(seq.seq_id, len(seq))
            seq.status = RUNNING
            self.running.append(seq)
            self._take(out, seq, self._portion(seq))

    # ---- after the step ----------------------------------------------------------------------------------
    def on_launched(self, batch: ScheduledBatch) -> List[bool]:
        """The step was handed to the device: its tokens count as cached, and every sequence that samples in it gets a
        placeholder for the token that is not known on the host yet.  Returns, per sequence, whether it samples."""
        sampled = []
        batch.sample_pos = []
        for seq in batch.seqs:
            samples = seq.samples_this_step()
            sampled.append(samples)
            seq.num_cached_tokens += seq.num_scheduled_tokens
            seq.num_scheduled_tokens = 0
            seq.num_inflight += 1
            if samples:
                batch.sample_pos.append(len(seq.token_ids))
                seq.token_ids.append(PENDING)
            else:
                batch.sample_pos.append(-1)
        return sampled

    def postprocess(self, batch: ScheduledBatch, sampled_flags: List[bool], tokens: List[int]) -> List[Sequence]:
        """The step's samples arrived (`tokens`: one per sampling sequence, in batch order): they replace the
        placeholders; requests finish and give back what they hold.  Results for a request that finished in an earlier
        step while this one was in flight are dropped.  Returns the sequences that finished."""
        finished = []
        it = iter(tokens)
        for seq, did, pos in zip(batch.seqs, sampled_flags, batch.sample_pos):
            seq.num_inflight -= 1
            if not did:
                if seq.status != FINISHED:
                    self.cache.commit(seq.seq_id, seq.token_ids)  # full pages of a prompt portion become shareable
                continue
            tok = int(next(it))
            if seq.status == FINISHED:
                continue
            seq.token_ids[pos] = tok
            hit_eos = (not seq.params.ignore_eos) and tok in self.cfg.eos_token_ids
            hit_len = pos + 1 - seq.num_prompt_tokens >= seq.params.max_tokens
            if hit_eos or hit_len:
                del seq.token_ids[pos + 1:]               # a placeholder of a later step that is still in flight
                seq.num_cached_tokens = min(seq.num_cached_tokens, len(seq.token_ids))
                seq.stopped_on_eos = hit_eos
                seq.status = FINISHED
                self.cache.commit(seq.seq_id, seq.token_ids)
                self.cache.release(seq.seq_id)
                finished.append(seq)
            else:
                self.cache.commit(seq.seq_id, seq.token_ids)
        if finished:
            self.running = [s for s in self.running if s.status != FINISHED]
        return finished
