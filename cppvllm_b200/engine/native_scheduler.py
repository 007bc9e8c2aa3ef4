"""The scheduler in C++ (csrc/scheduler_runtime.cpp) as the engine uses it.

The library keeps the requests (tokens, counters, state), decides every step and calls the cache manager in C++
directly; this wrapper passes arrays in and out and keeps the cache manager's Python view of the live requests
(request id -> lease) in step with what the library admitted and released.  The decisions are those of
engine/scheduler.py (the plain twin); tests run both on the same workloads and compare every batch.
"""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_float, c_int, c_longlong, c_ulonglong, c_void_p
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

from ..cache.native import NativeCacheManager, _library
from ..sampling.params import SamplingParams
from .scheduler import SchedulerConfig

_bound = False


def _lib():
    global _bound
    lib = _library()
    if not _bound:
        lib.cvb_sched_create.restype = c_void_p
        lib.cvb_sched_create.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, POINTER(c_int), c_int]
        lib.cvb_sched_destroy.argtypes = [c_void_p]
        lib.cvb_sched_add.argtypes = [c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_float, c_ulonglong]
        for name in ("cvb_sched_is_finished", "cvb_sched_num_waiting", "cvb_sched_num_running", "cvb_sched_num_inflight",
                     "cvb_sched_on_launched"):
            getattr(lib, name).argtypes = [c_void_p]
        lib.cvb_sched_num_preemptions.restype = c_longlong
        lib.cvb_sched_num_preemptions.argtypes = [c_void_p]
        lib.cvb_sched_queue.argtypes = [c_void_p, c_int, c_void_p, c_int]
        lib.cvb_sched_schedule.argtypes = [c_void_p, c_int, c_void_p]
        lib.cvb_sched_batch.argtypes = [c_void_p] + [c_void_p] * 11 + [POINTER(c_int)]
        lib.cvb_sched_postprocess.argtypes = [c_void_p, c_void_p, c_int, c_void_p, c_int]
        lib.cvb_sched_seq_info.argtypes = [c_void_p, c_int, c_void_p]
        lib.cvb_sched_seq_tokens.argtypes = [c_void_p, c_int, c_void_p, c_int]
        lib.cvb_sched_forget.argtypes = [c_void_p, c_int]
        _bound = True
    return lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(c_void_p)


@dataclass
class NativeBatch:
    """One step as the library decided it.  Arrays are copies (the next call may overwrite the library's buffers)."""
    ids: List[int] = field(default_factory=list)
    starts: List[int] = field(default_factory=list)          # tokens of the request that are in the cache already
    counts: List[int] = field(default_factory=list)          # tokens of the request that run in this step
    samples: List[bool] = field(default_factory=list)        # whether the step samples the request's next token
    tokens: Optional[np.ndarray] = None                      # all tokens of the step, flat (0 where fed on the device)
    feed_src: Optional[np.ndarray] = None                    # per token: row of the step in flight that feeds it, or -1
    need_feed: bool = False
    temps: List[float] = field(default_factory=list)         # per sampling row
    seeds: List[int] = field(default_factory=list)
    generated: List[int] = field(default_factory=list)       # tokens generated so far (the sample's output position)
    preempted: List[int] = field(default_factory=list)
    total_tokens: int = 0
    blocked: bool = False


class NativeScheduler:
    native = True

    def __init__(self, config: SchedulerConfig, cache: NativeCacheManager):
        if not getattr(cache, "native", False):
            raise TypeError("the scheduler in C++ needs the cache manager in C++")
        self.cfg, self.cache = config, cache
        self._l = _lib()
        eos = [int(t) for t in config.eos_token_ids]
        arr = (c_int * max(1, len(eos)))(*eos)
        smallest = min(p.num_pages for p in cache.pools)
        self._h = c_void_p(self._l.cvb_sched_create(cache._h, config.max_num_batched_tokens, config.max_num_seqs,
                                                    config.max_chunk_tokens, config.max_model_len, cache.page_size,
                                                    smallest, arr, len(eos)))
        if not self._h:
            raise ValueError("the scheduler could not be created from these sizes")
        self._smallest = smallest
        S, T = config.max_num_seqs, config.max_num_batched_tokens
        i32 = np.int32
        self._info = np.zeros(8, i32)
        self._ids, self._slots, self._starts, self._counts, self._samples = (np.zeros(S, i32) for _ in range(5))
        self._tokens, self._feed = np.zeros(T, i32), np.zeros(T, i32)
        self._temps, self._seeds, self._generated = np.zeros(S, np.float32), np.zeros(S, np.uint64), np.zeros(S, i32)
        self._lists = np.zeros(3 * S + 8, i32)
        self._finished = np.zeros(S + 8, i32)
        self._need_feed = c_int(0)
        self._seq = np.zeros(16, i32)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._l.cvb_sched_destroy(h)

    # ---- queue -------------------------------------------------------------------------------------------
    def add_request(self, request_id: int, prompt: Sequence[int], params: SamplingParams, row_seed: int) -> None:
        toks = np.asarray([int(t) for t in prompt], dtype=np.int32)
        rc = int(self._l.cvb_sched_add(self._h, int(request_id), _p(toks), int(toks.shape[0]), int(params.max_tokens),
                                       1 if params.ignore_eos else 0, float(params.temperature),
                                       int(row_seed) & 0xffffffffffffffff))
        if rc == -1:
            raise ValueError("a request needs at least one prompt token")
        if rc == -2:
            raise ValueError(f"request needs {len(toks) + max(params.max_tokens, 0)} tokens (prompt {len(toks)} + max_tokens "
                             f"{params.max_tokens}) but max_model_len is {self.cfg.max_model_len}")
        if rc == -3:
            need = self.cache.num_pages_for(len(toks) + max(params.max_tokens, 0))
            raise ValueError(f"request needs {need} cache pages but the pool only has {self._smallest}")
        if rc != 0:
            raise ValueError(f"request id {request_id} is in use")

    def is_finished(self) -> bool:
        return bool(self._l.cvb_sched_is_finished(self._h))

    @property
    def num_preemptions(self) -> int:
        return int(self._l.cvb_sched_num_preemptions(self._h))

    @property
    def num_inflight(self) -> int:
        return int(self._l.cvb_sched_num_inflight(self._h))

    def _queue(self, which: int) -> List[int]:
        n = int(self._l.cvb_sched_num_waiting(self._h) if which == 0 else self._l.cvb_sched_num_running(self._h))
        out = np.zeros(max(1, n), np.int32)
        n = int(self._l.cvb_sched_queue(self._h, which, _p(out), n))
        return out[:n].tolist()

    @property
    def waiting(self) -> List[int]:
        return self._queue(0)

    @property
    def running(self) -> List[int]:
        return self._queue(1)

    # ---- one step ----------------------------------------------------------------------------------------
    def schedule(self, allow_preempt: bool = True) -> NativeBatch:
        n = int(self._l.cvb_sched_schedule(self._h, 1 if allow_preempt else 0, _p(self._info)))
        total, blocked, n_pre, n_adm = (int(x) for x in self._info[1:5])
        rows = int(self._l.cvb_sched_batch(self._h, _p(self._ids), _p(self._slots), _p(self._starts), _p(self._counts),
                                           _p(self._samples), _p(self._tokens), _p(self._feed), _p(self._temps),
                                           _p(self._seeds), _p(self._generated), _p(self._lists),
                                           ctypes.byref(self._need_feed)))
        lists = self._lists[:n_pre + 2 * n_adm].tolist()
        preempted, admitted = lists[:n_pre], lists[n_pre:]
        for rid in preempted:                                  # the library released them
            self.cache.drop(rid)
        for k in range(0, len(admitted), 2):                   # and admitted these
            self.cache.adopt(admitted[k], admitted[k + 1])
        return NativeBatch(
            ids=self._ids[:n].tolist(), starts=self._starts[:n].tolist(), counts=self._counts[:n].tolist(),
            samples=[bool(x) for x in self._samples[:n].tolist()], tokens=self._tokens[:total].copy(),
            feed_src=self._feed[:total].copy(), need_feed=bool(self._need_feed.value), temps=self._temps[:rows].tolist(),
            seeds=self._seeds[:rows].tolist(), generated=self._generated[:rows].tolist(), preempted=preempted,
            total_tokens=total, blocked=bool(blocked))

    def on_launched(self) -> int:
        """The batch of the last schedule() was handed to the device; returns its number of sampling rows."""
        return int(self._l.cvb_sched_on_launched(self._h))

    def postprocess(self, tokens: Sequence[int]) -> List[int]:
        """The samples of the oldest step in flight; returns the ids of the requests that finished."""
        arr = np.asarray(list(tokens), dtype=np.int32) if len(tokens) else np.zeros(1, np.int32)
        n = int(self._l.cvb_sched_postprocess(self._h, _p(arr), len(tokens), _p(self._finished), int(self._finished.shape[0])))
        if n < 0:
            raise RuntimeError("postprocess: no step is in flight, or it sampled more rows than tokens were given")
        done = self._finished[:n].tolist()
        for rid in done:
            self.cache.drop(rid)
        return done

    # ---- requests ------------------------------------------------------------------------------------------
    def info(self, request_id: int) -> dict:
        if int(self._l.cvb_sched_seq_info(self._h, int(request_id), _p(self._seq))) != 0:
            raise KeyError(request_id)
        names = ("status", "num_prompt_tokens", "num_tokens", "num_cached_tokens", "num_scheduled_tokens", "num_preemptions",
                 "num_inflight", "stopped_on_eos", "state_slot")
        d = dict(zip(names, (int(x) for x in self._seq[:9])))
        d["status"] = ("waiting", "running", "finished")[d["status"]]
        d["stopped_on_eos"] = bool(d["stopped_on_eos"])
        return d

    def tokens(self, request_id: int) -> List[int]:
        n = int(self._l.cvb_sched_seq_tokens(self._h, int(request_id), _p(self._seq), 0))
        if n < 0:
            raise KeyError(request_id)
        out = np.zeros(max(1, n), np.int32)
        self._l.cvb_sched_seq_tokens(self._h, int(request_id), _p(out), n)
        return out[:n].tolist()

    def forget(self, request_id: int) -> bool:
        """Drop a finished request whose result was taken; False while a step in flight still names it."""
        return int(self._l.cvb_sched_forget(self._h, int(request_id))) == 0
