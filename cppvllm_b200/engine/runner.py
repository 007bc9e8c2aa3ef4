"""The step function: one flattened batch of (request, its next tokens) through the model, from the cache.

``ModelRunner`` owns the model, the device storage of the cache (pages per group, state tensors per slot), the
host-side ``CacheManager`` and the staging buffers.  ``step(entries)`` takes any mix of prompt portions and single
decoded tokens, cut anywhere, runs exactly those tokens as ONE forward pass (the reference runs up to three
separate passes per step, engine/model_runner.cpp:181-196), and returns float32 logits for the wanted tokens.

Per step the host fills one pinned int32 staging block (tokens, positions, request index per token, cumulative
lengths, lengths after the step, state slots, wanted rows and, per cache group, the slot of every token and
the block tables; the reference stages the same arrays, model_runner.cpp:290-320, but derives slots on the
device, model_architecture.cpp:137-141) and copies it with one asynchronous transfer.  Steps that consist only
of single decoded tokens replay a CUDA graph captured per batch-size bucket (reference model_runner.cpp:371-428);
rows that pad a bucket read and write a scratch page that no request owns (model_runner.cpp:69,329,346).
Other steps (prompt portions, mixed batches) are launched kernel by kernel the first time their shape (the tuple of
portion lengths and the number of wanted rows) occurs; the second time the shape is captured into a graph of its
own and replayed from then on: the launches of a long prompt cut into equal portions, or of a stream of equal
prompts, then cost the host one call instead of some hundred.
"""
from __future__ import annotations

import os
import sys
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, GroupConfig
from ..cache.native import NativeCacheManager
from ..config.model_config import read_config_json
from ..config.registry import resolve_architecture
from ..csrc import ops
from ..parts.base import Runtime, Workspace
from ..parts.context import CacheUnitView, GroupStepView, StepContext
from ..parts.model import CausalLM
from ..weights.loader import load_weights
from .. import models as _models  # noqa: F401  (registers the architectures)
from .. import parts as _parts  # noqa: F401


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, the absolute position of the first of them, and the
    indices (within these tokens) at which logits are wanted."""
    request_id: object
    tokens: Sequence[int]
    start: int
    want: Sequence[int] = ()


def _align(n: int, a: int = 4) -> int:
    return (n + a - 1) // a * a


GRAPH_BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
SHAPE_GRAPHS = 16             # graphs kept for steps that are not decode-only, least recently used first out
SHAPE_GRAPH_MIN_TOKENS = 64   # shorter steps are cheap to launch and come in too many shapes


class ModelRunner:
    def __init__(self, model_dir: str, dtype=torch.bfloat16, device="cuda:0", page_size: int = 32,
                 num_pages: Optional[int] = None, max_step_tokens: int = 4096, max_seqs: int = 256,
                 max_model_len: int = 4096, gpu_memory_utilization: float = 0.90, enforce_eager: bool = False,
                 num_state_slots: Optional[int] = None, enable_prefix_caching: bool = False, use_ref_kernels: bool = False,
                 native_cache_manager: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("cppvllm_b200 runs on a CUDA device only; torch.cuda.is_available() is False")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        ops.configure_library_matmul()
        ops.core()                                           # compile/load the kernels now; fails loudly
        self.dtype = dtype
        self.page_size = page_size
        self.max_step_tokens = int(max_step_tokens)
        self.max_seqs = int(max_seqs)
        self.enforce_eager = enforce_eager

        cfg_dict = read_config_json(model_dir)
        self.arch = resolve_architecture(cfg_dict)
        self.config = self.arch.parse_config(cfg_dict)
        spec = self.arch.build_spec(self.config)
        self.max_model_len = int(min(max_model_len, spec.max_positions) if spec.max_positions else max_model_len)
        self.workspace = Workspace(self.device, self.max_step_tokens, self.max_seqs)
        self.rt = Runtime(self.device, dtype, self.workspace, plain_kernels=bool(use_ref_kernels))
        self.model = CausalLM(spec, self.rt)
        self.model.bind(load_weights(self.model, model_dir, self.device, dtype))
        self.vocab_size = self.model.vocab_size

        # ---- cache groups: units with equal needs share a pool of pages -----------------------------------
        units = self.model.cache_units()                      # unit id -> CacheSpec
        self.group_specs = []
        self.unit_location: Dict[int, tuple] = {}             # unit id -> (group, index in group)
        for uid in sorted(units):
            cs = units[uid]
            for g, (gs, members) in enumerate(self.group_specs):
                if gs == cs:
                    self.unit_location[uid] = (g, len(members))
                    members.append(uid)
                    break
            else:
                self.unit_location[uid] = (len(self.group_specs), 0)
                self.group_specs.append((cs, [uid]))
        elem = torch.empty((), dtype=dtype).element_size()
        self.page_bytes = [len(m) * cs.elements_per_token() * page_size * elem for cs, m in self.group_specs]
        self.table_width = (self.max_model_len + page_size - 1) // page_size
        if num_pages is None:
            num_pages = self._pages_from_free_memory(gpu_memory_utilization)
        self.num_pages = int(num_pages)
        self.storage = [torch.zeros((len(m), self.num_pages + 1) + cs.page_shape(page_size), dtype=dtype, device=self.device)
                        for cs, m in self.group_specs]
        self.scratch_page = self.num_pages                    # the extra page: padding rows of captured graphs
        n_slots = int(num_state_slots if num_state_slots is not None else max_seqs)
        self.state_specs = self.model.state_specs()
        if enable_prefix_caching and (len(self.group_specs) != 1 or self.group_specs[0][0].window > 0
                                      or any(ss is not None for ss in self.state_specs)):
            print("[cppvllm_b200] the prefix cache is off: it needs one group of cache units that keeps all keys and "
                  "no per-request state", file=sys.stderr, flush=True)
            enable_prefix_caching = False
        groups = [GroupConfig(self.num_pages, cs.window, tuple(m)) for cs, m in self.group_specs]
        if native_cache_manager and groups:
            # the C++ manager keeps the block tables as dense arrays that the steps read in place
            self.cache = NativeCacheManager(groups, page_size, n_slots, self.table_width, prefix_caching=enable_prefix_caching)
        else:
            self.cache = CacheManager(groups, page_size, n_slots, prefix_caching=enable_prefix_caching)
        self.scratch_slot = n_slots
        self.states = {i: torch.zeros((n_slots + 1,) + tuple(ss.shape), dtype=ss.dtype, device=self.device)
                       for i, ss in enumerate(self.state_specs) if ss is not None}
        self.cache_views: Dict[int, CacheUnitView] = {}
        for i, e in enumerate(self.model.run_order):
            cs = self.model.blocks[e.layer].mixer.cache_spec()
            if cs is None:
                continue
            g, idx = self.unit_location[e.cache]
            self.cache_views[i] = CacheUnitView(self.storage[g][idx], g, cs, e.writes_cache)

        # ---- staging ----------------------------------------------------------------------------------
        G = max(1, len(self.group_specs))
        cap = (5 * _align(self.max_step_tokens) + 3 * _align(self.max_seqs + 1)
               + G * (_align(self.max_step_tokens) + _align(self.max_seqs * self.table_width)) + 64)
        self._stage_capacity = cap
        self._stage_host = [torch.empty(cap, dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._stage_np = [t.numpy() for t in self._stage_host]
        self._stage_events = [None] * 4
        self._stage_turn = 0
        self._stage_dev = torch.zeros(cap, dtype=torch.int32, device=self.device)
        self._logits = torch.empty((self.max_seqs, self.vocab_size), dtype=torch.float32, device=self.device)
        self._graphs: Dict[int, tuple] = {}
        self._graph_launches: Dict[int, int] = {}
        if getattr(self.cache, "native", False):
            self._tab_mirror = list(self.cache.tables)        # the manager's own arrays: nothing to mirror
        else:
            self._tab_mirror = [np.full((n_slots + 1, self.table_width), -1, dtype=np.int32) for _ in self.group_specs]
        self._mirror_owner = [[None] * (n_slots + 1) for _ in self.group_specs]
        self._mirror_len = [[0] * (n_slots + 1) for _ in self.group_specs]
        self._shape_graphs: "OrderedDict[tuple, tuple]" = OrderedDict()
        self._shape_seen: Dict[tuple, int] = {}
        self._feed = None
        self.h2d_bytes_last_step = 0
        self.stats = {"steps": 0, "graph_steps": 0, "tokens": 0}

    # ---- sizing -----------------------------------------------------------------------------------------
    def _pages_from_free_memory(self, utilization: float) -> int:
        """Pages that fit into `utilization` of the device after weights and a reserve for activations
        (the reference sizes its pool the same way from cudaMemGetInfo, engine/model_runner.cpp:116-145)."""
        torch.cuda.synchronize(self.device)
        free_b, total_b = torch.cuda.mem_get_info(self.device)
        used = total_b - free_b
        cfg = self.model
        act_reserve = self.max_step_tokens * (16 * cfg.hidden_size) * 4 + self.max_seqs * cfg.vocab_size * 4 * 2 + (1 << 30)
        budget = total_b * utilization - used - act_reserve
        per_page = sum(self.page_bytes) or 1
        n = int(budget // per_page)
        if n <= 0:
            raise RuntimeError("no memory is left for cache pages: lower max_num_batched_tokens or raise gpu_memory_utilization")
        # no request can use more than max_model_len tokens; cap the pool where more would never be used
        return min(n, self.max_seqs * self.table_width)

    def kv_bytes_per_token(self) -> int:
        return sum(pb // self.page_size for pb in self.page_bytes)

    # ---- staging ----------------------------------------------------------------------------------------
    def _layout(self, T: int, S: int, R: int, W: int):
        off, lay = 0, {}
        for name, n in (("tokens", T), ("positions", T), ("seq_of_token", T), ("logit_rows", max(R, 1)),
                        ("cu_seqlens", S + 1), ("kv_lens", S), ("state_slots", S)):
            lay[name] = (off, n)
            off += _align(n)
        lay["feed_src"] = (off, T)
        off += _align(T)
        for g in range(len(self.group_specs)):
            lay[f"slots{g}"] = (off, T)
            off += _align(T)
            lay[f"tables{g}"] = (off, S * W)
            off += _align(S * W)
        lay["_end"] = (off, 0)
        if off > self._stage_capacity:
            raise ValueError("the step's index arrays exceed the staging buffer")
        return lay

    def _next_stage(self):
        i = self._stage_turn
        self._stage_turn = (i + 1) % len(self._stage_host)
        ev = self._stage_events[i]
        if ev is not None:
            ev.synchronize()                                  # the copy that last read this buffer is done
        return i, self._stage_np[i]

    def _mirror_row(self, lease, W: int) -> int:
        """Block tables are mirrored on the host as integer arrays, one row per state slot, and brought up to date only
        where a request's table has grown: a step then copies whole rows instead of converting every list again.
        Returns the row of `lease`."""
        row = lease.state_slot
        if getattr(self.cache, "native", False):
            return row                                        # a row of the manager's dense table (never wider than W)
        for g in range(len(self.group_specs)):
            tab = lease.tables[g]
            n = len(tab)
            if n > W:
                raise ValueError("a request's block table is wider than the staged width")
            mirror = self._tab_mirror[g]
            if self._mirror_owner[g][row] is not lease:
                mirror[row, :] = -1
                self._mirror_owner[g][row] = lease
                self._mirror_len[g][row] = 0
            have = self._mirror_len[g][row]
            if self.group_specs[g][0].window > 0:
                have = 0                                      # a windowed group also gives pages back: copy the whole row
            if have < n:
                mirror[row, have:n] = tab[have:n]
                self._mirror_len[g][row] = n
        return row

    def _fill(self, entries: Sequence[StepEntry], T: int, S: int, R: int, W: int, pad_to: int = 0):
        """Write the step's index arrays into a pinned buffer and start its copy to the device."""
        S_pad = max(S, pad_to)
        T_pad = T + (S_pad - S)
        R_pad = R + (S_pad - S) if pad_to else R
        lay = self._layout(T_pad, S_pad, R_pad, W)
        idx, buf = self._next_stage()
        ps = self.page_size

        def reg(name):
            o, n = lay[name]
            return buf[o:o + n]

        tokens, positions, seq_of = reg("tokens"), reg("positions"), reg("seq_of_token")
        cu, kvl, sts, rows = reg("cu_seqlens"), reg("kv_lens"), reg("state_slots"), reg("logit_rows")
        slots = [reg(f"slots{g}") for g in range(len(self.group_specs))]
        tables = [reg(f"tables{g}").reshape(S_pad, W) for g in range(len(self.group_specs))]
        for tb in tables:
            tb.fill(-1)
        t = r = 0
        cu[0] = 0
        G = len(self.group_specs)
        mirror_rows = []
        decode_only = bool(entries) and T == S and R == S and all(len(e.want) == 1 for e in entries)
        if decode_only:
            # decoded tokens only, each with its logits wanted: the arrays are filled whole instead of entry by entry
            leases = [self.cache.lease(e.request_id) for e in entries]
            mirror_rows = [self._mirror_row(lease, W) for lease in leases]
            starts = np.fromiter((e.start for e in entries), dtype=np.int32, count=S)
            ar = np.arange(S, dtype=np.int32)
            tokens[:S] = [e.tokens[0] for e in entries]
            positions[:S] = starts
            seq_of[:S] = ar
            rows[:S] = ar
            cu[1:S + 1] = ar + 1
            kvl[:S] = starts + 1
            sts[:S] = mirror_rows                              # a request's mirror row is its state slot
            page_idx = starts // ps
            if (page_idx >= W).any():
                raise RuntimeError("pages for a decoded token's position were not reserved")
            idx_rows = np.asarray(mirror_rows, dtype=np.int64)
            for g in range(G):
                tables[g][:S, :] = self._tab_mirror[g][idx_rows, :W]
                page = tables[g][ar, page_idx]
                if (page < 0).any():
                    bad = entries[int(np.argmax(page < 0))]
                    raise RuntimeError(f"request {bad.request_id!r}: a token of this step has no page in group {g}")
                slots[g][:S] = page * ps + starts % ps
            t = r = S
        for s, e in enumerate(() if decode_only else entries):
            n = len(e.tokens)
            lease = self.cache.lease(e.request_id)
            start = e.start
            cu[s + 1] = t + n
            kvl[s] = start + n
            sts[s] = lease.state_slot
            mirror_rows.append(self._mirror_row(lease, W))
            if n == 1:                                        # a decoded token: plain integers instead of arrays
                tokens[t] = e.tokens[0]
                positions[t] = start
                seq_of[t] = s
                for w in e.want:
                    rows[r] = t + w
                    r += 1
                for g in range(G):
                    tab = lease.tables[g]
                    i = start // ps
                    if i >= len(tab):
                        raise RuntimeError(f"request {e.request_id!r}: pages for positions up to {start} were "
                                           f"not reserved in group {g}")
                    page = tab[i]
                    if page < 0:
                        raise RuntimeError(f"request {e.request_id!r}: a token of this step has no page in group {g}")
                    slots[g][t] = page * ps + start % ps
                t += 1
                continue
            tokens[t:t + n] = e.tokens
            positions[t:t + n] = np.arange(start, start + n, dtype=np.int32)
            seq_of[t:t + n] = s
            for w in e.want:
                rows[r] = t + w
                r += 1
            for g in range(G):
                tab = lease.tables[g]
                if start + n > len(tab) * ps:
                    raise RuntimeError(f"request {e.request_id!r}: pages for positions up to {start + n - 1} were "
                                       f"not reserved in group {g}")
                pos = positions[t:t + n]
                page_of = np.asarray(tab, dtype=np.int32)[pos // ps]
                if (page_of < 0).any():
                    raise RuntimeError(f"request {e.request_id!r}: a token of this step has no page in group {g}")
                slots[g][t:t + n] = page_of * ps + pos % ps
            t += n
        if entries and not decode_only:
            idx_rows = np.asarray(mirror_rows, dtype=np.int64)
            for g in range(G):
                tables[g][:S, :] = self._tab_mirror[g][idx_rows, :W]
        for s in range(S, S_pad):                             # padding rows of a captured graph
            tokens[t] = 0
            positions[t] = 0
            seq_of[t] = s
            cu[s + 1] = t + 1
            kvl[s] = 1
            sts[s] = self.scratch_slot
            rows[r] = t
            r += 1
            for g in range(len(self.group_specs)):
                tables[g][s, 0] = self.scratch_page
                slots[g][t] = self.scratch_page * ps
            t += 1
        if R == 0 and not pad_to:
            rows[0] = 0
        end = lay["_end"][0]
        feed = getattr(self, "_feed", None)
        if feed is not None and entries:
            o, n = lay["feed_src"]
            src = buf[o:o + n]
            src[:] = -1
            src[:len(feed[1])] = feed[1]
        self._stage_dev[:end].copy_(self._stage_host[idx][:end], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self._stage_events[idx] = ev
        self.h2d_bytes_last_step = end * 4
        if feed is not None and entries:
            o, n = lay["tokens"]
            fo, _ = lay["feed_src"]
            ops.feed_tokens(self._stage_dev[o:o + n], self._stage_dev[fo:fo + n], feed[0], T)
        return lay, T_pad, S_pad, R_pad

    def _context(self, lay, T: int, S: int, R: int, W: int, q_lens, max_kv: int) -> StepContext:
        d = self._stage_dev

        def reg(name):
            o, n = lay[name]
            return d[o:o + n]

        groups = []
        for g in range(len(self.group_specs)):
            groups.append(GroupStepView(reg(f"tables{g}").view(S, W), reg(f"slots{g}"), self.page_size, self.num_pages + 1))
        return StepContext(
            num_tokens=T, num_seqs=S, tokens=reg("tokens"), positions=reg("positions"), seq_of_token=reg("seq_of_token"),
            cu_seqlens=reg("cu_seqlens"), kv_lens=reg("kv_lens"), state_slots=reg("state_slots"), groups=groups,
            logit_rows=reg("logit_rows"), num_logit_rows=R, q_lens=q_lens, max_q_len=max(q_lens) if q_lens else 1,
            max_kv_len=max_kv, all_decode=all(q == 1 for q in q_lens) if q_lens else True)

    # ---- the step ---------------------------------------------------------------------------------------
    def _validate(self, entries: Sequence[StepEntry]) -> None:
        seen = set()
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} occurs twice in one step")
            seen.add(e.request_id)
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request_id!r} brings no tokens")
            lease = self.cache.lease(e.request_id)
            if e.start != lease.computed:
                raise ValueError(f"request {e.request_id!r}: step starts at position {e.start} but {lease.computed} "
                                 "tokens are in the cache")
            if e.start + n > self.max_model_len:
                raise ValueError(f"request {e.request_id!r} would reach {e.start + n} tokens; max_model_len is {self.max_model_len}")
            for w in e.want:
                if not (0 <= w < n):
                    raise ValueError(f"request {e.request_id!r}: wanted index {w} outside its {n} tokens")

    def step(self, entries: Sequence[StepEntry], feed=None) -> torch.Tensor:
        """Run one step.  Pages for every entry's tokens must have been reserved with ``cache.reserve``.
        Returns float32 logits [R, vocab] on the device, rows in the order of the entries and of their ``want``;
        the tensor is valid until the next step.

        ``feed = (sampled, src)`` hands tokens over on the device: ``sampled`` is an int32 device tensor (the
        previous step's samples, possibly still being computed) and ``src`` a list with one entry per token of
        this step, the index into ``sampled`` whose value replaces that token, or -1 to keep the given one
        (reference engine/model_runner.cpp:266-275, 299-303)."""
        entries = list(entries)
        if not entries:
            raise ValueError("a step needs at least one entry")
        self._validate(entries)
        q_lens = [len(e.tokens) for e in entries]
        T, S = sum(q_lens), len(entries)
        R = sum(len(e.want) for e in entries)
        if T > self.max_step_tokens:
            raise ValueError(f"a step of {T} tokens exceeds max_num_batched_tokens = {self.max_step_tokens}")
        if S > self.max_seqs:
            raise ValueError(f"a step of {S} requests exceeds max_num_seqs = {self.max_seqs}")
        fresh = self.cache.take_fresh_slots()
        if fresh and self.states:
            idx = torch.tensor(fresh, dtype=torch.long, device=self.device)
            for st in self.states.values():
                st.index_fill_(0, idx, 0)
        max_kv = max(e.start + len(e.tokens) for e in entries)

        self._feed = feed
        logits = None
        if (not self.enforce_eager and self.model.capturable and T == S and self._bucket(S)
                and all(len(e.want) == 1 for e in entries)):
            logits = self._step_graph(entries, S, max_kv)
        if (logits is None and not self.enforce_eager and self.model.capturable and T >= SHAPE_GRAPH_MIN_TOKENS
                and R <= self._logits.shape[0]):
            logits = self._step_shape_graph(entries, q_lens, T, S, R)
        if logits is None:
            W = max(1, max(len(self.cache.lease(e.request_id).tables[g]) for e in entries
                           for g in range(len(self.group_specs))) if self.group_specs else 1)
            lay, T_, S_, R_ = self._fill(entries, T, S, R, W)
            ctx = self._context(lay, T, S, R, W, q_lens, max_kv)
            out = self._logits if R <= self._logits.shape[0] else torch.empty(
                (R, self.vocab_size), dtype=torch.float32, device=self.device)
            logits = self.model.forward(ctx, self.cache_views, self.states, out)[:R] if R > 0 else \
                self._forward_no_logits(ctx)
        self._advance(entries)
        self.stats["steps"] += 1
        self.stats["tokens"] += T
        return logits

    def _advance(self, entries: Sequence[StepEntry]) -> None:
        """The step's tokens are in the cache now (windowed groups give pages back)."""
        many = getattr(self.cache, "advance_many", None)
        if many is not None:
            many([e.request_id for e in entries], [e.start + len(e.tokens) for e in entries])
        else:
            for e in entries:
                self.cache.advance(e.request_id, e.start + len(e.tokens))

    def _forward_no_logits(self, ctx) -> torch.Tensor:
        self.model.forward_hidden(ctx, self.cache_views, self.states)
        return self._logits[:0]

    # ---- CUDA graphs for decode-only steps -------------------------------------------------------------
    def _bucket(self, S: int) -> int:
        """The smallest captured batch size that holds S rows; 0 if S is beyond the largest bucket."""
        for b in GRAPH_BUCKETS:
            if b >= S:
                return min(b, max(self.max_seqs, S))
        return 0

    def _capture(self, B: int) -> bool:
        """Capture the graph of a decode-only step of B rows.  Warm-up and capture run on padding rows only (they
        read and write the scratch page and the scratch state slot), so no request's cache or state is touched
        before the real replay.  Returns False, and switches graphs off, if the model cannot be captured."""
        W = self.table_width
        lay, _, _, _ = self._fill([], 0, 0, 0, W, pad_to=B)
        ctx = self._context(lay, B, B, B, W, [1] * B, self.max_model_len)
        ctx.extras["captured"] = True
        try:
            # lazy initialisation (cuBLAS handles, kernel loading, workspace buffers) must happen outside capture
            self.model.forward(ctx, self.cache_views, self.states, self._logits)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = ops.launches()
            with torch.cuda.graph(graph):
                self.model.forward(ctx, self.cache_views, self.states, self._logits)
            self._graph_launches[B] = ops.launches() - before
            ops.LAUNCHES = before                             # recorded, not run: replays count them
        except Exception as ex:                               # a part that synchronises or allocates on the host
            torch.cuda.synchronize(self.device)
            self.enforce_eager = True
            print(f"[cppvllm_b200] decode steps cannot be captured in a CUDA graph ({type(ex).__name__}: "
                  f"{str(ex).splitlines()[0][:120]}); running eagerly", file=sys.stderr, flush=True)
            return False
        self._graphs[B] = (graph, ctx)
        return True

    def _step_graph(self, entries, S: int, max_kv: int):
        """Replay the captured graph of the bucket that fits S rows; None if graphs turned out to be unusable."""
        B = self._bucket(S)
        if B not in self._graphs and not self._capture(B):
            return None
        self._fill(entries, S, S, S, self.table_width, pad_to=B)
        self._graphs[B][0].replay()
        ops.LAUNCHES += self._graph_launches[B]
        self.stats["graph_steps"] += 1
        return self._logits[:S]

    # ---- CUDA graphs for other steps, by shape ---------------------------------------------------------
    def _step_shape_graph(self, entries, q_lens, T: int, S: int, R: int):
        """Replay the graph of this step's shape if there is one; capture one if the shape has occurred before;
        None (the caller launches the step kernel by kernel) otherwise.  Everything that differs between two steps
        of one shape (tokens, positions, slots, block tables, wanted rows) lies in the staging block on the device;
        block tables are staged at their full width and the split of decode attention is chosen for the longest
        context, so that the captured launches hold for every step of the shape."""
        key = (tuple(q_lens), R)
        hit = self._shape_graphs.get(key)
        if hit is None:
            seen = self._shape_seen.get(key, 0) + 1
            if len(self._shape_seen) > 4096:
                self._shape_seen.clear()
            self._shape_seen[key] = seen
            if seen < 2:
                return None
        W = self.table_width
        lay, _, _, _ = self._fill(entries, T, S, R, W)
        if hit is None:
            ctx = self._context(lay, T, S, R, W, q_lens, self.max_model_len)
            ctx.extras["captured"] = True
            graph = torch.cuda.CUDAGraph()
            before = ops.launches()
            try:
                # the first step of this shape ran eagerly: lazy initialisation is done.  Capture runs nothing.
                with torch.cuda.graph(graph):
                    if R > 0:
                        self.model.forward(ctx, self.cache_views, self.states, self._logits)
                    else:
                        self.model.forward_hidden(ctx, self.cache_views, self.states)
            except Exception as ex:
                torch.cuda.synchronize(self.device)
                ops.LAUNCHES = before
                self._shape_seen[key] = -(1 << 30)            # never try this shape again
                print(f"[cppvllm_b200] a step of shape {key if len(str(key)) < 80 else str(key)[:80] + '...'} cannot be "
                      f"captured ({type(ex).__name__}: {str(ex).splitlines()[0][:120]}); running it eagerly",
                      file=sys.stderr, flush=True)
                ctx = self._context(lay, T, S, R, W, q_lens, max(e.start + len(e.tokens) for e in entries))
                if R > 0:
                    return self.model.forward(ctx, self.cache_views, self.states, self._logits)[:R]
                return self._forward_no_logits(ctx)
            hit = (graph, ctx, ops.launches() - before)
            ops.LAUNCHES = before
            self._shape_graphs[key] = hit
            while len(self._shape_graphs) > SHAPE_GRAPHS:
                self._shape_graphs.popitem(last=False)
        else:
            self._shape_graphs.move_to_end(key)
        hit[0].replay()
        ops.LAUNCHES += hit[2]
        self.stats["graph_steps"] += 1
        return self._logits[:R]

    # ---- bookkeeping helpers ----------------------------------------------------------------------------
    def check_errors(self) -> None:
        """Raise if a kernel of an earlier step recorded an index it refused to follow (synchronises)."""
        ops.check_device_errors(self.device)
