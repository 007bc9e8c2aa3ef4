"""Host-side bookkeeping of the paged cache and of per-request state slots.  No tensors live here: the manager
deals in page numbers and slot numbers; the device storage they index belongs to the runner (engine/runner.py).

Pages.  Keys and values are kept in pages of ``page_size`` tokens.  Cache units (one per run-list entry that
writes a cache) whose needs are equal form a *group*; each group has its own pool of pages and each request
has one block table per group (logical page i -> physical page id, -1 where nothing is held).  One page id of
a group covers all units of that group, as one block id covers all layers in the reference
(engine/model_runner.cpp:104-113).  A group whose mixers look back only ``window`` positions gives a page back
as soon as every position in it lies before the window of the request's next token; a group that needs all
keys holds its pages until the request ends.

Policy, after the reference's BlockManager (engine/block_manager.cpp): pages are handed out least-recently-freed
first (:35-69); a request's pages are released last-logical-page first (:145-153); ``reserve`` tops a table up to
cover a given length like ``allocate``/``may_append`` (:80-126) and is all-or-nothing, so a failed reservation
changes nothing.  Not carried over: the prefix cache (hash chain over full blocks, :10-24,71-143).

State slots.  A request also receives one slot number for per-request state of fixed size (what a recurrent or
convolutional mixer would keep).  The attention-only architecture here keeps no such state, but the slot
travels with every step, and the runner zeroes a slot's tensors when it is handed out.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence


class OutOfPages(RuntimeError):
    """A reservation needs more pages than a group has free."""


class CacheError(RuntimeError):
    """Misuse of the manager: unknown request, double admission, double free."""


@dataclass(frozen=True)
class GroupConfig:
    num_pages: int
    window: int = 0          # 0 = all keys are kept; w > 0 = positions further back than w are given up
    units: tuple = ()        # cache unit ids served by this group (informational)


class PagePool:
    """Free list of one group, least-recently-freed first, with ownership tracking against double frees."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: Deque[int] = deque(range(num_pages))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.popleft()
        self._held[p] = True
        return p

    def give_back(self, page: int) -> None:
        if not (0 <= page < self.num_pages) or not self._held[page]:
            raise CacheError(f"page {page} is given back but is not held")
        self._held[page] = False
        self._free.append(page)


class SlotPool:
    """Numbers 0..n-1 for per-request state; lowest free number first."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError("no free state slot")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not (0 <= slot < self.num_slots) or not self._held[slot]:
            raise CacheError(f"state slot {slot} is given back but is not held")
        self._held[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)


@dataclass
class Lease:
    """What one live request holds."""
    request_id: object
    state_slot: int
    tables: List[List[int]]              # per group: logical page -> physical page or -1
    computed: int = 0                    # tokens whose keys are in the cache
    first_held: List[int] = field(default_factory=list)   # per group: first logical page still held


class CacheManager:
    def __init__(self, groups: Sequence[GroupConfig], page_size: int, num_state_slots: int):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.groups = list(groups)
        self.pools = [PagePool(g.num_pages) for g in self.groups]
        self.slots = SlotPool(num_state_slots)
        self.leases: Dict[object, Lease] = {}
        self._fresh_slots: List[int] = []

    # ---- requests ------------------------------------------------------------------------------------
    def admit(self, request_id) -> Lease:
        if request_id in self.leases:
            raise CacheError(f"request {request_id!r} is already admitted")
        lease = Lease(request_id, self.slots.take(), [[] for _ in self.groups], 0, [0] * len(self.groups))
        self.leases[request_id] = lease
        self._fresh_slots.append(lease.state_slot)
        return lease

    def lease(self, request_id) -> Lease:
        try:
            return self.leases[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not admitted") from None

    def take_fresh_slots(self) -> List[int]:
        """State slots handed out since the last call: their tensors must be zeroed before the next step."""
        out, self._fresh_slots = self._fresh_slots, []
        return out

    def num_pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    # ---- pages ---------------------------------------------------------------------------------------
    def _first_needed_page(self, group: int, computed: int) -> int:
        w = self.groups[group].window
        if w <= 0:
            return 0
        # the next token sits at position `computed` and reads positions >= computed - w + 1
        return max(0, computed - w + 1) // self.page_size

    def pages_missing(self, request_id, upto_len: int, computed: Optional[int] = None) -> List[int]:
        """Per group: pages to take so that positions first_needed .. upto_len-1 are covered."""
        lease = self.leases.get(request_id)
        need = []
        for g in range(len(self.groups)):
            have = len(lease.tables[g]) if lease else 0
            first = max(have, self._first_needed_page(g, lease.computed if lease else (computed or 0)))
            need.append(max(0, self.num_pages_for(upto_len) - first))
        return need

    def can_reserve(self, request_id, upto_len: int) -> bool:
        return all(n <= p.num_free for n, p in zip(self.pages_missing(request_id, upto_len), self.pools))

    def reserve(self, request_id, upto_len: int) -> None:
        """Cover positions below `upto_len` with pages, in every group.  All or nothing."""
        lease = self.lease(request_id)
        need = self.pages_missing(request_id, upto_len)
        for g, n in enumerate(need):
            if n > self.pools[g].num_free:
                raise OutOfPages(f"group {g} needs {n} pages for request {request_id!r} but has {self.pools[g].num_free} free")
        target = self.num_pages_for(upto_len)
        for g in range(len(self.groups)):
            table = lease.tables[g]
            first = self._first_needed_page(g, lease.computed)
            while len(table) < target:
                table.append(self.pools[g].take() if len(table) >= first else -1)

    def advance(self, request_id, computed: int) -> None:
        """Record that the request's first `computed` tokens are in the cache; windowed groups give back the
        pages that no later token can read."""
        lease = self.lease(request_id)
        if computed < lease.computed:
            raise CacheError("a request's computed length cannot shrink")
        lease.computed = computed
        for g in range(len(self.groups)):
            if self.groups[g].window <= 0:
                continue
            table = lease.tables[g]
            upto = min(self._first_needed_page(g, computed), len(table))
            for i in range(lease.first_held[g], upto):
                if table[i] >= 0:
                    self.pools[g].give_back(table[i])
                    table[i] = -1
            lease.first_held[g] = max(lease.first_held[g], upto)

    def release(self, request_id) -> None:
        lease = self.leases.pop(request_id, None)
        if lease is None:
            raise CacheError(f"request {request_id!r} is released but is not admitted")
        for g, table in enumerate(lease.tables):
            for page in reversed(table):
                if page >= 0:
                    self.pools[g].give_back(page)
            table.clear()
        self.slots.give_back(lease.state_slot)
        if lease.state_slot in self._fresh_slots:
            self._fresh_slots.remove(lease.state_slot)

    # ---- what a step needs ------------------------------------------------------------------------------
    def block_table(self, request_id, group: int) -> List[int]:
        return self.lease(request_id).tables[group]

    def slots_for(self, request_id, group: int, start: int, count: int) -> List[int]:
        """Flat cache slots (page id * page_size + offset) for positions start .. start+count-1."""
        table = self.lease(request_id).tables[group]
        ps = self.page_size
        out = []
        for pos in range(start, start + count):
            i = pos // ps
            if i >= len(table) or table[i] < 0:
                raise CacheError(f"request {request_id!r}: position {pos} has no page in group {group}")
            out.append(table[i] * ps + pos % ps)
        return out

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    # ---- self-check (used by tests) -------------------------------------------------------------------------
    def check_invariants(self) -> None:
        """Every page is either free exactly once or held by exactly one request exactly once."""
        for g, pool in enumerate(self.pools):
            seen = {}
            for p in pool._free:
                if p in seen:
                    raise AssertionError(f"group {g}: page {p} is in the free list twice")
                seen[p] = "free"
            for rid, lease in self.leases.items():
                for p in lease.tables[g]:
                    if p < 0:
                        continue
                    if p in seen:
                        raise AssertionError(f"group {g}: page {p} held by {rid!r} is also {seen[p]}")
                    seen[p] = f"held by {rid!r}"
            if len(seen) != pool.num_pages:
                lost = sorted(set(range(pool.num_pages)) - set(seen))
                raise AssertionError(f"group {g}: pages {lost} are neither free nor held")
        held_slots = [l.state_slot for l in self.leases.values()]
        if len(set(held_slots)) != len(held_slots):
            raise AssertionError("a state slot is held by two requests")
        if len(held_slots) + self.slots.num_free != self.slots.num_slots:
            raise AssertionError("a state slot is lost")
