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
changes nothing.

Prefix cache (optional, ``prefix_caching=True``; reference :10-24,71-143).  Full pages are registered under a chain
key (the key of the page before, and the page's tokens) once their keys are in the cache (``commit``); a page that is
given back keeps its key until it is handed out again for other contents.  ``admit`` with the request's tokens takes
the longest chain of registered pages that match its prefix, at most ``(len - 1) // page_size`` pages so that at
least one token is computed, and counts them as computed; pages are then shared (reference counts) and read-only for
the requests that share them, since a request only ever writes positions beyond its computed length.  The cache of a
windowed group or of per-request state cannot be shared this way: the manager refuses the option unless there is
exactly one group and it keeps all keys.

State slots.  A request also receives one slot number for per-request state of fixed size (what a recurrent or
convolutional mixer would keep).  The attention-only architecture here keeps no such state, but the slot
travels with every step, and the runner zeroes a slot's tensors when it is handed out.
"""
from __future__ import annotations

from collections import OrderedDict, deque
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
    """Pages of one group: a free list, least-recently-freed first, reference counts against double frees, and for the
    prefix cache the chain key and tokens of a page's contents."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: "OrderedDict[int, None]" = OrderedDict((p, None) for p in range(num_pages))
        self._refs = [0] * num_pages
        self._key: List[Optional[int]] = [None] * num_pages       # chain key of the page's contents, if registered
        self._tokens: List[Optional[tuple]] = [None] * num_pages
        self._by_key: Dict[int, int] = {}

    @property
    def num_free(self) -> int:
        return len(self._free)

    def refs(self, page: int) -> int:
        return self._refs[page]

    def take(self) -> int:
        """A page for new contents: the least recently freed one; what it was registered as is forgotten."""
        if not self._free:
            raise OutOfPages("no free page")
        p, _ = self._free.popitem(last=False)
        k = self._key[p]
        if k is not None:
            if self._by_key.get(k) == p:
                del self._by_key[k]
            self._key[p] = self._tokens[p] = None
        self._refs[p] = 1
        return p

    def give_back(self, page: int) -> None:
        if not (0 <= page < self.num_pages) or self._refs[page] <= 0:
            raise CacheError(f"page {page} is given back but is not held")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free[page] = None                               # to the tail; it keeps its key until taken again

    # ---- prefix cache ----
    @staticmethod
    def chain_key(prefix_key: Optional[int], tokens: tuple) -> int:
        return hash((prefix_key, tokens))

    def find(self, prefix_key: Optional[int], tokens: tuple):
        """(page, key) registered for these tokens after that prefix, or (None, key)."""
        k = self.chain_key(prefix_key, tokens)
        p = self._by_key.get(k)
        if p is None or self._tokens[p] != tokens:
            return None, k
        return p, k

    def share(self, page: int) -> None:
        """One more holder of a registered page (taken off the free list if nobody held it)."""
        if self._refs[page] == 0:
            del self._free[page]
        self._refs[page] += 1

    def register(self, page: int, prefix_key: Optional[int], tokens: tuple) -> int:
        """Record what a held page contains; returns its chain key.  The first page registered under a key keeps it."""
        if self._key[page] is None:
            k = self.chain_key(prefix_key, tokens)
            self._key[page] = k
            self._tokens[page] = tokens
            self._by_key.setdefault(k, page)
        return self._key[page]

    def key_of(self, page: int) -> Optional[int]:
        return self._key[page]


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
    registered: int = 0                  # prefix cache: leading pages whose contents are registered


class CacheManager:
    def __init__(self, groups: Sequence[GroupConfig], page_size: int, num_state_slots: int, prefix_caching: bool = False):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.groups = list(groups)
        if prefix_caching and not (len(self.groups) == 1 and self.groups[0].window <= 0):
            raise ValueError("the prefix cache needs exactly one group of cache units, and one that keeps all keys")
        self.prefix_caching = bool(prefix_caching)
        self.prefix_hits = 0                                      # pages taken from the prefix cache so far
        self.pools = [PagePool(g.num_pages) for g in self.groups]
        self.slots = SlotPool(num_state_slots)
        self.leases: Dict[object, Lease] = {}
        self._fresh_slots: List[int] = []

    # ---- requests ------------------------------------------------------------------------------------
    def _prefix_pages(self, tokens: Sequence[int]):
        """[(page, key)] of the longest registered chain that matches the prefix of `tokens`."""
        out = []
        if not self.prefix_caching or tokens is None:
            return out
        ps, pool = self.page_size, self.pools[0]
        key = None
        for i in range((len(tokens) - 1) // ps):                  # at least one token is always computed
            chunk = tuple(tokens[i * ps:(i + 1) * ps])
            if min(chunk) < 0:
                break
            page, key = pool.find(key, chunk)
            if page is None:
                break
            out.append((page, key))
        return out

    def can_admit(self, tokens: Sequence[int], upto_len: int) -> bool:
        """Whether a request with these tokens could be admitted and covered up to `upto_len` now.  Registered pages
        that somebody holds cost nothing; registered pages on the free list are counted as taken from it."""
        if self.slots.num_free == 0:
            return False
        shared = sum(1 for page, _ in self._prefix_pages(tokens) if self.pools[0].refs(page) > 0)
        need = self.num_pages_for(upto_len)
        return all((need - shared if g == 0 else need) <= p.num_free for g, p in enumerate(self.pools))

    def admit(self, request_id, tokens: Optional[Sequence[int]] = None) -> Lease:
        """A new request.  With the prefix cache and the request's tokens, the pages of its longest registered prefix
        are shared with it and count as computed (``lease.computed``)."""
        if request_id in self.leases:
            raise CacheError(f"request {request_id!r} is already admitted")
        lease = Lease(request_id, self.slots.take(), [[] for _ in self.groups], 0, [0] * len(self.groups))
        for page, _ in self._prefix_pages(tokens):
            self.pools[0].share(page)
            lease.tables[0].append(page)
        lease.registered = len(lease.tables[0]) if self.prefix_caching else 0
        lease.computed = lease.registered * self.page_size
        self.prefix_hits += lease.registered
        self.leases[request_id] = lease
        self._fresh_slots.append(lease.state_slot)
        return lease

    def commit(self, request_id, tokens: Sequence[int]) -> None:
        """Register the request's full pages whose keys are in the cache (and whose tokens are all known), so that
        later requests with the same prefix can share them.  Does nothing without the prefix cache."""
        if not self.prefix_caching:
            return
        lease = self.lease(request_id)
        ps, pool, table = self.page_size, self.pools[0], lease.tables[0]
        full = min(lease.computed, len(tokens)) // ps
        i = lease.registered
        while i < full:
            chunk = tuple(tokens[i * ps:(i + 1) * ps])
            if min(chunk) < 0:
                break                                             # a token that is not known on the host yet
            prefix = pool.key_of(table[i - 1]) if i > 0 else None
            pool.register(table[i], prefix, chunk)
            i += 1
        lease.registered = i

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

    def covered(self, request_id, upto_len: int) -> bool:
        """Whether the request's tables already reach `upto_len` in every group (nothing to reserve): the common case
        of a decoding request, checked without looking at the pools."""
        need = (upto_len + self.page_size - 1) // self.page_size
        for table in self.leases[request_id].tables:
            if len(table) < need:
                return False
        return True

    def can_reserve(self, request_id, upto_len: int) -> bool:
        return all(n <= p.num_free for n, p in zip(self.pages_missing(request_id, upto_len), self.pools))

    def reserve(self, request_id, upto_len: int) -> int:
        """Cover positions below `upto_len` with pages, in every group.  All or nothing.  Returns how many tokens the
        request's tables cover now (in every group), so that a caller can skip the call while it stays within that."""
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
        return min((len(t) for t in lease.tables), default=target) * self.page_size

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
        """Every page is either free exactly once, or held: by exactly one request, or (prefix cache) by as many
        requests as its reference count says, each at most once."""
        for g, pool in enumerate(self.pools):
            free = list(pool._free)
            if len(set(free)) != len(free):
                raise AssertionError(f"group {g}: a page is in the free list twice")
            holders: Dict[int, int] = {}
            for rid, lease in self.leases.items():
                mine = [p for p in lease.tables[g] if p >= 0]
                if len(set(mine)) != len(mine):
                    raise AssertionError(f"group {g}: request {rid!r} holds a page twice")
                for p in mine:
                    holders[p] = holders.get(p, 0) + 1
            for p in range(pool.num_pages):
                n = holders.get(p, 0)
                if n != pool.refs(p):
                    raise AssertionError(f"group {g}: page {p} is held by {n} requests but counts {pool.refs(p)}")
                if (n == 0) != (p in pool._free):
                    raise AssertionError(f"group {g}: page {p} is {'neither' if n == 0 else 'both'} free {'nor' if n == 0 else 'and'} held")
                if n > 1 and not self.prefix_caching:
                    raise AssertionError(f"group {g}: page {p} is held by {n} requests")
            for k, p in pool._by_key.items():
                if pool.key_of(p) != k:
                    raise AssertionError(f"group {g}: key of page {p} and the key table disagree")
        held_slots = [l.state_slot for l in self.leases.values()]
        if len(set(held_slots)) != len(held_slots):
            raise AssertionError("a state slot is held by two requests")
        if len(held_slots) + self.slots.num_free != self.slots.num_slots:
            raise AssertionError("a state slot is lost")
