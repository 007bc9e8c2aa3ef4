"""The cache manager in C++ (csrc/cache_runtime.cpp) behind the interface of cache/manager.py's CacheManager.

The policy is the one that manager.py states; that module stays as the plain twin, and tests drive both with the same
random sequences of calls and compare every table and count.  What this one adds for the step function: the block
tables of a group are one dense int32 array ``tables[g]`` of shape [state slots, table width] (-1 where nothing is
held) that lives in the library's memory and is read in place, so a step copies rows of it and converts nothing.
A request is known to the library by its state slot; this wrapper maps request ids to slots.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_void_p, c_longlong, POINTER
from typing import Dict, List, Optional, Sequence

import numpy as np

from .manager import CacheError, GroupConfig, OutOfPages

_lib = None


def _library():
    global _lib
    if _lib is None:
        from ..csrc.build import load_library
        lib = load_library("runtime")
        lib.cvb_cm_create.restype = c_void_p
        lib.cvb_cm_create.argtypes = [c_int, POINTER(c_int), POINTER(c_int), c_int, c_int, c_int, c_int]
        lib.cvb_cm_destroy.argtypes = [c_void_p]
        for name in ("cvb_cm_tables", "cvb_cm_table_len"):
            getattr(lib, name).restype = POINTER(c_int)
            getattr(lib, name).argtypes = [c_void_p, c_int]
        for name in ("cvb_cm_computed", "cvb_cm_registered"):
            getattr(lib, name).restype = POINTER(c_int)
            getattr(lib, name).argtypes = [c_void_p]
        lib.cvb_cm_prefix_hits.restype = c_longlong
        lib.cvb_cm_prefix_hits.argtypes = [c_void_p]
        lib.cvb_cm_message.restype = ctypes.c_char_p
        lib.cvb_cm_message.argtypes = [c_void_p]
        lib.cvb_cm_num_free.argtypes = [c_void_p, c_int]
        lib.cvb_cm_num_free_slots.argtypes = [c_void_p]
        lib.cvb_cm_refs.argtypes = [c_void_p, c_int, c_int]
        lib.cvb_cm_can_admit.argtypes = [c_void_p, c_void_p, c_int, c_int]
        lib.cvb_cm_admit.argtypes = [c_void_p, c_void_p, c_int]
        lib.cvb_cm_commit.argtypes = [c_void_p, c_int, c_void_p, c_int]
        lib.cvb_cm_take_fresh_slots.argtypes = [c_void_p, POINTER(c_int), c_int]
        lib.cvb_cm_pages_missing.argtypes = [c_void_p, c_int, c_int, POINTER(c_int)]
        for name in ("cvb_cm_covered", "cvb_cm_can_reserve", "cvb_cm_reserve", "cvb_cm_advance"):
            getattr(lib, name).argtypes = [c_void_p, c_int, c_int]
        lib.cvb_cm_advance_many.argtypes = [c_void_p, c_void_p, c_void_p, c_int]
        lib.cvb_cm_release.argtypes = [c_void_p, c_int]
        lib.cvb_cm_check.argtypes = [c_void_p]
        _lib = lib
    return _lib


def _tokens_array(tokens: Optional[Sequence[int]]):
    """(pointer, count, keep-alive) of the tokens as int32; a token that is not known on the host yet stays negative."""
    if tokens is None:
        return None, 0, None
    arr = np.asarray(tokens, dtype=np.int64)
    arr = np.where(arr < 0, -1, np.minimum(arr, 0x7fffffff)).astype(np.int32)
    return arr.ctypes.data_as(c_void_p), int(arr.shape[0]), arr


class _PoolView:
    """What callers read of a group's pool."""

    def __init__(self, mgr: "NativeCacheManager", group: int, num_pages: int):
        self._mgr, self._g, self.num_pages = mgr, group, num_pages

    @property
    def num_free(self) -> int:
        return int(self._mgr._lib.cvb_cm_num_free(self._mgr._h, self._g))

    def refs(self, page: int) -> int:
        return int(self._mgr._lib.cvb_cm_refs(self._mgr._h, self._g, int(page)))


class NativeLease:
    """What one live request holds; the tables are views of the library's arrays (valid until the request is released)."""
    __slots__ = ("_mgr", "request_id", "state_slot")

    def __init__(self, mgr: "NativeCacheManager", request_id, state_slot: int):
        self._mgr, self.request_id, self.state_slot = mgr, request_id, state_slot

    @property
    def computed(self) -> int:
        return int(self._mgr._computed[self.state_slot])

    @property
    def registered(self) -> int:
        return int(self._mgr._registered[self.state_slot])

    @property
    def tables(self) -> List[np.ndarray]:
        m, s = self._mgr, self.state_slot
        return [m.tables[g][s, :m._table_len[g][s]] for g in range(len(m.groups))]


class NativeCacheManager:
    native = True

    def __init__(self, groups: Sequence[GroupConfig], page_size: int, num_state_slots: int, table_width: int,
                 prefix_caching: bool = False):
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        self.page_size = page_size
        self.groups = list(groups)
        if prefix_caching and not (len(self.groups) == 1 and self.groups[0].window <= 0):
            raise ValueError("the prefix cache needs exactly one group of cache units, and one that keeps all keys")
        if any(g.num_pages <= 0 for g in self.groups):
            raise ValueError("a page pool needs at least one page")
        if table_width <= 0 or num_state_slots <= 0:
            raise ValueError("table_width and num_state_slots must be positive")
        self.prefix_caching = bool(prefix_caching)
        self.table_width = int(table_width)
        self.num_state_slots = int(num_state_slots)
        self._lib = _library()
        G = len(self.groups)
        pages = (c_int * G)(*[g.num_pages for g in self.groups])
        windows = (c_int * G)(*[g.window for g in self.groups])
        self._h = c_void_p(self._lib.cvb_cm_create(G, pages, windows, page_size, num_state_slots, table_width,
                                                   1 if prefix_caching else 0))
        if not self._h:
            raise ValueError("the cache manager could not be created from these sizes")

        def view(ptr, shape):
            n = int(np.prod(shape))
            return np.ctypeslib.as_array(ptr, shape=(n,)).reshape(shape)

        self.tables = [view(self._lib.cvb_cm_tables(self._h, g), (num_state_slots, table_width)) for g in range(G)]
        self._table_len = [view(self._lib.cvb_cm_table_len(self._h, g), (num_state_slots,)) for g in range(G)]
        self._computed = view(self._lib.cvb_cm_computed(self._h), (num_state_slots,))
        self._registered = view(self._lib.cvb_cm_registered(self._h), (num_state_slots,))
        self.pools = [_PoolView(self, g, self.groups[g].num_pages) for g in range(G)]
        self.leases: Dict[object, NativeLease] = {}
        self._missing = (c_int * G)()
        self._fresh = (c_int * num_state_slots)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self.tables = self._table_len = self._computed = self._registered = None
            self._lib.cvb_cm_destroy(h)

    # ---- errors ------------------------------------------------------------------------------------------
    def _raise(self, code: int, request_id, what: str):
        if code == -2:
            raise OutOfPages(f"a group has too few free pages for request {request_id!r} ({what})")
        if code == -3:
            raise ValueError(f"request {request_id!r}: {what} needs a block table wider than {self.table_width} pages")
        if code == -4:
            raise CacheError("no free state slot")
        raise CacheError(f"request {request_id!r}: {what} refused (not admitted, released twice, or a length that shrinks)")

    # ---- requests ----------------------------------------------------------------------------------------
    @property
    def prefix_hits(self) -> int:
        return int(self._lib.cvb_cm_prefix_hits(self._h))

    def can_admit(self, tokens: Sequence[int], upto_len: int) -> bool:
        ptr, n, keep = _tokens_array(tokens if self.prefix_caching else None)
        return bool(self._lib.cvb_cm_can_admit(self._h, ptr, n, int(upto_len)))

    def admit(self, request_id, tokens: Optional[Sequence[int]] = None) -> NativeLease:
        if request_id in self.leases:
            raise CacheError(f"request {request_id!r} is already admitted")
        ptr, n, keep = _tokens_array(tokens if self.prefix_caching else None)
        slot = int(self._lib.cvb_cm_admit(self._h, ptr, n))
        if slot < 0:
            self._raise(slot, request_id, "admission")
        lease = NativeLease(self, request_id, slot)
        self.leases[request_id] = lease
        return lease

    def commit(self, request_id, tokens: Sequence[int]) -> None:
        if not self.prefix_caching:
            return
        lease = self.lease(request_id)
        ptr, n, keep = _tokens_array(tokens)
        rc = int(self._lib.cvb_cm_commit(self._h, lease.state_slot, ptr, n))
        if rc < 0:
            self._raise(rc, request_id, "commit")

    def lease(self, request_id) -> NativeLease:
        try:
            return self.leases[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not admitted") from None

    def take_fresh_slots(self) -> List[int]:
        n = int(self._lib.cvb_cm_take_fresh_slots(self._h, self._fresh, self.num_state_slots))
        return list(self._fresh[:n])

    def num_pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    # ---- pages -------------------------------------------------------------------------------------------
    def pages_missing(self, request_id, upto_len: int, computed: Optional[int] = None) -> List[int]:
        lease = self.leases.get(request_id)
        if lease is None:                      # what a request that is not admitted yet would need
            out = []
            for g in self.groups:
                first = max(0, (computed or 0) - g.window + 1) // self.page_size if g.window > 0 else 0
                out.append(max(0, self.num_pages_for(upto_len) - first))
            return out
        rc = int(self._lib.cvb_cm_pages_missing(self._h, lease.state_slot, int(upto_len), self._missing))
        if rc < 0:
            self._raise(rc, request_id, "pages_missing")
        return list(self._missing)

    def covered(self, request_id, upto_len: int) -> bool:
        return bool(self._lib.cvb_cm_covered(self._h, self.lease(request_id).state_slot, int(upto_len)) > 0)

    def can_reserve(self, request_id, upto_len: int) -> bool:
        return bool(self._lib.cvb_cm_can_reserve(self._h, self.lease(request_id).state_slot, int(upto_len)) > 0)

    def reserve(self, request_id, upto_len: int) -> int:
        rc = int(self._lib.cvb_cm_reserve(self._h, self.lease(request_id).state_slot, int(upto_len)))
        if rc < 0:
            self._raise(rc, request_id, f"covering {upto_len} tokens")
        return rc

    def advance(self, request_id, computed: int) -> None:
        rc = int(self._lib.cvb_cm_advance(self._h, self.lease(request_id).state_slot, int(computed)))
        if rc < 0:
            raise CacheError("a request's computed length cannot shrink")

    def advance_many(self, request_ids, computed) -> None:
        """advance() for the requests of a step in one call into the library."""
        n = len(request_ids)
        try:
            slots = np.fromiter((self.leases[r].state_slot for r in request_ids), dtype=np.int32, count=n)
        except KeyError as e:
            raise CacheError(f"request {e.args[0]!r} is not admitted") from None
        upto = np.asarray(computed, dtype=np.int32)
        bad = int(self._lib.cvb_cm_advance_many(self._h, slots.ctypes.data_as(c_void_p), upto.ctypes.data_as(c_void_p), n))
        if bad >= 0:
            raise CacheError(f"request {request_ids[bad]!r}: a request's computed length cannot shrink")

    def release(self, request_id) -> None:
        lease = self.leases.pop(request_id, None)
        if lease is None:
            raise CacheError(f"request {request_id!r} is released but is not admitted")
        rc = int(self._lib.cvb_cm_release(self._h, lease.state_slot))
        if rc < 0:
            self._raise(rc, request_id, "release")

    # ---- requests that the scheduler in C++ admits and releases itself ---------------------------------------
    def adopt(self, request_id, state_slot: int) -> NativeLease:
        """The library admitted a request on its own (csrc/scheduler_runtime.cpp): make it known here by its id."""
        lease = NativeLease(self, request_id, int(state_slot))
        self.leases[request_id] = lease
        return lease

    def drop(self, request_id) -> None:
        """The library released a request on its own."""
        self.leases.pop(request_id, None)

    # ---- what a step needs -------------------------------------------------------------------------------
    def block_table(self, request_id, group: int) -> List[int]:
        return [int(p) for p in self.lease(request_id).tables[group]]

    def slots_for(self, request_id, group: int, start: int, count: int) -> List[int]:
        table = self.lease(request_id).tables[group]
        ps = self.page_size
        out = []
        for pos in range(start, start + count):
            i = pos // ps
            if i >= len(table) or table[i] < 0:
                raise CacheError(f"request {request_id!r}: position {pos} has no page in group {group}")
            out.append(int(table[i]) * ps + pos % ps)
        return out

    def num_free_pages(self, group: int = 0) -> int:
        return self.pools[group].num_free

    def check_invariants(self) -> None:
        if int(self._lib.cvb_cm_check(self._h)) != 0:
            raise AssertionError(self._lib.cvb_cm_message(self._h).decode())
        slots = [l.state_slot for l in self.leases.values()]
        if len(set(slots)) != len(slots):
            raise AssertionError("a state slot is held by two requests")
        if len(slots) + int(self._lib.cvb_cm_num_free_slots(self._h)) != self.num_state_slots:
            raise AssertionError("the wrapper and the library disagree on the live requests")
