"""The cache manager: who holds which pages.

Host-side bookkeeping only (the device tensors live in ``cache.storage``). Layers are
put into groups by what their mixer asks (``CacheNeed.group_key()``: all keys, or a
window of them, with their head count and size); every group has a page pool and, per
request, a block table of its own. One page id addresses that page in every layer of
its group (llm-core/src/backends/candle.rs:167,1493-1496 keys storage by (layer, page)).

Pages are reserved BEFORE a step for exactly the tokens the step brings, and the cached
length is advanced by ``commit`` after it (the reference grows a table by one page after
a step, llm-scheduler/src/scheduler.rs:161-167). Pages go back when a request is
released, and, in a window group, as soon as the window has passed them. Beside the
pages each live request holds one slot for fixed-size state.

The bookkeeping itself is C++ (``csrc/host/cache_manager.cpp``); this class holds its
handle, maps the caller's request ids (anything hashable) to the library's numbers and
turns its statuses into exceptions.
"""
from __future__ import annotations

import ctypes
from ctypes import byref, c_int, c_int32, c_int64, c_void_p
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

from .. import host
from ..parts.spec import CacheNeed
from .pool import CacheError, NoFreeSlot, OutOfPages, check  # noqa: F401  (re-exported)

RELEASED = -1  # table entry of a page that a window has passed


@dataclass
class GroupSpec:
    """One group of run-order entries with the same need."""
    need: CacheNeed
    entries: List[int]          # run-order indices whose keys and values live in this group
    n_pages: int


class RequestRecord:
    """A live request as the manager sees it; the numbers are read from the library."""

    def __init__(self, manager: "CacheManager", request_id: Hashable, number: int, slot: int):
        self._manager = manager
        self.request_id = request_id
        self.number = number        # the request's id inside the host library
        self.slot = slot

    def _info(self):
        info, edits = (c_int * 3)(), c_int64()
        m = self._manager
        check(m._lib.llmrs_cm_info(m._handle, self.number, info, byref(edits)), m._names)
        return info[1], info[2], edits.value

    @property
    def cached_len(self) -> int:
        return self._info()[0]

    @property
    def reserved_len(self) -> int:
        """Tokens that the tables cover (>= cached_len between reserve and commit)."""
        return self._info()[1]

    @property
    def edits(self) -> int:
        """Counts changes to the tables other than appending a page."""
        return self._info()[2]

    @property
    def tables(self) -> List[List[int]]:
        """Per group: logical page -> physical page."""
        return [self._manager.table(self.request_id, g) for g in range(len(self._manager.groups))]


class _PoolView:
    """Counts of one group's pool inside the manager."""

    def __init__(self, manager: "CacheManager", group: int):
        self._manager, self._group = manager, group
        self.capacity = manager.groups[group].n_pages

    def free_pages(self) -> int:
        m = self._manager
        free, cap = c_int(), c_int()
        check(m._lib.llmrs_cm_pool_counts(m._handle, self._group, byref(free), byref(cap)))
        return free.value

    def used_pages(self) -> int:
        return self.capacity - self.free_pages()


def pages_for(n_tokens: int, page_size: int) -> int:
    return -(-n_tokens // page_size)


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int, n_slots: int):
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        self.n_slots = n_slots
        self._lib = host.lib()
        self._handle = c_void_p()
        G = len(self.groups)
        n_pages = (c_int * max(G, 1))(*[g.n_pages for g in self.groups])
        windows = (c_int * max(G, 1))(*[g.need.window if g.need.kind == "window" and g.need.window > 0 else 0
                                        for g in self.groups])
        check(self._lib.llmrs_cm_create(n_pages, windows, G, page_size, n_slots, byref(self._handle)))
        self.pools = [_PoolView(self, g) for g in range(G)]
        self.requests: Dict[Hashable, RequestRecord] = {}
        self._names: Dict[int, Hashable] = {}
        self._next_number = 0
        self._other_numbers: Dict[Hashable, int] = {}
        self._need_buf = (c_int * max(G, 1))()

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.llmrs_cm_destroy(self._handle)
            self._handle = None

    # -- requests --------------------------------------------------------------------
    def admit(self, request_id: Hashable) -> RequestRecord:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already live")
        number = self.number_of(request_id)
        slot = c_int()
        check(self._lib.llmrs_cm_admit(self._handle, number, byref(slot)), self._names)
        rec = RequestRecord(self, request_id, number, slot.value)
        self.requests[request_id] = rec
        self._names[number] = request_id
        return rec

    def number_of(self, request_id: Hashable) -> int:
        """The request's number inside the host library: a non-negative integer id is its own number
        (the scheduler, which lives in the same library, then knows the request by the caller's id);
        any other id gets a negative number of its own."""
        if isinstance(request_id, int) and not isinstance(request_id, bool) and 0 <= request_id < 2 ** 62:
            return request_id
        number = self._other_numbers.get(request_id)
        if number is None:
            self._next_number += 1
            number = self._other_numbers[request_id] = -self._next_number
            if len(self._other_numbers) > 4 * self.n_slots + 64:    # forget ids that are no longer live
                self._other_numbers = {k: v for k, v in self._other_numbers.items()
                                       if k in self.requests or k == request_id}
        return number

    def has_free_slot(self) -> bool:
        return len(self.requests) < self.n_slots

    def record(self, request_id: Hashable) -> RequestRecord:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def release(self, request_id: Hashable) -> None:
        """Give back every page and the slot of a request."""
        rec = self.record(request_id)
        check(self._lib.llmrs_cm_release(self._handle, rec.number), self._names)
        del self.requests[request_id]
        del self._names[rec.number]

    # -- pages -----------------------------------------------------------------------
    def pages_needed(self, request_id: Optional[Hashable], n_new: int, cached_len: Optional[int] = None) -> List[int]:
        """Pages per group that ``reserve(request_id, n_new)`` would take from the pools.
        For a request that is not live yet pass ``request_id=None`` and its ``cached_len`` (0)."""
        live = request_id is not None
        number = self.record(request_id).number if live else 0
        check(self._lib.llmrs_cm_pages_needed(self._handle, int(live), number, n_new, cached_len or 0,
                                              self._need_buf), self._names)
        return list(self._need_buf[:len(self.groups)])

    def can_reserve(self, request_id: Optional[Hashable], n_new: int, cached_len: Optional[int] = None) -> bool:
        need = self.pages_needed(request_id, n_new, cached_len)
        return all(n <= pool.free_pages() for n, pool in zip(need, self.pools))

    def reserve(self, request_id: Hashable, n_new: int) -> None:
        """Cover positions cached_len .. cached_len+n_new-1 with pages in every group.
        Raises ``OutOfPages`` and changes nothing if any pool is short."""
        check(self._lib.llmrs_cm_reserve(self._handle, self.record(request_id).number, n_new), self._names)

    def cancel(self, request_id: Hashable) -> None:
        """Undo a reservation that was not committed (pages beyond the cached length go back)."""
        check(self._lib.llmrs_cm_cancel(self._handle, self.record(request_id).number), self._names)

    def commit(self, request_id: Hashable, n_new: int) -> None:
        """The step ran: the new tokens are cached. Pages a window has passed go back."""
        check(self._lib.llmrs_cm_commit(self._handle, self.record(request_id).number, n_new), self._names)

    # -- views -----------------------------------------------------------------------
    def table(self, request_id: Hashable, group: int) -> List[int]:
        rec = self.record(request_id)
        length = c_int()
        cap = 64
        while True:
            buf = (c_int32 * cap)()
            check(self._lib.llmrs_cm_table(self._handle, rec.number, group, buf, cap, byref(length)), self._names)
            if length.value <= cap:
                return list(buf[:length.value])
            cap = length.value

    def free_pages(self, group: int = 0) -> int:
        return self.pools[group].free_pages()

    def check_invariants(self) -> None:
        """Every page is either free or held by exactly as many tables as its count says; no
        request slot is lost or held twice; the library and this class know the same requests."""
        check(self._lib.llmrs_cm_check_invariants(self._handle), self._names)
        if {r.number for r in self.requests.values()} != set(self._names):
            raise CacheError("the request map and the library disagree")
