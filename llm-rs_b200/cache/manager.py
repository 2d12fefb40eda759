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
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence

from ..parts.spec import CacheNeed
from .pool import CacheError, OutOfPages, PagePool

RELEASED = -1  # table entry of a page that a window has passed


@dataclass
class GroupSpec:
    """One group of run-order entries with the same need."""
    need: CacheNeed
    entries: List[int]          # run-order indices whose keys and values live in this group
    n_pages: int


@dataclass
class RequestRecord:
    request_id: Hashable
    slot: int
    cached_len: int = 0
    reserved_len: int = 0       # tokens that the tables cover (>= cached_len between reserve and commit)
    tables: List[List[int]] = field(default_factory=list)   # per group: logical page -> physical page
    edits: int = 0              # counts changes to the tables other than appending a page


class NoFreeSlot(CacheError):
    pass


def pages_for(n_tokens: int, page_size: int) -> int:
    return -(-n_tokens // page_size)


class CacheManager:
    def __init__(self, groups: Sequence[GroupSpec], page_size: int, n_slots: int):
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        self.pools = [PagePool(g.n_pages) for g in self.groups]
        self.n_slots = n_slots
        self._free_slots = list(range(n_slots - 1, -1, -1))
        self.requests: Dict[Hashable, RequestRecord] = {}

    # -- requests --------------------------------------------------------------------
    def admit(self, request_id: Hashable) -> RequestRecord:
        if request_id in self.requests:
            raise CacheError(f"request {request_id!r} is already live")
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.n_slots} request slots are taken")
        rec = RequestRecord(request_id, self._free_slots.pop(), tables=[[] for _ in self.groups])
        self.requests[request_id] = rec
        return rec

    def has_free_slot(self) -> bool:
        return bool(self._free_slots)

    def record(self, request_id: Hashable) -> RequestRecord:
        try:
            return self.requests[request_id]
        except KeyError:
            raise CacheError(f"request {request_id!r} is not live") from None

    def release(self, request_id: Hashable) -> None:
        """Give back every page and the slot of a request."""
        rec = self.record(request_id)
        for g, table in enumerate(rec.tables):
            for page in table:
                if page != RELEASED:
                    self.pools[g].free(page)
        self._free_slots.append(rec.slot)
        del self.requests[request_id]

    # -- pages -----------------------------------------------------------------------
    def _first_needed_page(self, g: int, first_query_pos: int) -> int:
        """Logical page of the oldest key that a query at ``first_query_pos`` reads."""
        need = self.groups[g].need
        if need.kind != "window" or need.window <= 0:
            return 0
        return max(0, first_query_pos - need.window + 1) // self.page_size

    def pages_needed(self, request_id: Optional[Hashable], n_new: int, cached_len: Optional[int] = None) -> List[int]:
        """Pages per group that ``reserve(request_id, n_new)`` would take from the pools.
        For a request that is not live yet pass ``request_id=None`` and its ``cached_len`` (0)."""
        if request_id is not None:
            rec = self.record(request_id)
            have, base = [len(t) for t in rec.tables], rec.cached_len
        else:
            have, base = [0] * len(self.groups), cached_len or 0
        total = pages_for(base + n_new, self.page_size)
        out = []
        for g in range(len(self.groups)):
            first = self._first_needed_page(g, base)
            # Logical pages below `first` are never read: they need no physical page even
            # if they were never allocated (a window group joined late by a long portion).
            out.append(max(0, total - max(have[g], first)))
        return out

    def can_reserve(self, request_id: Optional[Hashable], n_new: int, cached_len: Optional[int] = None) -> bool:
        need = self.pages_needed(request_id, n_new, cached_len)
        return all(n <= pool.free_pages() for n, pool in zip(need, self.pools))

    def reserve(self, request_id: Hashable, n_new: int) -> None:
        """Cover positions cached_len .. cached_len+n_new-1 with pages in every group.
        Raises ``OutOfPages`` and changes nothing if any pool is short."""
        rec = self.record(request_id)
        if n_new < 1:
            raise CacheError("a step must bring at least one token for a request")
        if rec.reserved_len != rec.cached_len:
            raise CacheError(f"request {request_id!r} has an uncommitted reservation")
        need = self.pages_needed(request_id, n_new)
        for g, n in enumerate(need):
            if n > self.pools[g].free_pages():
                raise OutOfPages(
                    f"request {request_id!r} needs {n} pages in group {g}, {self.pools[g].free_pages()} free")
        total = pages_for(rec.cached_len + n_new, self.page_size)
        for g, table in enumerate(rec.tables):
            first = self._first_needed_page(g, rec.cached_len)
            while len(table) < total:
                table.append(RELEASED if len(table) < first else self.pools[g].allocate())
        rec.reserved_len = rec.cached_len + n_new

    def cancel(self, request_id: Hashable) -> None:
        """Undo a reservation that was not committed (pages beyond the cached length go back)."""
        rec = self.record(request_id)
        keep = pages_for(rec.cached_len, self.page_size)
        rec.edits += 1
        for g, table in enumerate(rec.tables):
            while len(table) > keep:
                page = table.pop()
                if page != RELEASED:
                    self.pools[g].free(page)
        rec.reserved_len = rec.cached_len

    def commit(self, request_id: Hashable, n_new: int) -> None:
        """The step ran: the new tokens are cached. Pages a window has passed go back."""
        rec = self.record(request_id)
        if rec.cached_len + n_new != rec.reserved_len:
            raise CacheError(
                f"commit of {n_new} tokens does not match the reservation of request {request_id!r}")
        rec.cached_len = rec.reserved_len
        for g, table in enumerate(rec.tables):
            first = min(self._first_needed_page(g, rec.cached_len), len(table))
            for j in range(first):
                if table[j] != RELEASED:
                    self.pools[g].free(table[j])
                    table[j] = RELEASED
                    rec.edits += 1

    # -- views -----------------------------------------------------------------------
    def table(self, request_id: Hashable, group: int) -> List[int]:
        return self.record(request_id).tables[group]

    def free_pages(self, group: int = 0) -> int:
        return self.pools[group].free_pages()

    def check_invariants(self) -> None:
        """Every page is either free or held by exactly as many tables as its count says."""
        for g, pool in enumerate(self.pools):
            held: Dict[int, int] = {}
            for rec in self.requests.values():
                for page in rec.tables[g]:
                    if page != RELEASED:
                        held[page] = held.get(page, 0) + 1
            free = list(pool._free)
            if len(set(free)) != len(free):
                raise CacheError(f"group {g}: a page is on the free list twice")
            if set(free) & set(held):
                raise CacheError(f"group {g}: a page is both free and held")
            if len(free) + len(held) != pool.capacity:
                raise CacheError(f"group {g}: {pool.capacity - len(free) - len(held)} pages are lost")
            for page, n in held.items():
                if pool.ref_count(page) != n:
                    raise CacheError(f"group {g}: page {page} is held {n} times, count says {pool.ref_count(page)}")
        slots = [r.slot for r in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise CacheError("a request slot is held twice")
        if len(slots) + len(self._free_slots) != self.n_slots:
            raise CacheError("a request slot is lost")
