"""A fixed pool of page ids with a free list and reference counts.

Same contract as llm-scheduler/src/block_allocator.rs:8-80: ids 0..capacity-1, pages are
handed out from the front of a FIFO free list and returned to its back, a page goes
back when its count drops to zero, and a double free or a bad id is an error.
"""
from __future__ import annotations

from collections import deque
from typing import Deque, List


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """The pool cannot cover what was asked. Nothing was allocated."""


class PagePool:
    def __init__(self, capacity: int):
        if capacity < 0:
            raise ValueError("capacity must not be negative")
        self.capacity = capacity
        self._free: Deque[int] = deque(range(capacity))
        self._refs: List[int] = [0] * capacity

    def free_pages(self) -> int:
        return len(self._free)

    def used_pages(self) -> int:
        return self.capacity - len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("out of pages in the cache pool")
        page = self._free.popleft()
        self._refs[page] = 1
        return page

    def allocate_many(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages asked, {len(self._free)} free")
        return [self.allocate() for _ in range(n)]

    def _check(self, page: int) -> None:
        if not 0 <= page < self.capacity:
            raise CacheError(f"invalid page id {page}")

    def increment_ref(self, page: int) -> None:
        self._check(page)
        if self._refs[page] == 0:
            raise CacheError(f"cannot share page {page}: it is not allocated")
        self._refs[page] += 1

    def ref_count(self, page: int) -> int:
        self._check(page)
        return self._refs[page]

    def free(self, page: int) -> bool:
        """Drop one reference; True if the page went back to the free list."""
        self._check(page)
        if self._refs[page] == 0:
            raise CacheError(f"double free of page {page}")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)
            return True
        return False
