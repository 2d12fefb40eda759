"""A fixed pool of page ids with a free list and reference counts.

Same contract as llm-scheduler/src/block_allocator.rs:8-80: ids 0..capacity-1, pages are
handed out from the front of a FIFO free list and returned to its back, a page goes
back when its count drops to zero, and a double free or a bad id is an error. The pool
itself is C++ (``csrc/host/cache_manager.cpp``); this class holds its handle.
"""
from __future__ import annotations

from ctypes import byref, c_int, c_int32, c_void_p
from typing import List

from .. import host


class CacheError(RuntimeError):
    pass


class OutOfPages(CacheError):
    """The pool cannot cover what was asked. Nothing was allocated."""


class NoFreeSlot(CacheError):
    pass


_ERRORS = {host.CACHE_ERROR: CacheError, host.OUT_OF_PAGES: OutOfPages, host.NO_FREE_SLOT: NoFreeSlot,
           host.BAD_ARGUMENT: ValueError}


def check(status: int, names=None) -> None:
    """Raise the exception that belongs to a status of the host library. ``names`` maps the
    library's request numbers back to the caller's request ids for the message."""
    if status == host.OK:
        return
    msg = host.last_error()
    if names and "request #" in msg:
        head, _, tail = msg.partition("request #")
        digits = ""
        while tail and tail[0].isdigit():
            digits, tail = digits + tail[0], tail[1:]
        if digits and int(digits) in names:
            msg = f"{head}request {names[int(digits)]!r}{tail}"
    raise _ERRORS.get(status, CacheError)(msg)


class PagePool:
    def __init__(self, capacity: int):
        if capacity < 0:
            raise ValueError("capacity must not be negative")
        self.capacity = capacity
        self._lib = host.lib()
        self._handle = c_void_p()
        check(self._lib.llmrs_pool_create(capacity, byref(self._handle)))

    def __del__(self):
        if getattr(self, "_handle", None):
            self._lib.llmrs_pool_destroy(self._handle)
            self._handle = None

    def free_pages(self) -> int:
        free, cap = c_int(), c_int()
        check(self._lib.llmrs_pool_counts(self._handle, byref(free), byref(cap)))
        return free.value

    def used_pages(self) -> int:
        return self.capacity - self.free_pages()

    def allocate(self) -> int:
        page = c_int32()
        check(self._lib.llmrs_pool_allocate(self._handle, byref(page)))
        return page.value

    def allocate_many(self, n: int) -> List[int]:
        if n > self.free_pages():
            raise OutOfPages(f"{n} pages asked, {self.free_pages()} free")
        return [self.allocate() for _ in range(n)]

    def increment_ref(self, page: int) -> None:
        check(self._lib.llmrs_pool_increment_ref(self._handle, page))

    def ref_count(self, page: int) -> int:
        count = c_int()
        check(self._lib.llmrs_pool_ref_count(self._handle, page, byref(count)))
        return count.value

    def free(self, page: int) -> bool:
        """Drop one reference; True if the page went back to the free list."""
        back = c_int()
        check(self._lib.llmrs_pool_free(self._handle, page, byref(back)))
        return bool(back.value)
