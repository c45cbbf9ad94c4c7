"""Host-side bookkeeping of cache pages and state slots (no device memory here).

``PagePool`` follows the reference's ``BlockPool`` (kv_cache.h:51-170,
kv_cache.cpp:52-101): pages carry a reference count; a page whose count drops to
zero goes to the front of the free list and allocation takes from the back, so the
page freed longest ago is reused first.  ``BlockTable`` is the reference's
per-request logical -> physical vector (kv_cache.h:175-243), with one addition: an
entry may be given back early (a window has passed it) and then reads ``-1``.
``StateSlots`` hands out fixed-size per-request state slots; the reference's nearest
notion is the running-slot index (decoder.cpp:123).
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Callable, List, Optional


class OutOfPages(RuntimeError):
    """The pool has fewer free pages than asked for."""


class CacheAccountingError(AssertionError):
    """A page or slot was freed twice, retained while free, or otherwise misused."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("num_pages must be >= 0")
        self.num_pages = num_pages
        self._ref: List[int] = [0] * num_pages
        # ordered front -> back; release puts a page at the front, allocate takes from the back
        self._free: "OrderedDict[int, None]" = OrderedDict((p, None) for p in range(num_pages - 1, -1, -1))
        # called with the page id when a free page is handed out again (its old content is about to be lost)
        self.on_allocate: Optional[Callable[[int], None]] = None

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def ref_count(self, page: int) -> int:
        return self._ref[page]

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free cache page")
        page, _ = self._free.popitem(last=True)
        if self._ref[page] != 0:
            raise CacheAccountingError(f"page {page} on the free list has reference count {self._ref[page]}")
        self._ref[page] = 1
        if self.on_allocate is not None:
            self.on_allocate(page)
        return page

    def take(self, page: int) -> None:
        """Take this particular free page (its content is wanted again: a prefix hit on a page
        nobody holds; kv_cache.h:147-158 take_from_free_list)."""
        if page not in self._free:
            raise CacheAccountingError(f"take of page {page} that is not free")
        del self._free[page]
        self._ref[page] = 1

    def retain(self, page: int) -> None:
        if self._ref[page] <= 0:
            raise CacheAccountingError(f"retain of free page {page}")
        self._ref[page] += 1

    def release(self, page: int) -> None:
        if not (0 <= page < self.num_pages) or self._ref[page] <= 0:
            raise CacheAccountingError(f"release of page {page} that is not held")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free[page] = None
            self._free.move_to_end(page, last=False)

    def check(self) -> None:
        """Every page is either free exactly once or held; raises otherwise."""
        free = set(self._free)
        for p in range(self.num_pages):
            if (self._ref[p] == 0) != (p in free):
                raise CacheAccountingError(f"page {p}: reference count {self._ref[p]} disagrees with the free list")


class BlockTable:
    """Logical page index -> physical page of one request in one cache group."""

    RELEASED = -1

    def __init__(self):
        self.pages: List[int] = []
        self.first_live = 0  # logical pages below this were given back early

    def __len__(self) -> int:
        return len(self.pages)

    def live_pages(self) -> List[int]:
        return [p for p in self.pages if p != self.RELEASED]


class StateSlots:
    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free state slot")
        s = self._free.pop()
        self._held[s] = True
        return s

    def release(self, slot: int) -> None:
        if not (0 <= slot < self.num_slots) or not self._held[slot]:
            raise CacheAccountingError(f"release of state slot {slot} that is not held")
        self._held[slot] = False
        self._free.append(slot)
