"""Host-side bookkeeping of the cache: sequence slots and pages.

Both allocators refuse misuse loudly: a slot or page is never handed out twice, never
freed twice, and `check()` proves that none is lost.  The reference holds one sequence
and needs neither (core/model.hpp:29-54).
"""
from __future__ import annotations


class CacheFull(RuntimeError):
    """No free slot or page is left: the batch holds more than the cache was sized for."""


class SlotAllocator:
    """Slots 0..n-1, one per live sequence; freed slots are used again (lowest first)."""

    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise ValueError("a cache needs at least one slot")
        self.n = n_slots
        self._free = list(range(n_slots - 1, -1, -1))
        self._held = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n} sequence slots are in use")
        s = self._free.pop()
        self._held.add(s)
        return s

    def free(self, slot: int) -> None:
        if slot not in self._held:
            raise ValueError(f"slot {slot} is not held (freed twice, or never allocated)")
        self._held.remove(slot)
        self._free.append(slot)
        self._free.sort(reverse=True)

    def is_held(self, slot: int) -> bool:
        return slot in self._held

    @property
    def n_free(self) -> int:
        return len(self._free)

    def check(self) -> None:
        assert len(self._free) == len(set(self._free)), "a slot is on the free list twice"
        assert not (set(self._free) & self._held), "a slot is both free and held"
        assert len(self._free) + len(self._held) == self.n, "a slot was lost"


class PagePool:
    """Pages 0..n-1 of one cache group."""

    def __init__(self, n_pages: int):
        self.n = n_pages
        self._free = list(range(n_pages - 1, -1, -1))
        self._used = set()

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n} cache pages are in use")
        p = self._free.pop()
        self._used.add(p)
        return p

    def release(self, page: int) -> None:
        if page not in self._used:
            raise ValueError(f"page {page} is not in use (released twice?)")
        self._used.remove(page)
        self._free.append(page)

    @property
    def n_free(self) -> int:
        return len(self._free)

    def check(self) -> None:
        assert len(self._free) == len(set(self._free)), "a page is on the free list twice"
        assert not (set(self._free) & self._used), "a page is both free and used"
        assert len(self._free) + len(self._used) == self.n, "a page was lost"
