"""Host-side bookkeeping of the cache: which pages and which slots are held.

Nothing here touches the device.  A page or a slot is either free or held by
exactly one owner; giving back what is not held, or taking more than there is,
raises.
"""
from __future__ import annotations


class CacheError(RuntimeError):
    pass


class CacheFull(CacheError):
    """More tokens or sequences are live than the cache was sized for."""


class PagePool:
    """A fixed set of page ids with a free list."""

    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise CacheError("a page pool cannot have a negative size")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))   # pop() hands out 0 first
        self._held = [False] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    @property
    def held_pages(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> list[int]:
        if n > len(self._free):
            raise CacheFull(f"the cache needs {n} more pages and has {len(self._free)} of {self.num_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def free(self, pages: list[int]) -> None:
        for p in pages:
            if not (0 <= p < self.num_pages) or not self._held[p]:
                raise CacheError(f"page {p} is given back but is not held")
            self._held[p] = False
            self._free.append(p)


class SlotTable:
    """Sequence slots: one per live sequence, used again after it ends."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def free_slots(self) -> int:
        return len(self._free)

    def is_held(self, slot: int) -> bool:
        return 0 <= slot < self.num_slots and self._held[slot]

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.num_slots} sequence slots are in use")
        s = self._free.pop()
        self._held[s] = True
        return s

    def free(self, slot: int) -> None:
        if not self.is_held(slot):
            raise CacheError(f"slot {slot} is given back but is not held")
        self._held[slot] = False
        self._free.append(slot)
