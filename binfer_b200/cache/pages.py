"""Free lists: pages of a key/value pool, and slots of fixed-size per-request state.

The reference keeps a ``Set`` of free block ids and hands them out in insertion
order (src/kv/paged.ts:138-155,160-168), so a freed block is reused last.  Here
the free list is a stack: the page freed last is handed out first, so a stale
block table or a missing write shows up at once.  Page 0 is never handed out:
padded rows of a captured decode step write there (the reference lets them
write into block 0 of a live request, src/engine/batched_engine.ts:2060-2078).
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """Not enough free pages (or state slots) for what was asked; nothing was changed."""


class PagePool:
    """Page ids ``1..num_pages``; id 0 is the scratch page and is never allocated."""

    SCRATCH = 0

    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages, 0, -1))   # pop() gives 1 first
        self._held = bytearray(self.num_pages + 1)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("page pool is empty")
        p = self._free.pop()
        assert not self._held[p], f"page {p} handed out twice"
        self._held[p] = 1
        return p

    def free(self, page: int) -> None:
        if page <= 0 or page > self.num_pages:
            raise ValueError(f"page id {page} is outside 1..{self.num_pages}")
        if not self._held[page]:
            raise ValueError(f"page {page} freed twice (or never allocated)")
        self._held[page] = 0
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return bool(self._held[page])


class SlotPool:
    """Slots ``0..num_slots-1`` for per-request state of fixed size."""

    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free: List[int] = list(range(self.num_slots - 1, -1, -1))
        self._held = bytearray(self.num_slots)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("no free request slot")
        s = self._free.pop()
        self._held[s] = 1
        return s

    def free(self, slot: int) -> None:
        if slot < 0 or slot >= self.num_slots or not self._held[slot]:
            raise ValueError(f"slot {slot} freed twice (or never allocated)")
        self._held[slot] = 0
        self._free.append(slot)
