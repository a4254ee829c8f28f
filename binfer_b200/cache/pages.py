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
    """Page ids ``1..num_pages``; id 0 is the scratch page and is never allocated.

    ``run``: pages per *run*, the pages that one tile of the attention kernels covers (128
    keys: eight 16-token pages).  The kernels fetch a tile whose pages lie side by side in
    the pool with one copy instead of one per page, so ``alloc`` tries to keep a request's
    pages that way, without ever refusing a page that is free: the page behind the
    request's last one if it is free; at the start of a tile the first page of a run that is
    wholly free (so that the request can grow into the rest of it); else the page freed
    last.  With ``run`` 1 it is the plain stack.
    """

    SCRATCH = 0

    def __init__(self, num_pages: int, run: int = 1):
        if num_pages < 1:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        self.run = max(1, int(run))
        # entries may be stale (the page was taken as a neighbour meanwhile): skipped when popped
        self._free: List[int] = list(range(self.num_pages, 0, -1))   # pop() gives 1 first
        self._held = bytearray(self.num_pages + 1)
        self._n_free = self.num_pages
        n_runs = -(-self.num_pages // self.run)
        self._run_free = [min(self.run, self.num_pages - r * self.run) for r in range(n_runs)]
        self._whole: List[int] = list(range(n_runs - 1, -1, -1)) if self.run > 1 else []

    @property
    def num_free(self) -> int:
        return self._n_free

    @property
    def num_held(self) -> int:
        return self.num_pages - self._n_free

    def _run_size(self, r: int) -> int:
        return min(self.run, self.num_pages - r * self.run)

    def _take(self, p: int) -> int:
        assert not self._held[p], f"page {p} handed out twice"
        self._held[p] = 1
        self._n_free -= 1
        self._run_free[(p - 1) // self.run] -= 1
        return p

    def alloc(self, after: int = 0, index: int = 0) -> int:
        """A free page.  ``after``: the request's last page (0: none), ``index``: the place
        in the request's block table that the new page takes."""
        if self._n_free <= 0:
            raise OutOfPages("page pool is empty")
        if self.run > 1:
            nxt = after + 1
            if (after > 0 and index % self.run and nxt <= self.num_pages
                    and not self._held[nxt]):
                return self._take(nxt)
            if index % self.run == 0:
                while self._whole:
                    r = self._whole.pop()
                    if self._run_free[r] == self._run_size(r):
                        return self._take(r * self.run + 1)
        while True:
            p = self._free.pop()
            if not self._held[p]:
                return self._take(p)

    def free(self, page: int) -> None:
        if page <= 0 or page > self.num_pages:
            raise ValueError(f"page id {page} is outside 1..{self.num_pages}")
        if not self._held[page]:
            raise ValueError(f"page {page} freed twice (or never allocated)")
        self._held[page] = 0
        self._n_free += 1
        self._free.append(page)
        r = (page - 1) // self.run
        self._run_free[r] += 1
        if self.run > 1 and self._run_free[r] == self._run_size(r):
            self._whole.append(r)
        if len(self._free) > 4 * self.num_pages + 64:      # drop the stale entries
            seen, keep = set(), []
            for p in reversed(self._free):
                if not self._held[p] and p not in seen:
                    seen.add(p)
                    keep.append(p)
            self._free = keep[::-1]
            self._whole = [r for r in dict.fromkeys(reversed(self._whole))
                           if self._run_free[r] == self._run_size(r)][::-1]

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
