"""The cache manager: paged keys and values with a block table per request, in groups.

A *group* is a set of schedule entries (layer executions) whose caches have the
same geometry and the same retention rule: same kv heads, head size and window.
Each group has a page pool and block tables of its own.  A page id is valid for
every entry of its group (the reference's one pool works the same way across
all layers, src/kv/paged.ts:71-81).  In a windowed group the pages that every
later query has passed are given back while the request is still running.

Beside the pages, every live request holds one *slot*: an index into
fixed-size per-request state tensors that mixers may ask for (this
architecture asks for none, so those tensors are empty).

Pages are allocated by ``reserve`` before a step for exactly the tokens the
step writes; a failure raises :class:`OutOfPages` and changes nothing (the
reference ignores the failure of ``extendSequence``, src/serve.ts:390,476).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

from .pages import OutOfPages, PagePool, SlotPool


@dataclass(frozen=True)
class KVNeed:
    """What one layer execution asks of the paged cache."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None     # None: every key is kept

    @property
    def group_key(self) -> Tuple[int, int, Optional[int]]:
        return (self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size that one layer execution keeps."""

    shape: Tuple[int, ...]
    dtype: str = "float32"


@dataclass
class RequestCache:
    rid: Hashable
    slot: int
    length: int = 0                            # tokens whose keys/values are cached
    tables: List[List[int]] = field(default_factory=list)   # per group: page id or -1
    fresh: bool = True                         # state slot not yet zeroed on the device
    # per group: the table as an int32 array for the step's batch description, kept in step
    # with `tables` (entries appended; rebuilt after a windowed page was released)
    np_tables: List[object] = field(default_factory=list)
    np_valid: List[int] = field(default_factory=list)

    def table_array(self, g: int):
        """``tables[g]`` as a numpy int32 array (a view of a cached buffer)."""
        import numpy as np
        table = self.tables[g]
        n = len(table)
        while len(self.np_tables) <= g:
            self.np_tables.append(None)
            self.np_valid.append(0)
        arr, valid = self.np_tables[g], self.np_valid[g]
        if arr is None or arr.shape[0] < n or valid < 0:
            arr = np.zeros(max(16, 2 * n), dtype=np.int32)
            arr[:n] = table
            self.np_tables[g] = arr
        elif valid < n:
            arr[valid:n] = table[valid:n]
        self.np_valid[g] = n
        return arr[:n]


def plan_pages(kv_needs: Sequence[Optional[KVNeed]], page_size: int, budget_bytes: int,
               element_size: int, max_requests: int, max_seq_len: int,
               max_tokens_per_step: int):
    """Share ``budget_bytes`` out among the cache groups; returns ``need -> pages`` for
    :class:`CacheManager`.

    A group that keeps every key needs ``max_seq_len`` tokens per request at most; a windowed
    one needs its window plus the longest portion a step may write (pages behind the window
    are given back before a step's new ones are taken) plus a page's slack at either end.
    Groups get pages in proportion to those needs, the windowed ones never more than
    ``max_requests`` requests can use; what that saves goes to the others.  (The reference
    has one pool, every layer alike: src/kv/paged.ts:55-62.)"""
    per_request, page_bytes = {}, {}
    for need in kv_needs:
        if need is None:
            continue
        key = need.group_key
        tokens = max_seq_len if need.window is None else min(
            max_seq_len, need.window + max_tokens_per_step)
        per_request[key] = -(-tokens // page_size) + 2
        page_bytes[key] = page_bytes.get(key, 0) + (
            2 * need.num_kv_heads * need.head_dim * page_size * element_size)
    # pages per unit of "request": scale every group's need by the same factor f
    unit = sum(per_request[k] * page_bytes[k] for k in per_request)
    f = min(float(max_requests), budget_bytes / unit) if unit else 0.0
    pages = {k: max(1, int(f * per_request[k])) for k in per_request}
    return lambda need: pages[need.group_key]


class CacheGroup:
    def __init__(self, index: int, need: KVNeed, num_pages: int, page_size: int):
        self.index = index
        self.need = need
        self.page_size = page_size
        # pages of one 128-key attention tile lie side by side in the pool where they can
        self.pool = PagePool(num_pages, run=max(1, 128 // page_size))
        self.entries: List[int] = []           # schedule entries stored here, in order
        self.storage = None                    # device tensor, see allocate_storage()

    def first_needed_page(self, length: int) -> int:
        """Index of the first logical page that a query at position >= ``length`` reads."""
        w = self.need.window
        if w is None:
            return 0
        first_key = max(0, length - w + 1)
        return first_key // self.page_size


class CacheManager:
    """Host-side bookkeeping; device storage is attached by ``allocate_storage``."""

    def __init__(self, kv_needs: Sequence[Optional[KVNeed]],
                 state_needs: Sequence[Optional[StateNeed]] = (),
                 page_size: int = 16, num_pages=64, max_requests: int = 64):
        """``num_pages``: pages of every group's pool, or a function of a group's
        :class:`KVNeed` that gives its pool's pages (a windowed group keeps far fewer keys
        per request than one that keeps them all: see :func:`plan_pages`)."""
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.page_size = int(page_size)
        pages_of = num_pages if callable(num_pages) else (lambda need: int(num_pages))
        self.groups: List[CacheGroup] = []
        # schedule entry -> (group index, index of the entry inside its group)
        self.entry_location: List[Optional[Tuple[int, int]]] = []
        by_key: Dict[Tuple, CacheGroup] = {}
        for e, need in enumerate(kv_needs):
            if need is None:
                self.entry_location.append(None)
                continue
            g = by_key.get(need.group_key)
            if g is None:
                g = CacheGroup(len(self.groups), need, int(pages_of(need)), self.page_size)
                by_key[need.group_key] = g
                self.groups.append(g)
            self.entry_location.append((g.index, len(g.entries)))
            g.entries.append(e)
        # the largest pool (what a request that keeps every key can draw on)
        self.num_pages = max([g.pool.num_pages for g in self.groups], default=0)
        self.state_needs = list(state_needs) + [None] * (len(kv_needs) - len(state_needs))
        self.slots = SlotPool(max_requests)
        self.requests: Dict[Hashable, RequestCache] = {}
        self.state_storage: List[object] = [None] * len(self.state_needs)

    # ------------------------------------------------------------- requests
    def add_request(self, rid: Hashable) -> RequestCache:
        if rid in self.requests:
            raise ValueError(f"request {rid!r} is already live")
        rc = RequestCache(rid, self.slots.alloc(), 0, [[] for _ in self.groups])
        self.requests[rid] = rc
        return rc

    def get(self, rid: Hashable) -> RequestCache:
        return self.requests[rid]

    def free_request(self, rid: Hashable) -> None:
        """Give back every page and the slot of ``rid``."""
        rc = self.requests.pop(rid)
        for g, table in zip(self.groups, rc.tables):
            for p in table:
                if p > 0:
                    g.pool.free(p)
            table.clear()
        self.slots.free(rc.slot)

    # ---------------------------------------------------------------- pages
    def pages_to_add(self, rc: RequestCache, new_len: int) -> List[int]:
        """Pages each group must newly allocate so that positions < ``new_len`` are
        covered, counting the pages that the step will release first."""
        out = []
        for g, table in zip(self.groups, rc.tables):
            want = -(-new_len // g.page_size)
            add = max(0, want - len(table))
            first = g.first_needed_page(rc.length)
            release = sum(1 for p in table[:first] if p > 0)
            out.append(add - release)
        return out

    def free_after(self, wants: Sequence[Tuple[Hashable, int]]) -> List[int]:
        """Free pages each group would have left after reserving every ``(rid, new_len)``
        (negative: that many pages short)."""
        need = [0] * len(self.groups)
        for rid, new_len in wants:
            rc = self.requests[rid]
            for i, n in enumerate(self.pages_to_add(rc, new_len)):
                need[i] += n
        return [g.pool.num_free - n for n, g in zip(need, self.groups)]

    def can_reserve(self, wants: Sequence[Tuple[Hashable, int]], spare: int = 0) -> bool:
        """Whether ``reserve`` would succeed for all ``(rid, new_len)`` together and still
        leave ``spare`` pages free in every group."""
        return all(n >= spare for n in self.free_after(wants))

    def reserve(self, rid: Hashable, new_len: int) -> None:
        """Make the block tables of ``rid`` cover positions < ``new_len``.

        Pages of a windowed group that lie wholly before the window of the
        request's next query are released first.  Raises :class:`OutOfPages`,
        with nothing changed, if any group lacks pages.
        """
        rc = self.requests[rid]
        if new_len < rc.length:
            raise ValueError(f"request {rid!r} holds {rc.length} tokens, cannot shrink to {new_len}")
        for g, n in zip(self.groups, self.pages_to_add(rc, new_len)):
            if n > g.pool.num_free:
                raise OutOfPages(
                    f"request {rid!r} needs {n} more pages in cache group {g.index}, "
                    f"{g.pool.num_free} free of {g.pool.num_pages}")
        for g, table in zip(self.groups, rc.tables):
            self._release_passed(g, rc, table)
            want = -(-new_len // g.page_size)
            while len(table) < want:
                table.append(g.pool.alloc(after=max(table[-1], 0) if table else 0,
                                          index=len(table)))

    def _release_passed(self, g: CacheGroup, rc: RequestCache, table: List[int]) -> None:
        first = min(g.first_needed_page(rc.length), len(table))
        for i in range(first):
            if table[i] > 0:
                g.pool.free(table[i])
                table[i] = -1
                if len(rc.np_valid) > g.index:
                    rc.np_valid[g.index] = -1      # the cached array is stale

    def commit(self, rid: Hashable, new_len: int) -> None:
        """Record that the step wrote keys/values up to ``new_len``."""
        rc = self.requests[rid]
        assert new_len >= rc.length
        for g, table in zip(self.groups, rc.tables):
            assert len(table) * g.page_size >= new_len, "commit beyond the reserved pages"
        rc.length = new_len

    def release_passed(self, rid: Hashable) -> None:
        """Give back windowed pages that the request's next query no longer reads."""
        rc = self.requests[rid]
        for g, table in zip(self.groups, rc.tables):
            self._release_passed(g, rc, table)

    # ---------------------------------------------------------------- views
    def num_free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def pages_for_tokens(self, n: int) -> int:
        """Pages one full-attention group needs for ``n`` tokens (src/kv/paged.ts:180)."""
        return -(-n // self.page_size)

    def can_ever_hold(self, n: int) -> bool:
        """Whether a lone request of ``n`` tokens fits every group's pool: all of its pages
        where every key is kept, its window's pages (and the one being written) elsewhere,
        where a long prompt can always come in short portions."""
        for g in self.groups:
            w = g.need.window
            need = -(-n // g.page_size) if w is None else -(-min(n, w + 1) // g.page_size) + 1
            if need > g.pool.num_pages:
                return False
        return True

    def check_consistent(self) -> None:
        """Every page is either free or held by exactly one live request."""
        for gi, g in enumerate(self.groups):
            seen = set()
            for rc in self.requests.values():
                for p in rc.tables[gi]:
                    if p > 0:
                        assert p not in seen, f"page {p} of group {gi} is held twice"
                        assert g.pool.is_held(p), f"page {p} of group {gi} is in a table but free"
                        seen.add(p)
            assert len(seen) == g.pool.num_held, (
                f"group {gi}: {g.pool.num_held} pages held, {len(seen)} in tables (a page is lost)")
        assert len(self.requests) == self.slots.num_slots - self.slots.num_free

    # -------------------------------------------------------------- storage
    def allocate_storage(self, dtype, device) -> None:
        """Device tensors: per group ``[entries, 2, pages + 1, kv_heads, page_size, head_dim]``
        (keys at index 0, values at 1; page 0 is scratch), and per schedule entry
        with a :class:`StateNeed` a tensor ``[slots, *shape]``."""
        import torch
        for g in self.groups:
            n = g.need
            g.storage = torch.zeros(
                (len(g.entries), 2, g.pool.num_pages + 1, n.num_kv_heads, g.page_size, n.head_dim),
                dtype=dtype, device=device)
        for e, need in enumerate(self.state_needs):
            if need is not None:
                self.state_storage[e] = torch.zeros(
                    (self.slots.num_slots,) + tuple(need.shape),
                    dtype=getattr(torch, need.dtype), device=device)

    def zero_fresh_state(self, rc: RequestCache) -> None:
        """Clear the state slot of a newly admitted request (its last owner's state is stale)."""
        if rc.fresh:
            for st in self.state_storage:
                if st is not None:
                    st[rc.slot].zero_()
            rc.fresh = False

    def kv_view(self, entry: int):
        """(keys, values) storage of schedule entry ``entry``: each
        ``[pages + 1, kv_heads, page_size, head_dim]``; and its group index."""
        gi, ei = self.entry_location[entry]
        st = self.groups[gi].storage
        return st[ei, 0], st[ei, 1], gi

    def storage_bytes(self) -> int:
        total = 0
        for g in self.groups:
            if g.storage is not None:
                total += g.storage.numel() * g.storage.element_size()
        return total
