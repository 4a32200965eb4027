"""Host-side cache manager: pages, block tables and per-request state slots.

Layers are put into *groups* by what they need from the cache:

* ``full``   -- every key and value of the request stays (Qwen3 dense: one such group);
* ``window`` -- only the last ``window`` keys are read, so pages that the window has
  passed are given back while the request is still running;
* ``state``  -- a fixed-size slot per request (recurrent or convolution state), no pages.

Each paged group has pages of its own (its own allocator and device tensors) and
each request has one block table per paged group.  Beside the pages every request
holds one *state slot* index, even when no layer of the model keeps state.

Pages are reserved for a span of tokens, never for the whole prompt, are returned
when the request closes, is reset (preemption) or a window passes them, and are
handed out again first-in first-out.  This file is pure bookkeeping: it touches no
device memory.  Parity: qwen3_runtime/engine/block_manager.py:59-105, 264-311
(span allocation, capacity queries, FIFO free list); groups, windows and state
slots have no counterpart there.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

import numpy as np

FREED = -1  # block-table entry of a page that a window has passed


class CacheError(RuntimeError):
    """The cache was asked for something it cannot give (no page, no slot, misuse)."""


@dataclass(frozen=True)
class GroupSpec:
    """What one group of cache layers needs.  ``kind``: full | window | state."""

    kind: str
    window: int | None = None

    def __post_init__(self) -> None:
        if self.kind not in ("full", "window", "state"):
            raise ValueError(f"unknown cache group kind {self.kind!r}")
        if self.kind == "window" and (self.window is None or self.window < 1):
            raise ValueError("a window group needs window >= 1")

    @property
    def paged(self) -> bool:
        return self.kind != "state"


class PageAllocator:
    """Page ids ``0..num_pages-1`` with a first-in first-out free list and owner checks."""

    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise ValueError("num_pages must be positive")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(num_pages))
        self._held = [False] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise CacheError("page pool exhausted")
        page = self._free.popleft()
        if self._held[page]:
            raise CacheError(f"page {page} handed out twice")
        self._held[page] = True
        return page

    def release(self, page: int) -> None:
        if not 0 <= page < self.num_pages or not self._held[page]:
            raise CacheError(f"page {page} freed but not held")
        self._held[page] = False
        self._free.append(page)

    def held_pages(self) -> list[int]:
        return [p for p, h in enumerate(self._held) if h]


class SlotAllocator:
    """Fixed-size per-request state slots ``0..num_slots-1``."""

    def __init__(self, num_slots: int):
        if num_slots < 1:
            raise ValueError("num_slots must be positive")
        self.num_slots = num_slots
        self._free: deque[int] = deque(range(num_slots))
        self._held = [False] * num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise CacheError("no free state slot")
        slot = self._free.popleft()
        self._held[slot] = True
        return slot

    def release(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise CacheError(f"state slot {slot} freed but not held")
        self._held[slot] = False
        self._free.append(slot)


@dataclass
class RequestCache:
    """What one live request holds: a state slot and one block table per paged group."""

    request_id: object
    slot: int
    tables: list[list[int]]
    num_computed: int = 0  # tokens whose keys/values/state are in the cache
    num_reserved: int = 0  # tokens for which pages are reserved (>= num_computed)
    needs_state_reset: bool = True  # its slot must be zeroed before its next step
    closed: bool = field(default=False, repr=False)
    # int32 copies of ``tables`` kept in step with them, so that a step's block tables are
    # filled with array copies instead of per-element conversions
    table_arrays: list = field(default_factory=list, repr=False)

    def table_array(self, paged_index: int) -> np.ndarray:
        """The block table of one paged group as an int32 array (a view; do not keep it)."""
        return self.table_arrays[paged_index][: len(self.tables[paged_index])]

    def _append_page(self, paged_index: int, page: int) -> None:
        table = self.tables[paged_index]
        arr = self.table_arrays[paged_index]
        if len(table) >= arr.size:
            grown = np.empty(max(16, 2 * arr.size), dtype=np.int32)
            grown[: arr.size] = arr
            self.table_arrays[paged_index] = arr = grown
        arr[len(table)] = page
        table.append(page)


class CacheManager:
    def __init__(self, groups: list[GroupSpec], page_size: int, num_pages: int | list[int], num_slots: int):
        if page_size < 1:
            raise ValueError("page_size must be positive")
        self.groups = list(groups)
        self.page_size = page_size
        self.paged_groups = [i for i, g in enumerate(self.groups) if g.paged]
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.paged_groups)
        if len(num_pages) != len(self.paged_groups):
            raise ValueError("one page count per paged group is required")
        self.allocators = [PageAllocator(n) for n in num_pages]
        self.slots = SlotAllocator(num_slots)
        self.live: dict[object, RequestCache] = {}

    # ---- capacity -------------------------------------------------------------------
    def pages_for(self, num_tokens: int) -> int:
        return 0 if num_tokens <= 0 else -(-num_tokens // self.page_size)

    @property
    def num_free_pages(self) -> list[int]:
        return [a.num_free for a in self.allocators]

    @property
    def num_pages(self) -> list[int]:
        return [a.num_pages for a in self.allocators]

    def fits_at_all(self, num_tokens: int) -> bool:
        """Could a request of this many tokens ever be held, with the pool otherwise empty?"""
        need = self.pages_for(num_tokens)
        return all(need <= a.num_pages for a in self.allocators)

    def max_reservable(self, rc: RequestCache, limit: int) -> int:
        """Largest ``n <= limit`` such that tokens ``[computed, computed+n)`` fit in the
        pages the request holds plus the free ones, in every paged group."""
        if limit <= 0:
            return 0
        n = limit
        for table, alloc in zip(rc.tables, self.allocators):
            capacity = (len(table) + alloc.num_free) * self.page_size
            n = min(n, capacity - rc.num_computed)
        return max(0, n)

    def new_pages_needed(self, rc: RequestCache, num_tokens: int) -> list[int]:
        """Pages that :meth:`reserve` would take from each paged group's pool for these tokens."""
        need = self.pages_for(rc.num_computed + num_tokens)
        return [max(0, need - len(table)) for table in rc.tables]

    def can_reserve(self, rc: RequestCache, num_tokens: int) -> bool:
        return self.max_reservable(rc, num_tokens) >= num_tokens

    # ---- life cycle -----------------------------------------------------------------
    def open(self, request_id: object) -> RequestCache:
        if request_id in self.live:
            raise CacheError(f"request {request_id!r} is already open")
        rc = RequestCache(request_id, self.slots.allocate(), [[] for _ in self.paged_groups])
        rc.table_arrays = [np.empty(16, dtype=np.int32) for _ in self.paged_groups]
        self.live[request_id] = rc
        return rc

    def reserve(self, rc: RequestCache, num_tokens: int) -> None:
        """Grow the block tables so that tokens ``[computed, computed+num_tokens)`` have pages."""
        self._check_open(rc)
        if num_tokens < 0:
            raise ValueError("num_tokens must be non-negative")
        if not self.can_reserve(rc, num_tokens):
            raise CacheError("page pool exhausted")
        end = rc.num_computed + num_tokens
        need = self.pages_for(end)
        for pi, (table, alloc) in enumerate(zip(rc.tables, self.allocators)):
            while len(table) < need:
                rc._append_page(pi, alloc.allocate())
        rc.num_reserved = max(rc.num_reserved, end)

    def commit(self, rc: RequestCache, num_tokens: int) -> None:
        """Record that ``num_tokens`` more tokens are in the cache; free what windows passed."""
        self._check_open(rc)
        end = rc.num_computed + num_tokens
        if end > rc.num_reserved:
            raise CacheError("commit beyond the reserved span")
        rc.num_computed = end
        for gi, table, alloc in zip(self.paged_groups, rc.tables, self.allocators):
            group = self.groups[gi]
            if group.kind != "window":
                continue
            # the next query sits at position >= end and reads keys > end - window
            first_needed = max(0, end - group.window + 1)
            for idx in range(min(first_needed // self.page_size, len(table))):
                if table[idx] != FREED:
                    alloc.release(table[idx])
                    table[idx] = FREED
                    rc.table_arrays[self.paged_groups.index(gi)][idx] = FREED

    def reset(self, rc: RequestCache) -> None:
        """Give back every page and forget what was computed (preemption by recompute)."""
        self._check_open(rc)
        self._release_pages(rc)
        rc.num_computed = 0
        rc.num_reserved = 0
        rc.needs_state_reset = True

    def close(self, rc: RequestCache) -> None:
        self._check_open(rc)
        self._release_pages(rc)
        self.slots.release(rc.slot)
        rc.closed = True
        del self.live[rc.request_id]

    # ---- views ----------------------------------------------------------------------
    def first_live_token(self, rc: RequestCache, paged_index: int) -> int:
        """Lowest token position whose page is still held in that paged group."""
        for idx, page in enumerate(rc.tables[paged_index]):
            if page != FREED:
                return idx * self.page_size
        return len(rc.tables[paged_index]) * self.page_size

    def check_invariants(self) -> None:
        """No page lost, held twice, or both free and held.  For tests and debug runs."""
        for pi, alloc in enumerate(self.allocators):
            held = [p for rc in self.live.values() for p in rc.tables[pi] if p != FREED]
            if len(held) != len(set(held)):
                raise CacheError(f"group {pi}: a page is in two block tables")
            if sorted(held) != alloc.held_pages():
                raise CacheError(f"group {pi}: pages held by requests differ from pages marked held")
            free = list(alloc._free)
            if len(free) != len(set(free)) or set(free) & set(held):
                raise CacheError(f"group {pi}: free list is inconsistent")
            if len(free) + len(held) != alloc.num_pages:
                raise CacheError(f"group {pi}: {alloc.num_pages - len(free) - len(held)} pages lost")
        slots = [rc.slot for rc in self.live.values()]
        if len(slots) != len(set(slots)):
            raise CacheError("a state slot is held by two requests")

    # ---- internals ------------------------------------------------------------------
    def _check_open(self, rc: RequestCache) -> None:
        if rc.closed or self.live.get(rc.request_id) is not rc:
            raise CacheError(f"request {rc.request_id!r} is not open")

    def _release_pages(self, rc: RequestCache) -> None:
        for table, alloc in zip(rc.tables, self.allocators):
            for page in table:
                if page != FREED:
                    alloc.release(page)
            table.clear()
