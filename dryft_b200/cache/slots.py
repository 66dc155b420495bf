"""Host-side bookkeeping of the cache: which sequence holds which slot and which pages.

A *slot* is one live sequence's row of per-sequence state (its length, its page-table row, any
fixed-size mixer state).  A *page* is ``page_size`` consecutive token positions of keys and values
for every layer of one layer group.  A sequence holds exactly the pages that cover its tokens, so
the cache is sized in tokens, not in ``batch x longest sequence`` as the reference's static
``[layers, b_cap, kv_heads, l_cap, head_dim]`` tensor is (``engine/dryft_qwen3/cache.py:43-47``).

Nothing here touches a device: the allocators are plain Python and are tested on the CPU for
"no slot or page lost, held twice or freed twice".
"""

from __future__ import annotations

from typing import Dict, List, Optional


class CacheError(RuntimeError):
    """A request the cache cannot serve (no free slot, not enough pages, too long) or a misuse
    (a slot freed twice, a slot that is not held)."""


class FreeList:
    """Ids ``0..capacity-1``; each is either free or held, never both, never neither."""

    def __init__(self, capacity: int, what: str):
        if capacity <= 0:
            raise CacheError(f"{what} capacity must be positive, got {capacity}")
        self.capacity = capacity
        self.what = what
        # lowest id first, so that a freed id is the next one handed out: reuse is exercised early
        self._free: List[int] = list(range(capacity - 1, -1, -1))
        self._held = [False] * capacity

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.capacity - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.capacity and self._held[i]

    def take(self, n: int = 1) -> List[int]:
        if n < 0:
            raise CacheError(f"cannot take {n} {self.what}s")
        if n > len(self._free):
            raise CacheError(f"out of {self.what}s: {n} wanted, {len(self._free)} of {self.capacity} free")
        out = [self._free.pop() for _ in range(n)]
        for i in out:
            self._held[i] = True
        return out

    def give_back(self, ids: List[int]) -> None:
        for i in ids:
            if not 0 <= i < self.capacity:
                raise CacheError(f"{self.what} {i} does not exist (capacity {self.capacity})")
            if not self._held[i]:
                raise CacheError(f"{self.what} {i} freed twice (or never taken)")
        if len(set(ids)) != len(ids):
            raise CacheError(f"{self.what} list {ids} names an id twice")
        for i in ids:
            self._held[i] = False
        # keep "lowest id first" order
        self._free.extend(ids)
        self._free.sort(reverse=True)

    def check(self) -> None:
        """Invariant: every id is exactly once in (free list) xor (held)."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError(f"{self.what} free list holds an id twice")
        for i in range(self.capacity):
            if self._held[i] == (i in free):
                raise CacheError(f"{self.what} {i} is {'both held and free' if self._held[i] else 'lost'}")


def pages_for(n_tokens: int, page_size: int) -> int:
    return (n_tokens + page_size - 1) // page_size


class PageLedger:
    """The pages each slot holds in ONE layer group.

    ``window`` (tokens, or None): a group whose layers only ever read the last ``window`` keys
    gives pages back as soon as every position in them has fallen out of every future query's
    sight; the page-table entry then goes stale and is never read again.
    """

    def __init__(self, n_pages: int, page_size: int, max_pages_per_slot: int, window: Optional[int] = None):
        self.page_size = page_size
        self.max_pages_per_slot = max_pages_per_slot
        self.window = window
        self.pool = FreeList(n_pages, "page")
        self._pages: Dict[int, Dict[int, int]] = {}  # slot -> {logical page index -> physical page}

    def open(self, slot: int) -> None:
        if slot in self._pages:
            raise CacheError(f"slot {slot} already holds pages")
        self._pages[slot] = {}

    def first_live_page(self, next_pos: int) -> int:
        """Logical index of the first page a query at position >= next_pos can still see."""
        if self.window is None:
            return 0
        first_key = max(0, next_pos - self.window + 1)
        return first_key // self.page_size

    def pages_needed(self, cur_len: int, new_len: int) -> int:
        """Pages that growing a sequence from ``cur_len`` to ``new_len`` tokens takes from the pool
        (before any page is given back)."""
        return pages_for(new_len, self.page_size) - pages_for(cur_len, self.page_size)

    def grow(self, slot: int, cur_len: int, new_len: int) -> Dict[int, int]:
        """Make room for positions ``cur_len..new_len-1``.  Returns {logical page: physical page} of
        the pages added (what has to be written into the device page table)."""
        held = self._pages.get(slot)
        if held is None:
            raise CacheError(f"slot {slot} is not open")
        need_hi = pages_for(new_len, self.page_size)
        if need_hi > self.max_pages_per_slot:
            raise CacheError(
                f"sequence of {new_len} tokens exceeds the longest sequence the cache was built for "
                f"({self.max_pages_per_slot * self.page_size} tokens)"
            )
        first = pages_for(cur_len, self.page_size)
        wanted = [lp for lp in range(first, need_hi) if lp not in held]
        phys = self.pool.take(len(wanted))
        added = dict(zip(wanted, phys))
        held.update(added)
        return added

    def trim(self, slot: int, next_pos: int) -> List[int]:
        """Give back pages no future query (position >= next_pos) can see.  Only a windowed
        group ever returns any."""
        held = self._pages.get(slot)
        if held is None:
            raise CacheError(f"slot {slot} is not open")
        first = self.first_live_page(next_pos)
        dead = [lp for lp in held if lp < first]
        phys = [held.pop(lp) for lp in dead]
        self.pool.give_back(phys)
        return phys

    def close(self, slot: int) -> None:
        held = self._pages.pop(slot, None)
        if held is None:
            raise CacheError(f"slot {slot} holds no pages (freed twice?)")
        self.pool.give_back(list(held.values()))

    def held(self, slot: int) -> Dict[int, int]:
        return dict(self._pages.get(slot, {}))

    def check(self) -> None:
        self.pool.check()
        seen = set()
        for slot, held in self._pages.items():
            for p in held.values():
                if p in seen:
                    raise CacheError(f"page {p} is held twice")
                if not self.pool.is_held(p):
                    raise CacheError(f"page {p} of slot {slot} is on the free list")
                seen.add(p)
        if len(seen) != self.pool.n_held:
            raise CacheError(f"{self.pool.n_held - len(seen)} page(s) lost: held by no slot and not free")
