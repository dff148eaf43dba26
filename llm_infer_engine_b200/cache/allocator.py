"""Host-side bookkeeping of the cache: which slots and pages are free, and who holds what.

Pure Python, no device: the rules (no slot or page lost, held twice or freed twice) are
tested without a GPU. The reference has no allocator: its cache row is the batch row and a new
cache is made per request (src/kv_cache.py:15-17, main.py:217).
"""
from __future__ import annotations

from typing import Dict, List


class CacheError(RuntimeError):
    """Out of slots or pages, or a slot or page handled wrongly."""


class FreeList:
    """Ids 0..n-1, handed out lowest first so that runs are reproducible; an id given back is
    handed out again."""

    def __init__(self, n: int, what: str):
        if n < 0:
            raise ValueError(f"number of {what}s must not be negative")
        self.n = n
        self.what = what
        self._free: List[int] = list(range(n - 1, -1, -1))   # pop() yields the lowest id
        self._held = [False] * n

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n - len(self._free)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} left (all {self.n} are held)")
        i = self._free.pop()
        self._held[i] = True
        return i

    def take_many(self, k: int) -> List[int]:
        if k > len(self._free):
            raise CacheError(f"{k} {self.what}s wanted but only {len(self._free)} of {self.n} are free")
        return [self.take() for _ in range(k)]

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is given back but is not held (freed twice?)")
        self._held[i] = False
        self._free.append(i)
        # keep lowest-first order cheaply: the list is small compared with a step's work
        if len(self._free) > 1 and self._free[-2] < i:
            self._free.sort(reverse=True)

    def check(self) -> None:
        """Every id is either free once or held, never both, never missing."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError(f"a {self.what} is in the free list twice")
        for i in range(self.n):
            if self._held[i] == (i in free):
                raise CacheError(f"{self.what} {i} is {'held and free' if self._held[i] else 'neither held nor free'}")


class PageTableHost:
    """Pages of one cache group, per slot: logical page number -> physical page.

    `window` > 0 means that only the last `window` positions of a sequence are ever read, so
    pages wholly below that range are given back after each step (`trim`)."""

    def __init__(self, n_pages: int, page_size: int, max_pages_per_seq: int, window: int = 0):
        self.pages = FreeList(n_pages, "page")
        self.page_size = page_size
        self.max_pages_per_seq = max_pages_per_seq
        self.window = window
        self._held: Dict[int, Dict[int, int]] = {}      # slot -> {logical page: physical page}

    def open_slot(self, slot: int) -> None:
        if slot in self._held:
            raise CacheError(f"slot {slot} is opened twice")
        self._held[slot] = {}

    def pages_needed(self, slot: int, old_len: int, new_len: int) -> int:
        """How many free pages `grow(slot, old_len, new_len)` would take."""
        if new_len <= old_len:
            return 0
        held = self._held[slot]
        return sum(1 for p in range(old_len // self.page_size, (new_len - 1) // self.page_size + 1)
                   if p not in held)

    def grow(self, slot: int, old_len: int, new_len: int) -> List[tuple]:
        """Makes positions old_len..new_len-1 writable. Returns [(logical, physical)] newly mapped."""
        held = self._held[slot]
        if new_len > self.max_pages_per_seq * self.page_size:
            raise CacheError(f"slot {slot}: length {new_len} exceeds the per-sequence limit "
                             f"{self.max_pages_per_seq * self.page_size}")
        first = old_len // self.page_size
        last = (new_len - 1) // self.page_size
        missing = [p for p in range(first, last + 1) if p not in held]
        phys = self.pages.take_many(len(missing))
        for lp, pp in zip(missing, phys):
            held[lp] = pp
        return list(zip(missing, phys))

    def trim(self, slot: int, length: int) -> List[int]:
        """Gives back pages that no later token of this slot can read (window groups only)."""
        if self.window <= 0:
            return []
        held = self._held[slot]
        first = max(0, length + 1 - self.window) // self.page_size
        dead = [lp for lp in held if lp < first]
        for lp in dead:
            self.pages.give_back(held.pop(lp))
        return dead

    def close_slot(self, slot: int) -> None:
        held = self._held.pop(slot, None)
        if held is None:
            raise CacheError(f"slot {slot} is closed but was not open")
        for pp in held.values():
            self.pages.give_back(pp)

    def held_pages(self, slot: int) -> Dict[int, int]:
        return dict(self._held[slot])

    def check(self) -> None:
        self.pages.check()
        seen = set()
        for slot, held in self._held.items():
            for pp in held.values():
                if pp in seen:
                    raise CacheError(f"page {pp} is held twice")
                if not self.pages.is_held(pp):
                    raise CacheError(f"page {pp} of slot {slot} is on the free list")
                seen.add(pp)
        if len(seen) != self.pages.n_held:
            raise CacheError(f"{self.pages.n_held - len(seen)} pages are held by no slot (lost)")
