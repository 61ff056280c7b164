"""Bookkeeping of the cache, all on the host and free of torch: which slots
are held, which pages each slot holds in each group, how long each sequence
is.  Every misuse (no slot left, a slot freed twice, a page held twice) raises
before anything is launched.

Reference: src/models/turbo_generic.rs:1606-1618 keeps one growing (K, V)
pair per layer for a single sequence and src/engine.rs:117 one `position`;
tq-kv/src/candle_kv.rs:53-153 shows the interface (append / current_seq_len /
reset) that a slot offers here per sequence.
"""
from __future__ import annotations


class CacheError(RuntimeError):
    """The cache cannot serve a request (capacity) or was misused."""


class IndexPool:
    """A pool of integer handles 0..n-1 (slots, or pages of one group).
    Handles are given out lowest first, so that a handle given back is used
    again soon — stale contents then show up in tests rather than in use."""

    def __init__(self, n: int, what: str):
        self.n = int(n)
        self.what = what
        self._free = list(range(self.n - 1, -1, -1))   # pop() yields the lowest
        self._held = [False] * self.n

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.n - len(self._free)

    def take(self) -> int:
        if not self._free:
            raise CacheError(f"no free {self.what} left (all {self.n} are held)")
        i = self._free.pop()
        if self._held[i]:
            raise CacheError(f"{self.what} {i} would be held twice")
        self._held[i] = True
        return i

    def give_back(self, i: int) -> None:
        if not 0 <= i < self.n:
            raise CacheError(f"{self.what} {i} does not exist (0..{self.n - 1})")
        if not self._held[i]:
            raise CacheError(f"{self.what} {i} is freed twice or was never held")
        self._held[i] = False
        # keep the free list sorted descending so that take() stays lowest-first
        lo, hi = 0, len(self._free)
        while lo < hi:
            mid = (lo + hi) // 2
            if self._free[mid] > i:
                lo = mid + 1
            else:
                hi = mid
        self._free.insert(lo, i)

    def is_held(self, i: int) -> bool:
        return 0 <= i < self.n and self._held[i]

    def check(self) -> None:
        """Invariant: every handle is either free or held, never both or neither."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise CacheError(f"a {self.what} is on the free list twice")
        for i in range(self.n):
            if (i in free) == self._held[i]:
                raise CacheError(f"{self.what} {i} is {'both free and held' if self._held[i] else 'lost'}")


class GroupPages:
    """Pages of one group of layers.  A sequence's logical page i (tokens
    i*page_tokens ..) lives in physical page `pages[slot][i]`; a ring group
    holds at most `ring_pages` pages per sequence and reuses them modulo."""

    def __init__(self, name: str, n_pages: int, page_tokens: int, ring_pages: int | None):
        self.name = name
        self.page_tokens = page_tokens
        self.ring_pages = ring_pages
        self.pool = IndexPool(n_pages, f"page of cache group '{name}'")
        self.pages: dict[int, list[int]] = {}

    def pages_for_length(self, length: int) -> int:
        n = -(-length // self.page_tokens)
        return n if self.ring_pages is None else min(n, self.ring_pages)

    def need(self, slot: int, new_length: int) -> int:
        n = -(-new_length // self.page_tokens)
        if self.ring_pages is not None and n > self.ring_pages:
            n = self.ring_pages
        have = self.pages.get(slot)
        n -= len(have) if have is not None else 0
        return n if n > 0 else 0

    def grow(self, slot: int, new_length: int) -> None:
        have = self.pages.setdefault(slot, [])
        for _ in range(self.need(slot, new_length)):
            have.append(self.pool.take())

    def release(self, slot: int) -> None:
        for p in self.pages.pop(slot, []):
            self.pool.give_back(p)


class SlotBook:
    """Slots, lengths and page lists of all groups together.  `reserve` is
    all-or-nothing: it checks every group's pool before it takes a page."""

    def __init__(self, max_slots: int, groups: list[GroupPages], max_length: int):
        self.slots = IndexPool(max_slots, "slot")
        self.groups = groups
        self.max_length = max_length
        self.length: dict[int, int] = {}

    def alloc(self) -> int:
        s = self.slots.take()
        self.length[s] = 0
        return s

    def free(self, slot: int) -> None:
        self.slots.give_back(slot)       # raises on a double free before any page moves
        for g in self.groups:
            g.release(slot)
        del self.length[slot]

    def reserve(self, slots: list[int], new_tokens: list[int]) -> None:
        """Pages for `new_tokens[i]` more tokens in `slots[i]`, for all rows or none."""
        if len(set(slots)) != len(slots):
            raise CacheError(f"a slot is named twice in one step: {slots}")
        for s, n in zip(slots, new_tokens):
            if not self.slots.is_held(s):
                raise CacheError(f"slot {s} is not held")
            if n <= 0:
                raise CacheError(f"slot {s}: a step must bring at least one token")
            if self.length[s] + n > self.max_length:
                raise CacheError(
                    f"slot {s}: {self.length[s]} cached + {n} new tokens exceed the context limit {self.max_length}")
        # pages each row needs in each group, counted once (a decode step of many rows passes here every token)
        new_lengths = [self.length[s] + n for s, n in zip(slots, new_tokens)]
        needs = []
        for g in self.groups:
            row = [g.need(s, length) for s, length in zip(slots, new_lengths)]
            want = sum(row)
            if want > g.pool.free_count:
                raise CacheError(
                    f"cache group '{g.name}' is full: the step needs {want} more pages of {g.page_tokens} tokens, "
                    f"{g.pool.free_count} of {g.pool.n} are free")
            needs.append(row if want else None)
        for g, row in zip(self.groups, needs):
            if row is None:
                continue
            for s, k in zip(slots, row):
                if k:
                    have = g.pages.setdefault(s, [])
                    for _ in range(k):
                        have.append(g.pool.take())

    def commit(self, slots: list[int], new_tokens: list[int]) -> None:
        for s, n in zip(slots, new_tokens):
            self.length[s] += n

    def trim(self, slots: list[int]) -> None:
        """Gives back the pages of `slots` beyond what their committed lengths
        need (pages reserved for a step that did not happen)."""
        for s in slots:
            if not self.slots.is_held(s):
                continue
            for g in self.groups:
                have = g.pages.get(s)
                if have is None:
                    continue
                keep = g.pages_for_length(self.length[s])
                if len(have) > keep:
                    for p in have[keep:]:
                        g.pool.give_back(p)
                    g.pages[s] = have[:keep]       # a new list: whoever remembers the old one sees the change

    def check(self) -> None:
        self.slots.check()
        for g in self.groups:
            g.pool.check()
            seen: set[int] = set()
            for s, pages in g.pages.items():
                if not self.slots.is_held(s):
                    raise CacheError(f"group '{g.name}' keeps pages for slot {s}, which is not held")
                for p in pages:
                    if p in seen or not g.pool.is_held(p):
                        raise CacheError(f"group '{g.name}': page {p} is held twice or not marked held")
                    seen.add(p)
            if len(seen) != g.pool.held_count:
                raise CacheError(f"group '{g.name}': {g.pool.held_count - len(seen)} pages are lost")
