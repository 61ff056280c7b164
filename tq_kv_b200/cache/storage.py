"""Device storage of the cache: key/value pages per group of layers and the
fixed-size state per sequence, above the host bookkeeping of `pool.py`.

Layout of a group: K is `[entries, pages, kv_heads, page_tokens, head_dim]`
and V the same with the value rows' width.  Token position p of a sequence lives in the sequence's logical
page p // page_tokens (modulo the ring length in a window group) at row
p % page_tokens; all layers of a group share the page numbering, so one block
table per group and step serves every layer of the group.

Keys are stored after the position encoding has been applied
(src/models/turbo_generic.rs:832-833 then :1606-1618).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .pool import CacheError, PageGroup, SlotBook

PAGE_TOKENS = 64


@dataclass(frozen=True)
class KVRequest:
    """What a mixer asks of the cache: per token and per each of `n_kv_heads`
    heads a key row of `head_dim` values and a value row of `value_dim` values
    (None: as wide as the key), of all earlier tokens (`window` None) or of
    the last `window` tokens.  What the rows mean is the mixer's business: a
    mixer that caches one latent per token asks for one head of the latent's
    width and may leave the value rows a single column."""
    n_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    value_dim: Optional[int] = None


@dataclass(frozen=True)
class StateRequest:
    """Fixed-size state per sequence: one tensor of `shape` and `dtype`,
    zeroed when a slot is handed out."""
    shape: tuple[int, ...]
    dtype: torch.dtype


@dataclass
class KVLayerView:
    """What a mixer sees of the cache during one step."""
    k_pages: torch.Tensor            # [pages, kv_heads, page_tokens, head_dim]
    v_pages: torch.Tensor            # [pages, kv_heads, page_tokens, value_dim]
    block_table: torch.Tensor        # int32 [rows, table_width], physical page per logical page
    table_width: int
    ring_pages: int                  # 0: all keys are kept
    page_tokens: int
    writes: bool                     # False: the layer reads another layer's cache


def ring_pages_for(window: int, slack: int) -> int:
    """Pages a sequence keeps in a window group.  A step that continues a
    sequence by n tokens writes all n keys before any of its queries reads, so
    the first query still finds its oldest key only if window + n - 1 keys fit:
    the ring holds `slack` keys more than the window (n <= slack + 1 always
    fits), rounded up to whole pages."""
    return -(-(window + max(0, slack)) // PAGE_TOKENS)


class KVGroup:
    def __init__(self, name: str, request: KVRequest, entries: list[int], n_pages: int, dtype, device,
                 window_slack: int = 0):
        self.name = name
        self.request = request
        self.entries = list(entries)
        ring = None
        if request.window is not None:
            ring = ring_pages_for(request.window, window_slack)
        self.book = PageGroup(name, n_pages, PAGE_TOKENS, ring)     # the group's geometry; the engine's SlotBook keeps its pages
        shape = (len(entries), n_pages, request.n_kv_heads, PAGE_TOKENS)
        self.k = torch.zeros((*shape, request.head_dim), dtype=dtype, device=device)
        self.v = torch.zeros((*shape, request.value_dim or request.head_dim), dtype=dtype, device=device)

    @property
    def ring_pages(self) -> int:
        return self.book.ring_pages or 0

    def bytes(self) -> int:
        return (self.k.numel() + self.v.numel()) * self.k.element_size()


class SequenceCache:
    """Slots, key/value groups and per-sequence state of one engine.

    `kv_requests` / `state_requests` map a schedule-entry index to what that
    entry's mixer asks for.  Entries with equal `KVRequest`s share a group.
    `max_tokens` is the number of tokens that live sequences may hold together
    (each sequence rounded up to whole pages)."""

    def __init__(self, kv_requests: dict[int, KVRequest], state_requests: dict[int, StateRequest], *,
                 max_tokens: int, max_slots: int, max_length: int, dtype: torch.dtype, device,
                 window_slack: int = 0):
        if max_tokens <= 0 or max_slots <= 0 or max_length <= 0:
            raise CacheError("cache sizes must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_slots = max_slots
        total_pages = -(-max_tokens // PAGE_TOKENS)
        by_request: dict[KVRequest, list[int]] = {}
        for entry in sorted(kv_requests):
            by_request.setdefault(kv_requests[entry], []).append(entry)
        self.groups: list[KVGroup] = []
        self.group_of_entry: dict[int, tuple[int, int]] = {}
        for gi, (req, entries) in enumerate(by_request.items()):
            if req.window is None:
                n_pages, name = total_pages, f"all-keys/{req.n_kv_heads}x{req.head_dim}"
            else:
                ring = ring_pages_for(req.window, window_slack)
                n_pages = min(total_pages, max_slots * ring)
                name = f"window-{req.window}/{req.n_kv_heads}x{req.head_dim}"
            g = KVGroup(name, req, entries, n_pages, dtype, self.device, window_slack)
            self.groups.append(g)
            for li, entry in enumerate(entries):
                self.group_of_entry[entry] = (gi, li)
        self.book = SlotBook(max_slots, [g.book for g in self.groups], max_length)
        self.state: dict[int, torch.Tensor] = {
            entry: torch.zeros((max_slots, *req.shape), dtype=req.dtype, device=self.device)
            for entry, req in state_requests.items()
        }

    # ---- slots -----------------------------------------------------------
    def alloc_slot(self) -> int:
        s = self.book.alloc()
        for t in self.state.values():
            t[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.book.free(slot)

    def length(self, slot: int) -> int:
        return self.book.length(slot)

    @property
    def free_slots(self) -> int:
        return self.book.free_slots

    # ---- one step ----------------------------------------------------------
    def reserve(self, slots: list[int], new_tokens: list[int]) -> None:
        self.book.reserve(slots, new_tokens)

    def commit(self, slots: list[int], new_tokens: list[int]) -> None:
        self.book.commit(slots, new_tokens)

    def trim(self, slots: list[int]) -> None:
        self.book.trim(slots)

    def block_table_rows(self, group: int, slots: list[int]) -> tuple[list[list[int]], int]:
        """The page lists of `slots` in group `group` and the widest of them."""
        rows = [self.book.pages(group, s) for s in slots]
        return rows, max((len(r) for r in rows), default=0)

    def layer_pages(self, entry: int) -> tuple[int, torch.Tensor, torch.Tensor]:
        gi, li = self.group_of_entry[entry]
        g = self.groups[gi]
        return gi, g.k[li], g.v[li]

    def free_pages(self) -> int:
        """Pages a new sequence can still get: the scarcest all-keys group
        decides (a window group never needs more pages than those)."""
        full = [self.book.free_pages(gi) for gi, g in enumerate(self.groups) if g.book.ring_pages is None]
        if full:
            return min(full)
        return min((self.book.free_pages(gi) for gi in range(len(self.groups))), default=1 << 30)

    def bytes(self) -> int:
        return sum(g.bytes() for g in self.groups) + sum(t.numel() * t.element_size() for t in self.state.values())
