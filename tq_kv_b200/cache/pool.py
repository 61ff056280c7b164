"""Bookkeeping of the cache and the host side of a step: which slots are held,
which pages each slot holds in each group, how long each sequence is; the
checks a step must pass before anything is launched; the packing of a step's
rows into one int32 buffer.  All of it lives in the host runtime
(csrc/host_runtime.cpp: C++, no CUDA, no torch); this module is its Python
face.  Every misuse (no slot left, a slot freed twice, a page held twice)
raises before anything is launched.

Reference: src/models/turbo_generic.rs:1606-1618 keeps one growing (K, V)
pair per layer for a single sequence and src/engine.rs:117 one `position`;
tq-kv/src/candle_kv.rs:53-153 shows the interface (append / current_seq_len /
reset) that a slot offers here per sequence.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_int, c_void_p
from dataclasses import dataclass
from typing import Optional, Sequence

import numpy as np

from ..csrc import build as _build


class CacheError(RuntimeError):
    """The cache cannot serve a request (capacity) or was misused."""


class StepError(ValueError):
    """A step that cannot run; raised before anything is launched."""


@dataclass(frozen=True)
class PageGroup:
    """Pages of one group of layers.  A sequence's logical page i (tokens
    i*page_tokens ..) lives in one physical page of the group; a ring group
    (`ring_pages` set) holds at most that many pages per sequence and reuses
    them modulo."""
    name: str
    n_pages: int
    page_tokens: int
    ring_pages: Optional[int] = None

    def pages_for_length(self, length: int) -> int:
        n = -(-length // self.page_tokens)
        return n if self.ring_pages is None else min(n, self.ring_pages)


_SIGNATURES = {
    "tqh_book_new": ([c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p], c_void_p),
    "tqh_book_delete": ([c_void_p], None),
    "tqh_error": ([c_void_p], c_char_p),
    "tqh_alloc": ([c_void_p], c_int),
    "tqh_free": ([c_void_p, c_int], c_int),
    "tqh_reserve": ([c_void_p, c_int, c_void_p, c_void_p], c_int),
    "tqh_commit": ([c_void_p, c_int, c_void_p, c_void_p], c_int),
    "tqh_trim": ([c_void_p, c_int, c_void_p], c_int),
    "tqh_length": ([c_void_p, c_int], c_int),
    "tqh_lengths": ([c_void_p, c_int, c_void_p, c_void_p], c_int),
    "tqh_is_held": ([c_void_p, c_int], c_int),
    "tqh_free_slots": ([c_void_p], c_int),
    "tqh_free_pages": ([c_void_p, c_int], c_int),
    "tqh_total_pages": ([c_void_p, c_int], c_int),
    "tqh_page_count": ([c_void_p, c_int, c_int], c_int),
    "tqh_pages": ([c_void_p, c_int, c_int, c_void_p, c_int], c_int),
    "tqh_check": ([c_void_p], c_int),
    "tqh_begin_step": ([c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int], c_int),
    "tqh_step_layout": ([c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p], c_int),
    "tqh_pack_step": ([c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_int, c_void_p], c_int),
    "tqh_pack_decode": ([c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p], c_int),
}
_lib = None


def host_library() -> ctypes.CDLL:
    """The host runtime, built at first use (a C++ compiler is all it needs)."""
    global _lib
    if _lib is None:
        lib = _build.load("host")
        for name, (argtypes, restype) in _SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes, fn.restype = argtypes, restype
        _lib = lib
    return _lib


def _ints(values) -> np.ndarray:
    """A contiguous int32 array of `values` (kept by the caller while the C side reads it)."""
    if isinstance(values, np.ndarray) and values.dtype == np.int32 and values.flags.c_contiguous:
        return values
    return np.ascontiguousarray(values, dtype=np.int32)


class StepLayout:
    """Where the segments of a packed step lie in its int32 buffer (see `SlotBook.step_layout`)."""
    __slots__ = ("offs", "widths", "total")

    def __init__(self, offs: np.ndarray, widths: np.ndarray, total: int):
        self.offs, self.widths, self.total = offs, widths, total


class SlotBook:
    """Slots, lengths and page lists of all groups together.  `reserve` is
    all-or-nothing: it checks every group's pool before it takes a page."""

    def __init__(self, max_slots: int, groups: Sequence[PageGroup], max_length: int):
        self._lib = host_library()
        self.groups = list(groups)
        self.max_slots, self.max_length = int(max_slots), int(max_length)
        n = len(self.groups)
        names = (c_char_p * max(n, 1))(*[g.name.encode() for g in self.groups])
        pages = _ints([g.n_pages for g in self.groups] or [0])           # (locals: alive while the C side reads them)
        tokens = _ints([g.page_tokens for g in self.groups] or [0])
        rings = _ints([g.ring_pages or 0 for g in self.groups] or [0])
        self._h = self._lib.tqh_book_new(self.max_slots, self.max_length, n, pages.ctypes.data, tokens.ctypes.data,
                                         rings.ctypes.data, ctypes.cast(names, c_void_p))
        if not self._h:
            raise CacheError("cache sizes must be positive")

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        lib = getattr(self, "_lib", None)
        if h and lib is not None:                          # (at interpreter exit the library may be gone already)
            try:
                lib.tqh_book_delete(h)
            except Exception:
                pass

    def _raise(self, code: int):
        msg = self._lib.tqh_error(self._h).decode()
        raise (StepError if code == -2 else CacheError)(msg)

    # ---- slots ----------------------------------------------------------------
    def alloc(self) -> int:
        s = self._lib.tqh_alloc(self._h)
        if s < 0:
            self._raise(s)
        return s

    def free(self, slot: int) -> None:
        r = self._lib.tqh_free(self._h, int(slot))
        if r:
            self._raise(r)

    def is_held(self, slot: int) -> bool:
        return bool(self._lib.tqh_is_held(self._h, int(slot)))

    def length(self, slot: int) -> int:
        n = self._lib.tqh_length(self._h, int(slot))
        if n < 0:
            raise CacheError(f"slot {slot} is not held")
        return n

    def lengths(self, slots) -> list[int]:
        """The lengths of several slots (-1 for one that is not held)."""
        s = _ints(slots)
        out = np.empty(max(len(s), 1), dtype=np.int32)
        self._lib.tqh_lengths(self._h, len(s), s.ctypes.data, out.ctypes.data)
        return out[:len(s)].tolist()

    @property
    def free_slots(self) -> int:
        return self._lib.tqh_free_slots(self._h)

    # ---- pages ----------------------------------------------------------------
    def reserve(self, slots, new_tokens) -> None:
        """Pages for `new_tokens[i]` more tokens in `slots[i]`, for all rows or none."""
        s, n = _ints(slots), _ints(new_tokens)
        r = self._lib.tqh_reserve(self._h, len(s), s.ctypes.data, n.ctypes.data)
        if r:
            self._raise(r)

    def commit(self, slots, new_tokens) -> None:
        s, n = _ints(slots), _ints(new_tokens)
        self._lib.tqh_commit(self._h, len(s), s.ctypes.data, n.ctypes.data)

    def trim(self, slots) -> None:
        """Gives back the pages of `slots` beyond what their committed lengths
        need (pages reserved for a step that did not happen)."""
        s = _ints(slots)
        r = self._lib.tqh_trim(self._h, len(s), s.ctypes.data)
        if r:
            self._raise(r)

    def free_pages(self, group: int) -> int:
        return self._lib.tqh_free_pages(self._h, group)

    def total_pages(self, group: int) -> int:
        return self._lib.tqh_total_pages(self._h, group)

    def pages(self, group: int, slot: int) -> list[int]:
        """The slot's physical pages in `group`, in logical order."""
        n = self._lib.tqh_page_count(self._h, group, int(slot))
        out = np.empty(max(n, 1), dtype=np.int32)
        self._lib.tqh_pages(self._h, group, int(slot), out.ctypes.data, n)
        return out[:n].tolist()

    def check(self) -> None:
        """Invariants: every slot and page is either free or held, never both
        or neither; a page is held once, by a slot that is held; every sequence
        has the pages its length needs."""
        r = self._lib.tqh_check(self._h)
        if r:
            self._raise(r)

    # ---- a step's rows ----------------------------------------------------------
    # Rows are given flat: lens[i] tokens of row i follow one another in `tokens`, want_counts[i] places in
    # `want`; sources[i] >= 0 names the row of the sampler's ids on the device that holds row i's one token.
    def begin_step(self, slots, lens, tokens, want_counts, want, sources, vocab: int, source_rows: int) -> None:
        """The checks of a step that need no device (raises StepError), nothing is changed."""
        s, n, t, wc, w = _ints(slots), _ints(lens), _ints(tokens), _ints(want_counts), _ints(want)
        src = _ints(sources) if sources is not None else None
        r = self._lib.tqh_begin_step(self._h, len(s), s.ctypes.data, n.ctypes.data, t.ctypes.data, wc.ctypes.data,
                                     w.ctypes.data, src.ctypes.data if src is not None else None, int(vocab),
                                     int(source_rows))
        if r:
            self._raise(r)

    def step_layout(self, slots, lens, want_counts) -> StepLayout:
        """Offsets of tokens | tok_seq | tok_pos | cu_seqlens | slots | start_pos | new_lens | logit_rows |
        tok_src | one block table per group in the packed buffer, the tables' widths, the buffer's length."""
        s, n, wc = _ints(slots), _ints(lens), _ints(want_counts)
        offs = np.empty(9 + len(self.groups), dtype=np.int32)
        widths = np.empty(max(len(self.groups), 1), dtype=np.int32)
        total = self._lib.tqh_step_layout(self._h, len(s), s.ctypes.data, n.ctypes.data, wc.ctypes.data,
                                          offs.ctypes.data, widths.ctypes.data)
        return StepLayout(offs, widths, total)

    def pack_step(self, slots, lens, tokens, want_counts, want, sources, layout: StepLayout, buf: np.ndarray) -> None:
        """Fills `buf` (int32, `layout.total` words) for rows whose pages are reserved."""
        s, n, t, wc, w = _ints(slots), _ints(lens), _ints(tokens), _ints(want_counts), _ints(want)
        src = _ints(sources) if sources is not None else None
        r = self._lib.tqh_pack_step(self._h, len(s), s.ctypes.data, n.ctypes.data, t.ctypes.data, wc.ctypes.data,
                                    w.ctypes.data, src.ctypes.data if src is not None else None,
                                    layout.offs.ctypes.data, layout.widths.ctypes.data, layout.total, buf.ctypes.data)
        if r:
            self._raise(r)

    def pack_decode(self, slots: np.ndarray, tokens: np.ndarray, sources: np.ndarray, offs: np.ndarray,
                    widths: np.ndarray, buf_address: int) -> None:
        """What changes from one decode step to the next (tokens, sources, positions, slots, lengths, block
        tables) of B one-token rows, written into a buffer of fixed layout at `buf_address`."""
        r = self._lib.tqh_pack_decode(self._h, len(slots), slots.ctypes.data, tokens.ctypes.data, sources.ctypes.data,
                                      offs.ctypes.data, widths.ctypes.data, buf_address)
        if r:
            self._raise(r)
