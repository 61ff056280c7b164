"""The cache's bookkeeping (the host runtime, csrc/host_runtime.cpp, through its Python face): no slot or
page lost, held twice or freed twice; the checks of a step; the packing of a step's rows (CPU; storage on the CPU
device is only memory, no kernel runs)."""
import random

import numpy as np
import pytest
import torch

from tq_kv_b200.cache import (CacheError, KVRequest, PageGroup, SequenceCache, SlotBook, StateRequest, StepError,
                              PAGE_TOKENS)


def test_slots_lowest_first_and_reuse():
    b = SlotBook(3, [], 100)
    assert [b.alloc(), b.alloc(), b.alloc()] == [0, 1, 2]
    with pytest.raises(CacheError, match="no free slot"):
        b.alloc()
    b.free(1)
    b.free(0)
    assert b.alloc() == 0 and b.alloc() == 1
    b.check()


def test_double_free_and_foreign_handles_raise():
    b = SlotBook(2, [], 100)
    s = b.alloc()
    b.free(s)
    with pytest.raises(CacheError, match="freed twice"):
        b.free(s)
    with pytest.raises(CacheError, match="does not exist"):
        b.free(5)
    with pytest.raises(CacheError, match="not held"):
        b.length(s)
    b.check()


def _book(slots=4, pages=8, ring=None, max_len=10_000):
    groups = [PageGroup("full", pages, PAGE_TOKENS, None)]
    if ring:
        groups.append(PageGroup("win", pages, PAGE_TOKENS, ring))
    return SlotBook(slots, groups, max_len)


def test_pages_follow_lengths_and_come_back():
    b = _book(ring=2)
    s = b.alloc()
    b.reserve([s], [65]); b.commit([s], [65])
    assert len(b.pages(0, s)) == 2 and len(b.pages(1, s)) == 2
    b.reserve([s], [64]); b.commit([s], [64])
    assert len(b.pages(0, s)) == 3 and len(b.pages(1, s)) == 2     # the ring stops growing
    assert b.pages(0, s) == [0, 1, 2]                              # pages are handed out lowest first
    b.check()
    b.free(s)
    assert b.free_pages(0) == 8 and b.free_pages(1) == 8 and not b.is_held(s)
    with pytest.raises(CacheError, match="freed twice"):
        b.free(s)
    b.check()


def test_reserve_is_all_or_nothing():
    b = _book(pages=3)
    s0, s1 = b.alloc(), b.alloc()
    b.reserve([s0], [100]); b.commit([s0], [100])                  # 2 pages
    before = (b.free_pages(0), b.lengths([s0, s1]))
    with pytest.raises(CacheError, match="is full"):
        b.reserve([s0, s1], [28, 65])                               # s0 fits in its pages, s1 needs 2, 1 is free
    assert (b.free_pages(0), b.lengths([s0, s1])) == before and b.pages(0, s1) == []
    with pytest.raises(CacheError, match="named twice"):
        b.reserve([s0, s0], [1, 1])
    with pytest.raises(CacheError, match="not held"):
        b.reserve([3], [1])
    with pytest.raises(CacheError, match="at least one token"):
        b.reserve([s0], [0])
    b.check()


def test_context_limit():
    b = _book(max_len=100)
    s = b.alloc()
    b.reserve([s], [100]); b.commit([s], [100])
    with pytest.raises(CacheError, match="context limit"):
        b.reserve([s], [1])


def test_random_walk_keeps_every_invariant():
    rng = random.Random(0)
    b = _book(slots=5, pages=12, ring=2)
    live, length = [], {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and len(live) < 5:
            s = b.alloc()
            assert s not in live                                # no slot is held twice
            live.append(s)
            length[s] = 0
        elif op < 0.5 and live:
            b.free(live.pop(rng.randrange(len(live))))
        elif live:
            rows = rng.sample(live, rng.randint(1, len(live)))
            n = [rng.randint(1, 90) for _ in rows]
            try:
                b.reserve(rows, n)
                b.commit(rows, n)
                for s, k in zip(rows, n):
                    length[s] += k
            except CacheError:
                pass
        b.check()
        held = [set(), set()]
        for gi, g in enumerate(b.groups):
            for s in live:
                pages = b.pages(gi, s)
                assert len(pages) >= g.pages_for_length(length[s]) and b.length(s) == length[s]
                assert not held[gi] & set(pages)                # no page is held by two slots
                held[gi] |= set(pages)
            assert len(held[gi]) == g.n_pages - b.free_pages(gi)    # and none is lost
    for s in live:
        b.free(s)
    b.check()
    assert all(b.free_pages(gi) == g.n_pages for gi, g in enumerate(b.groups)) and b.free_slots == 5


def test_sequence_cache_groups_and_state():
    kv = {0: KVRequest(2, 16, None), 1: KVRequest(2, 16, 100), 2: KVRequest(2, 16, None), 4: KVRequest(2, 16, 100)}
    st = {3: StateRequest((4, 2), torch.float32)}
    c = SequenceCache(kv, st, max_tokens=640, max_slots=3, max_length=512, dtype=torch.float32, device="cpu")
    assert len(c.groups) == 2
    full, win = c.groups
    assert full.entries == [0, 2] and win.entries == [1, 4] and win.ring_pages == 2 and full.ring_pages == 0
    assert tuple(full.k.shape) == (2, 10, 2, PAGE_TOKENS, 16) and tuple(win.k.shape) == (2, 6, 2, PAGE_TOKENS, 16)
    assert c.group_of_entry[2] == (0, 1) and c.group_of_entry[4] == (1, 1)
    s = c.alloc_slot()
    c.state[3][s] += 1.0
    c.reserve([s], [130]); c.commit([s], [130])
    rows, width = c.block_table_rows(0, [s])
    assert width == 3 and len(rows[0]) == 3
    rows, width = c.block_table_rows(1, [s])
    assert width == 2
    c.free_slot(s)
    s2 = c.alloc_slot()
    assert s2 == s and float(c.state[3][s2].abs().sum()) == 0.0          # state is zeroed when a slot is handed out
    assert c.length(s2) == 0 and c.free_pages() == 10


def test_trim_gives_back_pages_reserved_for_a_step_that_did_not_happen():
    b = _book(slots=2, pages=8, ring=2)
    s = b.alloc()
    b.reserve([s], [70])
    b.commit([s], [70])
    before = [b.pages(gi, s) for gi in range(2)]
    b.reserve([s], [200])                       # the step then fails: nothing is committed
    assert len(b.pages(0, s)) == 5
    b.trim([s])
    assert [b.pages(gi, s) for gi in range(2)] == before
    assert b.free_pages(0) == 6
    b.check()
    b.trim([s])                                 # nothing to give back: no change
    b.check()
    b.free(s)
    assert b.free_pages(0) == 8 and b.free_pages(1) == 8


def test_the_checks_of_a_step_refuse_before_anything_changes():
    b = _book(slots=3, pages=4)
    s0, s1 = b.alloc(), b.alloc()
    ok = dict(slots=[s0, s1], lens=[3, 1], tokens=[5, 6, 7, 8], want_counts=[2, 1], want=[0, 2, 0], sources=[-1, -1],
              vocab=10, source_rows=4)
    b.begin_step(**ok)
    for change, message in [
            (dict(lens=[0, 1], tokens=[8], want_counts=[0, 1], want=[0]), "Empty prompt"),
            (dict(tokens=[5, 6, 10, 8]), "token id 10 is outside the vocabulary"),
            (dict(tokens=[5, -1, 7, 8]), "outside the vocabulary"),
            (dict(want=[0, 3, 0]), "wanted place 3 is outside the 3 tokens"),
            (dict(slots=[s0, 2]), "slot 2 is not held"),
            (dict(sources=[1, -1]), "exactly one token"),
            (dict(sources=[-1, 4]), "exactly one token")]:
        with pytest.raises(StepError, match=message):
            b.begin_step(**{**ok, **change})
    b.begin_step(**{**ok, "sources": [-1, 3], "tokens": [5, 6, 7, 99]})    # a row fed on the device: its id is not looked at
    with pytest.raises(StepError, match="at least one row"):
        b.begin_step([], [], [], [], [], [], 10, 4)
    assert b.free_pages(0) == 4 and b.lengths([s0, s1]) == [0, 0]
    b.check()


def test_a_packed_step_holds_what_the_kernels_read():
    b = _book(slots=3, pages=6, ring=2)
    s0, s1 = b.alloc(), b.alloc()
    b.reserve([s0], [70]); b.commit([s0], [70])                    # s0 holds 70 tokens already
    slots, lens, tokens = [s1, s0], [3, 2], [11, 12, 13, 21, 22]
    want_counts, want, sources = [1, 2], [2, 0, 1], [-1, -1]
    b.reserve(slots, lens)
    lay = b.step_layout(slots, lens, want_counts)
    assert all(o % 4 == 0 for o in lay.offs) and lay.widths.tolist() == [2, 2]
    buf = np.full(lay.total, -7, dtype=np.int32)
    b.pack_step(slots, lens, tokens, want_counts, want, sources, lay, buf)
    o = lay.offs
    seg = lambda i, n: buf[o[i]:o[i] + n].tolist()
    assert seg(0, 5) == tokens and seg(1, 5) == [0, 0, 0, 1, 1] and seg(2, 5) == [0, 1, 2, 70, 71]
    assert seg(3, 3) == [0, 3, 5] and seg(4, 2) == [s1, s0] and seg(5, 2) == [0, 70] and seg(6, 2) == [3, 72]
    assert seg(7, 3) == [2, 3, 4] and seg(8, 5) == [-1] * 5
    assert seg(9, 4) == b.pages(0, s1) + [0] + b.pages(0, s0) and seg(10, 4) == b.pages(1, s1) + [0] + b.pages(1, s0)
    b.commit(slots, lens)
    # a decode step of the same two rows into a buffer of fixed layout: full-width tables
    offs = np.asarray([0, 4, 8, 12, 16, 20, 24, 28, 32, 36, 48], dtype=np.int32)
    widths = np.asarray([5, 2], dtype=np.int32)
    dec = np.full(60, -7, dtype=np.int32)
    b.reserve(slots, [1, 1])
    b.pack_decode(np.asarray(slots, dtype=np.int32), np.asarray([31, 0], dtype=np.int32),
                  np.asarray([-1, 3], dtype=np.int32), offs, widths, dec.ctypes.data)
    assert dec[0:2].tolist() == [31, 0] and dec[32:34].tolist() == [-1, 3] and dec[8:10].tolist() == [3, 72]
    assert dec[16:18].tolist() == [s1, s0] and dec[20:22].tolist() == [3, 72] and dec[24:26].tolist() == [4, 73]
    assert dec[36:37].tolist() == b.pages(0, s1) and dec[41:43].tolist() == b.pages(0, s0)
    assert dec[48:49].tolist() == b.pages(1, s1) and dec[50:52].tolist() == b.pages(1, s0)
    with pytest.raises(StepError, match="table has room for 1"):
        b.pack_decode(np.asarray(slots, dtype=np.int32), np.asarray([31, 0], dtype=np.int32),
                      np.asarray([-1, 3], dtype=np.int32), offs, np.asarray([1, 2], dtype=np.int32), dec.ctypes.data)
    b.check()


def test_ring_holds_the_window_plus_the_slack():
    from tq_kv_b200.cache import ring_pages_for
    assert ring_pages_for(16, 0) == 1 and ring_pages_for(64, 0) == 1 and ring_pages_for(65, 0) == 2
    assert ring_pages_for(64, 63) == 2 and ring_pages_for(128, 63) == 3 and ring_pages_for(16, 63) == 2
    for window in (8, 16, 64, 70, 128, 4096):
        for chunk in (1, 17, 64, 200):
            ring_tokens = ring_pages_for(window, chunk - 1) * PAGE_TOKENS
            assert ring_tokens - window + 1 >= chunk            # a step of `chunk` tokens always fits
    c = SequenceCache({0: KVRequest(1, 16, 64)}, {}, max_tokens=1024, max_slots=2, max_length=1024,
                      dtype=torch.float32, device="cpu", window_slack=63)
    assert c.groups[0].ring_pages == 2


def test_packed_steps_of_random_rows_equal_a_plain_packing():
    """The host runtime's packing against the same layout written out in plain Python, for random rows on a
    book in a random state (several groups, a ring, slots with history)."""
    rng = random.Random(3)
    for trial in range(40):
        groups = [PageGroup("full", 64, PAGE_TOKENS, None)]
        if trial % 2:
            groups.append(PageGroup("win", 32, PAGE_TOKENS, rng.randint(1, 3)))
        b = SlotBook(8, groups, 2000)
        slots = [b.alloc() for _ in range(rng.randint(1, 8))]
        for s in slots:                                             # some history
            n = rng.randint(0, 300)
            if n:
                b.reserve([s], [n]); b.commit([s], [n])
        rows = rng.sample(slots, rng.randint(1, len(slots)))
        lens = [rng.randint(1, 90) for _ in rows]
        tokens = [rng.randrange(1000) for _ in range(sum(lens))]
        wants = [sorted(rng.sample(range(n), rng.randint(0, min(n, 3)))) for n in lens]
        sources = [rng.randrange(8) if n == 1 and rng.random() < 0.5 else -1 for n in lens]
        b.begin_step(rows, lens, tokens, [len(w) for w in wants], [x for w in wants for x in w], sources, 1000, 8)
        b.reserve(rows, lens)
        lay = b.step_layout(rows, lens, [len(w) for w in wants])
        buf = np.full(lay.total, -9, dtype=np.int32)
        b.pack_step(rows, lens, tokens, [len(w) for w in wants], [x for w in wants for x in w], sources, lay, buf)
        # the same, written out
        starts = b.lengths(rows)
        T, B, R = sum(lens), len(rows), sum(len(w) for w in wants)
        cu = [0]
        for n in lens:
            cu.append(cu[-1] + n)
        widths = [max([len(b.pages(g, s)) for s in rows] + [1]) for g in range(len(groups))]
        segs = [tokens, [i for i, n in enumerate(lens) for _ in range(n)],
                [starts[i] + j for i, n in enumerate(lens) for j in range(n)], cu, rows, starts,
                [s + n for s, n in zip(starts, lens)], [cu[i] + x for i, w in enumerate(wants) for x in w],
                [sources[i] if j == 0 else -1 for i, n in enumerate(lens) for j in range(n)]]
        for g, w in enumerate(widths):
            table = []
            for s in rows:
                p = b.pages(g, s)
                table += p + [0] * (w - len(p))
            segs.append(table)
        assert lay.widths.tolist()[:len(groups)] == widths
        off = 0
        for i, seg in enumerate(segs):
            assert lay.offs[i] == off and buf[off:off + len(seg)].tolist() == list(seg), (trial, i)
            off += (max(len(seg), 1) + 3) // 4 * 4
        assert lay.total == off and (T, B, R) == (len(segs[0]), len(segs[4]), len(segs[7]))
        b.commit(rows, lens)
        b.check()
