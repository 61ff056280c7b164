"""The cache's bookkeeping: no slot or page lost, held twice or freed twice
(CPU; storage on the CPU device is only memory, no kernel runs)."""
import random

import pytest
import torch

from tq_kv_b200.cache import (CacheError, GroupPages, IndexPool, KVRequest, SequenceCache, SlotBook, StateRequest,
                              PAGE_TOKENS)


def test_index_pool_lowest_first_and_reuse():
    p = IndexPool(3, "slot")
    assert [p.take(), p.take(), p.take()] == [0, 1, 2]
    with pytest.raises(CacheError, match="no free slot"):
        p.take()
    p.give_back(1)
    p.give_back(0)
    assert p.take() == 0 and p.take() == 1
    p.check()


def test_double_free_and_foreign_handles_raise():
    p = IndexPool(2, "slot")
    s = p.take()
    p.give_back(s)
    with pytest.raises(CacheError, match="freed twice"):
        p.give_back(s)
    with pytest.raises(CacheError, match="does not exist"):
        p.give_back(5)
    p.check()


def _book(slots=4, pages=8, ring=None, max_len=10_000):
    groups = [GroupPages("full", pages, PAGE_TOKENS, None)]
    if ring:
        groups.append(GroupPages("win", pages, PAGE_TOKENS, ring))
    return SlotBook(slots, groups, max_len)


def test_pages_follow_lengths_and_come_back():
    b = _book(ring=2)
    s = b.alloc()
    b.reserve([s], [65]); b.commit([s], [65])
    assert len(b.groups[0].pages[s]) == 2 and len(b.groups[1].pages[s]) == 2
    b.reserve([s], [64]); b.commit([s], [64])
    assert len(b.groups[0].pages[s]) == 3 and len(b.groups[1].pages[s]) == 2     # the ring stops growing
    b.check()
    b.free(s)
    assert b.groups[0].pool.free_count == 8 and b.groups[1].pool.free_count == 8 and s not in b.length
    with pytest.raises(CacheError, match="freed twice"):
        b.free(s)
    b.check()


def test_reserve_is_all_or_nothing():
    b = _book(pages=3)
    s0, s1 = b.alloc(), b.alloc()
    b.reserve([s0], [100]); b.commit([s0], [100])                  # 2 pages
    before = (b.groups[0].pool.free_count, dict(b.length))
    with pytest.raises(CacheError, match="is full"):
        b.reserve([s0, s1], [28, 65])                               # s0 fits in its pages, s1 needs 2, 1 is free
    assert (b.groups[0].pool.free_count, dict(b.length)) == before and s1 not in b.groups[0].pages
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
    live = []
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and len(live) < 5:
            live.append(b.alloc())
        elif op < 0.5 and live:
            b.free(live.pop(rng.randrange(len(live))))
        elif live:
            rows = rng.sample(live, rng.randint(1, len(live)))
            n = [rng.randint(1, 90) for _ in rows]
            try:
                b.reserve(rows, n)
                b.commit(rows, n)
            except CacheError:
                pass
        b.check()
        for g in b.groups:
            for s in live:
                assert len(g.pages.get(s, [])) >= g.pages_for_length(b.length[s])
    for s in live:
        b.free(s)
    b.check()
    assert all(g.pool.free_count == g.pool.n for g in b.groups) and b.slots.free_count == 5


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
    before = {g.name: list(g.pages[s]) for g in b.groups}
    b.reserve([s], [200])                       # the step then fails: nothing is committed
    held = b.groups[0].pages[s]
    assert len(held) == 5
    b.trim([s])
    assert {g.name: g.pages[s] for g in b.groups} == before
    assert b.groups[0].pages[s] is not held     # a new list, so that cached views of the old one are seen stale
    assert b.groups[0].pool.free_count == 6
    b.check()
    b.trim([s])                                 # nothing to give back: no change
    b.check()
    b.free(s)
    assert b.groups[0].pool.free_count == 8 and b.groups[1].pool.free_count == 8


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
