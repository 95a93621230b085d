"""The cache manager on the host: pages are never lost, held twice or freed twice, under random orders of requests;
windows give back the pages they have passed; groups with different needs have pools of their own; slots of
fixed-size state are zeroed for a new request."""
from __future__ import annotations

import random

import pytest
import torch

from holon_b200.cache import CacheManager, OutOfPages, PageError, PagePool
from holon_b200.parts import CacheEntry, PagedKV, SlotState


def manager(entries=None, **kw):
    entries = entries or [CacheEntry(i, i, PagedKV(2, 16), ()) for i in range(3)]
    args = dict(page_size=4, max_seqs=4, max_model_len=64, dtype=torch.float32, device="cpu", pages=20)
    args.update(kw)
    return CacheManager(entries, **args)


def test_pool_hands_out_low_pages_first_and_reuses_freed_ones():
    pool = PagePool(6)
    assert pool.take(3, holder=0) == [0, 1, 2]
    assert pool.take(4, holder=1) is None and pool.available == 3          # all or nothing
    pool.give([1], holder=0)
    assert pool.take(2, holder=1) == [1, 3]                                # the freed page is used again first
    with pytest.raises(PageError, match="held by 1"):
        pool.give([1], holder=0)
    pool.give([0, 2], holder=0)
    with pytest.raises(PageError):
        pool.give([0], holder=0)                                           # freed twice
    with pytest.raises(PageError, match="no such page"):
        pool.give([9], holder=0)


def test_reserve_release_and_block_table():
    m = manager()
    a, b = m.admit(), m.admit()
    assert (a, b) == (0, 1)
    assert m.reserve(a, 9) and m.capacity(a) == 12
    g = m.groups[0]
    assert g.table[a, :3].tolist() == [0, 1, 2] and (g.table[a, 3:] == g.null_page).all()
    assert m.reserve(a, 12) and g.pool.available == 17                     # already covered: nothing taken
    assert m.reserve(b, 64) and g.pool.available == 1 and sorted(g.table[b, :16].tolist()) == list(range(3, 19))
    assert not m.reserve(a, 21) and m.capacity(a) == 12                    # needs 3 more, 1 free: nothing taken
    assert m.could_fit(a, 21, releasing=[b]) and not m.could_fit(a, 21)
    m.check()
    m.release(b)
    held_by_b = set(range(3, 19))
    assert m.reserve(a, 21) and set(g.table[a, 3:6].tolist()) <= held_by_b      # b's pages are used again
    m.check()
    with pytest.raises(KeyError):
        m.release(b)
    with pytest.raises(ValueError, match="max_model_len"):
        m.reserve(a, 65)
    w = g.write_index(torch.tensor([a, a]).numpy(), torch.tensor([0, 5]).numpy())
    assert w.tolist() == [g.table[a, 0] * 4, g.table[a, 1] * 4 + 1]


def test_pool_must_hold_one_longest_request():
    with pytest.raises(OutOfPages, match="max_model_len 64 needs 16"):
        manager(pages=15)
    entries = [CacheEntry(0, 0, PagedKV(2, 16), ())]
    per_page = 2 * 2 * 4 * 16 * 4
    m = manager(entries, pages=None, state_memory=per_page * 31)
    assert m.pages == 30                                                   # one page of the budget is the null page


def test_window_group_gives_pages_back_and_groups_have_own_pools():
    entries = [CacheEntry(0, 0, PagedKV(2, 16), ()), CacheEntry(1, 1, PagedKV(2, 16, window=6), ()),
               CacheEntry(2, 2, PagedKV(2, 16), ()), CacheEntry(3, 3, PagedKV(1, 32, window=6), ())]
    m = manager(entries)
    assert [g.entries for g in m.groups] == [[0, 2], [1], [3]]            # same needs share pages, others do not
    full, win = m.groups[0], m.groups[1]
    assert m.kv_of_entry[2].shape == (21, 2, 2, 4, 16) and m.kv_of_entry[3].shape == (21, 2, 1, 4, 32)
    s = m.admit()
    assert m.reserve(s, 20)
    m.advance(s, 20)                       # next token at 20 sees keys 15..19: pages 0..2 (keys 0..11) have passed
    assert win.first[s] == 3 and win.pool.available == 20 - 2 and full.pool.available == 15
    assert (win.table[s, :3] == win.null_page).all() and win.table[s, 3] != win.null_page
    m.check()
    assert m.reserve(s, 24)                # the window group's new page is one that was given back
    assert win.table[s, 5] in (0, 1, 2)
    m.advance(s, 24)
    m.check()
    m.release(s)
    assert win.pool.available == 20 and full.pool.available == 20
    m.check()


def test_slot_state_is_zeroed_on_admission():
    entries = [CacheEntry(0, 0, PagedKV(2, 16), (SlotState("sum", (3,)),)), CacheEntry(1, 1, None, (SlotState("sum", (5,), "int32"),))]
    m = manager(entries)
    assert m.slot_states[(0, "sum")].shape == (5, 3) and m.slot_states[(1, "sum")].dtype == torch.int32
    assert len(m.groups) == 1 and m.groups[0].entries == [0]              # an entry without pages joins no group
    s = m.admit()
    m.slot_states[(0, "sum")][s] = 7.0
    m.release(s)
    assert m.admit() == s and float(m.slot_states[(0, "sum")][s].abs().sum()) == 0.0


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_keeps_the_books(seed):
    rng = random.Random(seed)
    entries = [CacheEntry(0, 0, PagedKV(2, 16), ()), CacheEntry(1, 1, PagedKV(2, 16, window=rng.choice([3, 9, 17])), ())]
    m = manager(entries, pages=rng.choice([16, 19, 30]), max_seqs=5)
    live: dict[int, int] = {}
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 5:
            slot = m.admit()
            assert slot is not None and slot not in live
            live[slot] = 0
        elif op < 0.8 and live:
            slot = rng.choice(list(live))
            want = min(64, live[slot] + rng.choice([1, 1, 1, 2, 5, 17]))
            if want > live[slot] and m.reserve(slot, want):
                m.advance(slot, want)
                live[slot] = want
        elif live:
            slot = rng.choice(list(live))
            m.release(slot)
            del live[slot]
        m.check()
        for g in m.groups:                                 # every live position the next token may read has a real page
            for slot, n in live.items():
                lo = max(0, n - g.decl.window + 1) if g.decl.window else 0
                pages = g.table[slot, lo // 4: -(-n // 4)] if n else []
                assert all(p != g.null_page for p in pages)
    for slot in list(live):
        m.release(slot)
    m.check()
    assert all(g.pool.available == g.pool.pages for g in m.groups) and m.admit() is not None
