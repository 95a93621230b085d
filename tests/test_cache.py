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
    with pytest.raises(PageError, match=r"held by \[1\]"):
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


def one_group(**kw):
    return manager([CacheEntry(i, i, PagedKV(2, 16), ()) for i in range(2)], prefix_cache=True, **kw)


def test_equal_prefixes_share_whole_pages():
    """A request starts on the pages that another one published for the same tokens: whole pages only, at least one
    token left to compute; the shared pages have both as holders and are kept, not freed, when both have gone."""
    m = one_group()
    g = m.groups[0]
    prompt = list(range(100, 111))                                    # 11 tokens: two whole pages and three tokens
    a = m.admit(prompt)
    assert int(m.computed[a]) == 0 and m.reserve(a, 11)
    m.advance(a, 11)
    m.publish(a, prompt)
    m.check()
    assert len(m.prefix) == 2 and all(g.pool.registered(p) for p in g.table[a, :2].tolist())
    assert not g.pool.registered(int(g.table[a, 2]))                  # the page that is not full stays private
    b = m.admit(prompt + [7, 8])
    assert int(m.computed[b]) == 8 and g.table[b, :2].tolist() == g.table[a, :2].tolist()
    assert g.pool.holders(int(g.table[a, 0])) == {a, b}
    c = m.admit(prompt[:8])                                           # all of it is cached: one token must be computed still
    assert int(m.computed[c]) == 4
    d = m.admit([1, 2, 3, 4] + prompt)                                # the same tokens elsewhere are another prefix
    assert int(m.computed[d]) == 0
    m.check()
    assert m.reserve(b, 13) and g.table[b, 2] != g.table[a, 2]        # b's own third page
    m.advance(b, 13)
    m.publish(b, prompt + [7, 8])                                     # its third block differs from nothing known: entered
    assert len(m.prefix) == 3
    free = g.pool.available
    for slot in (a, b, c, d):
        m.release(slot)
        m.check()
    assert g.pool.available == g.pool.pages and len(g.pool._kept) == 3 and free < g.pool.pages
    e = m.admit(prompt + [7, 8, 9])                                   # the kept pages serve the next request
    assert int(m.computed[e]) == 12 and len(g.pool._kept) == 0
    m.release(e)
    with pytest.raises(PageError):
        g.pool.share(int(g.table[e, 0]), 3)                           # (the null page: nothing to share)


def test_kept_pages_are_evicted_oldest_first_and_forgotten():
    m = one_group(pages=16, max_model_len=32)
    g = m.groups[0]
    first, second = list(range(50, 59)), list(range(70, 83))          # 2 and 3 whole pages
    for prompt in (first, second):
        s = m.admit(prompt)
        assert m.reserve(s, len(prompt))
        m.advance(s, len(prompt))
        m.publish(s, prompt)
        m.release(s)
    assert len(m.prefix) == 5 and len(g.pool._kept) == 5 and g.pool.available == 16
    s = m.admit([9] * 30)
    assert m.reserve(s, 30) and g.pool.available == 8                 # 8 pages: the 11 free ones sufficed
    assert len(m.prefix) == 5
    t = m.admit([8] * 32)
    assert m.reserve(t, 16) and len(g.pool._kept) == 4                # 4 pages: 3 free, then the one kept longest
    m.check()
    assert int(m.computed[m.admit(first)]) == 4                       # its leaf went first; the parent still serves
    assert len(m.prefix) == 3 + 1 and m.prefix.match(second)[0] > 0
    assert not m.reserve(t, 32) and m.reserve(t, 28) and len(g.pool._kept) == 0   # everything else is taken now
    assert m.prefix.match(second)[0] == 0 and len(m.prefix) == 1
    m.check()


def test_no_prefix_index_where_a_prompt_cannot_be_entered_in_the_middle():
    window = [CacheEntry(0, 0, PagedKV(2, 16), ()), CacheEntry(1, 1, PagedKV(2, 16, window=8), ())]
    state = [CacheEntry(0, 0, PagedKV(2, 16), (SlotState("sum", (4,), "float32"),))]
    assert manager(window, prefix_cache=True).prefix is not None
    assert manager(state, prefix_cache=True).prefix is None           # a state of fixed size has no copy to start from
    assert manager(prefix_cache=False).prefix is None and one_group().prefix is not None


def full_and_window(window=6, **kw):
    entries = [CacheEntry(0, 0, PagedKV(2, 16), ()), CacheEntry(1, 1, PagedKV(2, 16, window=window), ()),
               CacheEntry(2, 2, PagedKV(2, 16), ())]
    return manager(entries, prefix_cache=True, **kw)


def walk(m, slot, tokens, upto, step=3):
    """The request computes its tokens `step` at a time, publishing as it goes (as the engine does after every step)."""
    at = int(m.computed[slot])
    while at < upto:
        at = min(upto, at + step)
        assert m.reserve(slot, at)
        m.advance(slot, at)
        m.publish(slot, tokens)


def test_prefixes_are_shared_in_every_group_and_a_window_needs_only_what_reaches_into_it():
    """Two groups, one with a window of 6 on pages of 4: a request that starts after n shared blocks holds all n pages
    in the full group and, in the other, only those that position 4 n can still see."""
    m = full_and_window()
    full, near = m.groups
    assert near.decl.window == 6 and m.prefix.windows == (0, 6)
    prompt = list(range(200, 223))                                    # 23 tokens: five whole pages
    a = m.admit(prompt)
    walk(m, a, prompt, 23)
    m.check()
    assert len(m.prefix) == 5 and int(near.first[a]) == 4             # the window has let go of blocks 0 to 3 ...
    assert len(near.pool._kept) == 4 and len(full.pool._kept) == 0    # ... which are kept, not freed
    b = m.admit(prompt + [1, 2])
    assert int(m.computed[b]) == 20                                   # five blocks; the window sees positions 15 to 19
    assert full.table[b, :5].tolist() == full.table[a, :5].tolist()
    assert int(near.first[b]) == 3 and (near.table[b, :3] == near.null_page).all()
    assert near.table[b, 4] == near.table[a, 4] and near.pool.holders(int(near.table[b, 3])) == {b}
    assert len(near.pool._kept) == 3                                  # block 3 came out of the kept ones
    m.check()
    walk(m, b, prompt + [1, 2], 25)
    m.check()
    m.release(a)
    m.release(b)
    m.check()
    assert all(g.pool.available == g.pool.pages for g in m.groups)
    # the window's pool loses a page that the cut needs: the match falls back to a cut that needs none of the lost ones
    lost = m.prefix._pages_of[m.prefix.match(prompt)[2]][1]           # the window group's page of block 4
    m.prefix.evicted(1, lost)
    near.pool._kept.pop(lost)
    near.pool._registered.discard(lost)
    near.pool._free.append(lost)
    m.check()
    c = m.admit(prompt + [1, 2])
    assert int(m.computed[c]) == 16 and int(near.first[c]) == 2       # four blocks: positions 11 to 15 lie in blocks 2 and 3
    d = m.admit(prompt[:21])
    walk(m, d, prompt[:21], 21)                                       # block 4 again: its page fills the node's gap
    assert m.prefix._pages_of[m.prefix.match(prompt)[2]][1] == int(near.table[d, 4])
    e = m.admit(prompt + [5])
    assert int(m.computed[e]) == 20
    m.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_with_shared_prefixes_in_two_groups(seed):
    """As the test above with random traffic, with a full group and one with a window, in pools so small that kept pages
    are evicted in one group while the other still has them."""
    rng = random.Random(300 + seed)
    window = rng.choice([3, 6, 9])
    m = full_and_window(window=window, pages=rng.choice([16, 22, 30]), max_seqs=4)
    families = [[rng.randrange(1000) for _ in range(40)] for _ in range(3)]
    live: dict[int, tuple[list[int], int]] = {}
    hits = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.3 and len(live) < 4:
            tokens = families[rng.randrange(3)][:rng.choice([4, 9, 16, 23, 40])] + [rng.randrange(1000) for _ in range(rng.randrange(6))]
            slot = m.admit(tokens)
            hit = int(m.computed[slot])
            assert hit % 4 == 0 and hit < len(tokens)
            hits += hit
            live[slot] = (tokens, hit)
        elif op < 0.8 and live:
            slot = rng.choice(list(live))
            tokens, have = live[slot]
            want = min(len(tokens), have + rng.choice([1, 2, 5, 17]))
            if want > have and m.reserve(slot, want):
                m.advance(slot, want)
                m.publish(slot, tokens)
                live[slot] = (tokens, want)
        elif live:
            slot = rng.choice(list(live))
            m.release(slot)
            del live[slot]
        m.check()
        for g in m.groups:
            for slot, (tokens, have) in live.items():                  # every position the next token may read has a real page
                lo = max(0, have - g.decl.window + 1) if g.decl.window else 0
                assert all(p != g.null_page for p in g.table[slot, lo // 4: -(-have // 4)])
            for page in range(g.pool.pages):                           # a page with two holders holds the same tokens for both
                holders = sorted(g.pool.holders(page))
                if len(holders) > 1:
                    at = {g.table[s, :int(g.count[s])].tolist().index(page) for s in holders}
                    assert len(at) == 1
                    assert len({tuple(live[s][0][:(min(at) + 1) * 4]) for s in holders}) == 1
    assert hits > 0
    for slot in list(live):
        m.release(slot)
    m.check()
    assert all(g.pool.available == g.pool.pages for g in m.groups)


@pytest.mark.parametrize("seed", range(6))
def test_random_traffic_with_shared_prefixes_keeps_the_books(seed):
    """Requests drawn from a few prompt families (equal beginnings) come and go in random order in a pool too small
    for all of them: after every operation the books are right, every position a request may read has a page, and a
    request's shared pages are exactly those of its family's beginning."""
    rng = random.Random(100 + seed)
    m = one_group(pages=rng.choice([18, 24, 40]), max_seqs=5)
    g = m.groups[0]
    families = [[rng.randrange(1000) for _ in range(40)] for _ in range(3)]
    live: dict[int, tuple[list[int], int]] = {}
    for _ in range(500):
        op = rng.random()
        if op < 0.3 and len(live) < 5:
            tokens = families[rng.randrange(3)][:rng.choice([4, 9, 16, 23, 40])] + [rng.randrange(1000) for _ in range(rng.randrange(6))]
            slot = m.admit(tokens)
            hit = int(m.computed[slot])
            assert hit % 4 == 0 and hit < len(tokens)
            live[slot] = (tokens, hit)
        elif op < 0.8 and live:
            slot = rng.choice(list(live))
            tokens, have = live[slot]
            want = min(len(tokens), have + rng.choice([1, 2, 5, 17]))
            if want > have and m.reserve(slot, want):
                m.advance(slot, want)
                m.publish(slot, tokens)
                live[slot] = (tokens, want)
        elif live:
            slot = rng.choice(list(live))
            m.release(slot)
            del live[slot]
        m.check()
        for slot, (tokens, have) in live.items():
            assert all(p != g.null_page for p in g.table[slot, :-(-have // 4)])
        for page in range(g.pool.pages):                           # a page with two holders holds the same tokens for both
            holders = sorted(g.pool.holders(page))
            if len(holders) > 1:
                at = [g.table[s, :int(g.count[s])].tolist().index(page) for s in holders]
                assert len(set(at)) == 1
                blocks = {tuple(live[s][0][:(at[0] + 1) * 4]) for s in holders}
                assert len(blocks) == 1, "two requests share a page but not the tokens up to it"
    for slot in list(live):
        m.release(slot)
    m.check()
    assert g.pool.available == g.pool.pages
