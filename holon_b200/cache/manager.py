"""The cache manager: pages of keys and values with a block table per request, in groups; request slots; state of
fixed size per request.

A group is a set of cache entries whose mixers asked for the same thing (`PagedKV`: heads, head size, window). One
page number of a group names the same page in each of its entries, so a request has one block-table row per group.
Groups have pools of their own, sized to hold the same number of tokens
(core/holon/core/memory.py:327-330; core/holon/core/assembly.py:140-189). A page goes back to its pool when its
request ends, or, in a group with a window, when every position in it lies before the window of the next token
(core/holon/core/state.py:398-418, 499-517). The last page of each pool's tensor is the null page: never handed
out, it stands in every unused block-table cell (memory.py:49-54).

With `prefix_cache` whole pages of prompts are shared between requests through `prefix.PrefixIndex`, in every group
at once: `admit(tokens)` starts a request on the pages of the longest known prefix of its tokens for which every
group still has what the next token can read (a group with a window needs only the pages that reach into it),
`publish(slot, tokens)` enters the pages its computed tokens have filled. A model with state of fixed size gets no
index: such a state cannot be entered in the middle of a prompt without a copy of it taken there.

Slots: a request holds one slot from admission to release; the slot is its row in every block table and in every
per-request tensor (state.py:154, 183-186). Mixers may declare state of fixed size (`SlotState`); it is zeroed when
a request takes the slot.
"""
from __future__ import annotations

import functools
import math

import numpy as np
import torch

from ..parts.base import PagedKV
from .pages import OutOfPages, PagePool
from .prefix import DEAD, ROOT, PrefixIndex


class CacheGroup:
    def __init__(self, index: int, decl: PagedKV, entries: list[int], page_size: int, max_seqs: int,
                 max_model_len: int, pages: int, dtype: torch.dtype, device) -> None:
        self.index, self.decl, self.entries, self.page_size = index, decl, list(entries), page_size
        self.max_pages = math.ceil(max_model_len / page_size)
        self.pool = PagePool(pages)
        self.null_page = pages
        self.table = np.full((max_seqs + 1, self.max_pages), self.null_page, dtype=np.int32)   # the host block table
        self.first = np.zeros(max_seqs + 1, dtype=np.int64)       # first logical page still held
        self.count = np.zeros(max_seqs + 1, dtype=np.int64)       # logical pages reserved so far
        self.dirty: set[int] = set()
        self.kv = torch.zeros((len(entries), pages + 1, 2, decl.kv_heads, page_size, decl.head_dim), dtype=dtype,
                              device=device)
        self.table_device = torch.from_numpy(self.table).to(device)

    @staticmethod
    def page_bytes(decl: PagedKV, entries: int, page_size: int, itemsize: int) -> int:
        return entries * 2 * decl.kv_heads * page_size * decl.head_dim * itemsize

    def need(self, slot: int, tokens: int) -> int:
        return max(0, math.ceil(tokens / self.page_size) - int(self.count[slot]))

    def grow(self, slot: int, tokens: int) -> bool:
        n = self.need(slot, tokens)
        if n == 0:
            return True
        pages = self.pool.take(n, slot)
        if pages is None:
            return False
        at = int(self.count[slot])
        self.table[slot, at:at + n] = pages
        self.count[slot] = at + n
        self.dirty.add(slot)
        return True

    def shrink_to(self, slot: int, pages: int) -> None:
        """Undo of `grow`: give back logical pages from `pages` on (a reservation that another group refused)."""
        at = int(self.count[slot])
        if pages < at:
            self.pool.give(self.table[slot, pages:at].tolist(), slot)
            self.table[slot, pages:at] = self.null_page
            self.count[slot] = pages
            self.dirty.add(slot)

    def passed(self, slot: int, computed: int) -> None:
        """With a window W the next token (position `computed`) reads keys after computed − W only: pages that end
        at or before computed − W + 1 go back."""
        w = self.decl.window
        if w <= 0:
            return
        keep_from = max(0, computed - w + 1) // self.page_size
        first = int(self.first[slot])
        if keep_from > first:
            keep_from = min(keep_from, int(self.count[slot]))
            self.pool.give(self.table[slot, first:keep_from].tolist(), slot)
            self.table[slot, first:keep_from] = self.null_page
            self.first[slot] = keep_from
            self.dirty.add(slot)

    def release(self, slot: int) -> None:
        first, count = int(self.first[slot]), int(self.count[slot])
        self.pool.give(self.table[slot, first:count].tolist()[::-1], slot)     # the last block first: kept leaves go first
        self.table[slot, :count] = self.null_page
        self.first[slot] = self.count[slot] = 0
        self.dirty.add(slot)

    def take_dirty(self) -> tuple[np.ndarray, np.ndarray]:
        """(slots [n], rows [n, max_pages]) of the block-table rows that changed since the last call, as copies: the
        host table may change again at once (a window lets go of pages, a request ends) while the step that these
        rows were taken for is still on its way to the device. The caller uploads them with the step's other arrays
        and scatters them into `table_device` ahead of the step's kernels."""
        slots = np.array(sorted(self.dirty), dtype=np.int32)
        self.dirty.clear()
        return slots, self.table[slots]

    def write_index(self, slots: np.ndarray, positions: np.ndarray) -> np.ndarray:
        """page · page_size + offset for each (slot, position) of a step's tokens."""
        p = self.page_size
        return self.table[slots, positions // p].astype(np.int64) * p + positions % p


class CacheManager:
    def __init__(self, entries, page_size: int, max_seqs: int, max_model_len: int, dtype: torch.dtype, device,
                 state_memory: int | None = None, pages: int | None = None, prefix_cache: bool = False) -> None:
        """`entries`: the model's `CacheEntry` list. Give either `state_memory` (bytes for all pools together) or
        `pages` (pages per pool). `prefix_cache`: share whole pages of equal prompt prefixes between requests, in
        all groups; it takes effect unless a part keeps state of fixed size (which cannot be entered in the middle of
        a prompt)."""
        self.page_size, self.max_seqs, self.max_model_len = page_size, max_seqs, max_model_len
        self.dtype, self.device = dtype, torch.device(device)
        by_decl: dict[PagedKV, list[int]] = {}
        for e in entries:
            if e.decl is not None:
                by_decl.setdefault(e.decl, []).append(e.entry)
        itemsize = torch.empty((), dtype=dtype).element_size()
        per_page = sum(CacheGroup.page_bytes(d, len(es), page_size, itemsize) for d, es in by_decl.items())
        least = math.ceil(max_model_len / page_size)
        if pages is None:
            if state_memory is None:
                raise ValueError("CacheManager needs state_memory or pages")
            pages = (state_memory // per_page - 1) if per_page else 0
        if by_decl and pages < least:
            raise OutOfPages(f"the cache pools hold {pages} pages of {page_size} tokens each; one request of "
                             f"max_model_len {max_model_len} needs {least} ({least * per_page} bytes and one page more)")
        self.pages = pages
        self.groups = [CacheGroup(i, d, es, page_size, max_seqs, max_model_len, pages, dtype, device)
                       for i, (d, es) in enumerate(by_decl.items())]
        self.group_of_entry = {e: g for g in self.groups for e in g.entries}
        self.kv_of_entry = {e: g.kv[i] for g in self.groups for i, e in enumerate(g.entries)}
        self.bytes = sum(g.kv.numel() * g.kv.element_size() for g in self.groups)
        self._free_slots = list(range(max_seqs - 1, -1, -1))
        self.live: set[int] = set()
        self.computed = np.zeros(max_seqs + 1, dtype=np.int64)
        self.padding_slot = max_seqs
        self.slot_states: dict[tuple[int, str], torch.Tensor] = {}
        self.chunk = 1                       # prompts are cut at multiples of this: the least common multiple of the
        for e in entries:                    # chunks that the fixed-size states ask for
            for s in e.slot_states:
                self.chunk = math.lcm(self.chunk, max(1, int(getattr(s, "chunk", 1))))
                self.slot_states[(e.entry, s.name)] = torch.zeros((max_seqs + 1, *s.shape),
                                                                  dtype=getattr(torch, s.dtype), device=device)
        self.prefix: PrefixIndex | None = None
        if prefix_cache and self.groups and not self.slot_states:
            self.prefix = PrefixIndex(page_size, [max(0, g.decl.window) for g in self.groups])
            for g in self.groups:
                g.pool.on_evict = functools.partial(self.prefix.evicted, g.index)
        self._chain_node = np.full(max_seqs + 1, ROOT, dtype=np.int64)    # per slot: the index node of its last known block
        self._chain_blocks = np.zeros(max_seqs + 1, dtype=np.int64)      # and how many blocks lead there

    # ---- slots
    def admit(self, tokens=None) -> int | None:
        """A free slot (lowest first), its fixed-size state zeroed; None if every slot is taken. With a prefix index
        and the request's `tokens`, the slot starts on the pages of the longest known prefix: `computed[slot]` says
        how many tokens those hold (whole pages, at least one token is left to compute)."""
        if not self._free_slots:
            return None
        slot = self._free_slots.pop()
        self.live.add(slot)
        self.computed[slot] = 0
        self._chain_node[slot], self._chain_blocks[slot] = ROOT, 0
        for t in self.slot_states.values():
            t[slot].zero_()
        if self.prefix is not None and tokens is not None:
            blocks, share, node = self.prefix.match(tokens)
            if blocks:
                for g, cells in zip(self.groups, share):
                    for i, page in cells:
                        g.pool.share(page, slot)
                        g.table[slot, i] = page
                    g.first[slot] = self.prefix.first_needed(g.index, blocks)     # (a window: the blocks before it are not held)
                    g.count[slot] = blocks
                    g.dirty.add(slot)
                self.computed[slot] = blocks * self.page_size
                self._chain_node[slot], self._chain_blocks[slot] = node, blocks
        return slot

    def publish(self, slot: int, tokens) -> None:
        """Enters the pages that the request's computed tokens have filled into the prefix index. `tokens`: the
        request's tokens as far as the host knows them (a token still on the device is left for the next call)."""
        if self.prefix is None:
            return
        p = self.page_size
        known = min(len(tokens), int(self.computed[slot]))
        i, node = int(self._chain_blocks[slot]), int(self._chain_node[slot])
        while (i + 1) * p <= known and node != DEAD:
            pages = [int(g.table[slot, i]) if i >= int(g.first[slot]) else None for g in self.groups]   # None: passed by the window
            node, entered = self.prefix.extend(node, tokens[i * p:(i + 1) * p], pages)
            for g, page, new in zip(self.groups, pages, entered):
                if new:
                    g.pool.register(page)
            i += 1
        self._chain_node[slot], self._chain_blocks[slot] = node, i

    def release(self, slot: int) -> None:
        if slot not in self.live:
            raise KeyError(f"slot {slot} is not live")
        for g in self.groups:
            g.release(slot)
        self.live.remove(slot)
        self.computed[slot] = 0
        self._free_slots.append(slot)

    # ---- pages
    def reserve(self, slot: int, tokens: int) -> bool:
        """Pages so that the request holds positions below `tokens` in every group: all of them or none."""
        if tokens > self.max_model_len:
            raise ValueError(f"{tokens} tokens exceed max_model_len {self.max_model_len}")
        before = [int(g.count[slot]) for g in self.groups]
        for g in self.groups:
            if not g.grow(slot, tokens):
                for h, n in zip(self.groups, before):
                    h.shrink_to(slot, n)
                return False
        return True

    def capacity(self, slot: int) -> int:
        """Tokens the slot's pages hold now (the smallest over the groups)."""
        return min((int(g.count[slot]) * g.page_size for g in self.groups), default=self.max_model_len)

    def advance(self, slot: int, tokens: int) -> None:
        """The request now holds `tokens` computed positions; windows let go of the pages they have passed."""
        self.computed[slot] = tokens
        for g in self.groups:
            g.passed(slot, tokens)

    def could_fit(self, slot: int | None, tokens: int, releasing=()) -> bool:
        """Whether `reserve(slot, tokens)` would succeed once the slots in `releasing` were released."""
        gone = set(releasing)
        for g in self.groups:
            freed = {page for s in gone for page in g.table[s, int(g.first[s]):int(g.count[s])].tolist()
                     if g.pool.holders(page) <= gone}             # (a page shared with a request that stays is not freed)
            have = g.pool.available + len(freed)
            need = math.ceil(tokens / g.page_size) - (int(g.count[slot]) if slot is not None else 0)
            if need > have:
                return False
        return True

    def free_tokens(self) -> int:
        return min((g.pool.available * g.page_size for g in self.groups), default=self.max_model_len)

    # ---- checks (tests call this after every operation)
    def check(self) -> None:
        """No page lost, none both free and held; a page held by two requests is one the prefix index knows; tables
        agree with the pools."""
        for g in self.groups:
            g.pool.check()
            held: dict[int, set[int]] = {}
            for slot in range(self.max_seqs + 1):
                first, count = int(g.first[slot]), int(g.count[slot])
                row = g.table[slot]
                if slot not in self.live:
                    assert count == 0 and (row == g.null_page).all(), f"slot {slot} is free but holds pages"
                    continue
                assert (row[:first] == g.null_page).all() and (row[count:] == g.null_page).all()
                pages = row[first:count].tolist()
                assert len(set(pages)) == len(pages), f"slot {slot} holds a page twice"
                for page in pages:
                    assert 0 <= page < g.pool.pages, f"slot {slot} holds page {page}"
                    held.setdefault(page, set()).add(slot)
            for page, slots in held.items():
                assert g.pool.holders(page) == slots, f"page {page}: table says {slots}, pool says {g.pool.holders(page)}"
                assert len(slots) == 1 or g.pool.registered(page), f"page {page} is shared by {slots} but not registered"
            assert len(held) + g.pool.available == g.pool.pages, "a page is neither available nor held"
            assert all(not g.pool.holders(p) for p in range(g.pool.pages) if p not in held), "a page is held by no table"
        if self.prefix is not None:
            for g in self.groups:
                assert all(g.pool.registered(p) for p in self.prefix.pages(g.index)), \
                    "the index names a page that is not registered"
