"""An index of cached prompt prefixes: which pages hold the keys and values of which block of tokens.

A block is one page's worth of tokens. Its identity is its tokens and the block before it, so the index is a tree:
`(parent node, tokens of the block) -> node`. A node names one page per cache group (the groups have pools and page
numbers of their own), or none for a group whose page has gone: a group with a window lets go of the pages its
requests have passed, and a pool that runs short evicts the page kept longest. Nodes are numbered once and never
again, so a stale entry can never be mistaken for new content. A request that is admitted walks the tree along its
prompt and starts at the longest cut for which every group still has the pages that the next token can read: all of
them in a group of full attention, those that reach into the window in a group with one. A request whose computed
tokens fill a page enters it, unless the same block is known already (then its own copy stays private, except in a
group where the known node has lost its page: there it fills the gap). The pools keep entered pages whose holders have
all gone and evict the one kept longest when they need a page; a request lets go of its last block first, so leaves go
before their parents (core/holon/core/state.py:180-223; core/holon/core/prefix.py:135-152). A node whose parent has
lost all its pages can no longer be reached; its pages stay kept until their turn comes.

Only whole pages are shared, and a match always leaves at least one token to compute, so a shared page is never
written: a request writes at positions from its first uncomputed token on, which lie in pages of its own.
"""
from __future__ import annotations

from collections.abc import Sequence

ROOT = 0
DEAD = -1            # a chain that cannot be continued (its last block had no page left in any group)


class PrefixIndex:
    def __init__(self, page_size: int, windows: Sequence[int] = (0,)) -> None:
        """`windows`: per cache group its window (0: full attention)."""
        self.page_size, self.windows = page_size, tuple(windows)
        self._node: dict[tuple[int, tuple[int, ...]], int] = {}
        self._pages_of: dict[int, list[int | None]] = {}
        self._key_of: dict[int, tuple[int, tuple[int, ...]]] = {}
        self._node_of_page: list[dict[int, int]] = [{} for _ in self.windows]
        self._next = ROOT + 1
        self.hits = self.queries = 0                          # tokens found, tokens asked for

    def __len__(self) -> int:
        return len(self._node)

    def first_needed(self, group: int, blocks: int) -> int:
        """The first block whose page group `group` still needs when a request starts after `blocks` blocks."""
        w = self.windows[group]
        return max(0, blocks * self.page_size - w + 1) // self.page_size if w > 0 else 0

    def match(self, tokens: Sequence[int]) -> tuple[int, list[list[tuple[int, int]]], int]:
        """(blocks, per group the (block, page) pairs to share, the chain's node after `blocks` blocks) of the longest
        usable cut at the start of `tokens`, always leaving at least one token unmatched."""
        p, node, chain = self.page_size, ROOT, []
        for i in range((len(tokens) - 1) // p):
            found = self._node.get((node, tuple(tokens[i * p:(i + 1) * p])))
            if found is None:
                break
            node = found
            chain.append(node)
        groups = range(len(self.windows))
        run = [[0] * (len(chain) + 1) for _ in groups]       # run[g][n]: blocks in a row that end with block n - 1 and have g's page
        for g in groups:
            for n, node in enumerate(chain, 1):
                run[g][n] = run[g][n - 1] + 1 if self._pages_of[node][g] is not None else 0
        best = 0
        for n in range(len(chain), 0, -1):
            if all(run[g][n] >= n - self.first_needed(g, n) for g in groups):
                best = n
                break
        share = [[(i, self._pages_of[chain[i]][g]) for i in range(self.first_needed(g, best), best)] for g in groups]
        self.queries += len(tokens)
        self.hits += best * p
        return best, share, chain[best - 1] if best else ROOT

    def extend(self, node: int, block: Sequence[int], pages: Sequence[int | None]) -> tuple[int, list[bool]]:
        """The node of `block` after `node`, and per group whether `pages[group]` was entered for it (the caller must
        then register that page with the group's pool). A new block enters every page it is given; a known one only
        where its node had none. DEAD comes back for a new block without any page."""
        key = (node, tuple(block))
        found = self._node.get(key)
        if found is None:
            if node == DEAD or all(page is None for page in pages):
                return DEAD, [False] * len(pages)
            found, self._next = self._next, self._next + 1
            self._node[key], self._key_of[found], self._pages_of[found] = found, key, [None] * len(pages)
        have, entered = self._pages_of[found], []
        for g, page in enumerate(pages):
            entered.append(have[g] is None and page is not None)
            if entered[-1]:
                have[g] = page
                self._node_of_page[g][page] = found
        return found, entered

    def evicted(self, group: int, page: int) -> None:
        """The pool of `group` took a kept page for something else: its node forgets it, and is forgotten itself
        when it has no page left."""
        node = self._node_of_page[group].pop(page, None)
        if node is None:
            return
        have = self._pages_of[node]
        have[group] = None
        if all(p is None for p in have):
            del self._node[self._key_of.pop(node)]
            del self._pages_of[node]

    def pages(self, group: int = 0) -> set[int]:
        return set(self._node_of_page[group])
