"""An index of cached prompt prefixes: which page holds the keys and values of which block of tokens.

A block is one page's worth of tokens. Its identity is its tokens and the block before it, so the index is a tree:
`(parent node, tokens of the block) -> node`, a node naming one page. Nodes are numbered once and never again, so a
stale entry can never be mistaken for new content. A request that is admitted walks the tree along its prompt and
shares the pages it finds; a request whose computed tokens fill a page registers it, unless the same block is known
already (then its own copy stays private). The pool keeps registered pages whose holders have all gone and evicts the
one kept longest when it needs a page; a request lets go of its last block first, so leaves go before their parents
(core/holon/core/state.py:180-223; core/holon/core/prefix.py:135-152). A node whose parent was evicted can no longer
be reached; its page stays kept until its turn comes.

Only whole pages are shared, and a match always leaves at least one token to compute, so a shared page is never
written: a request writes at positions from its first uncomputed token on, which lie in pages of its own.
"""
from __future__ import annotations

from collections.abc import Sequence

ROOT = 0


class PrefixIndex:
    def __init__(self, page_size: int) -> None:
        self.page_size = page_size
        self._node: dict[tuple[int, tuple[int, ...]], int] = {}
        self._page_of: dict[int, int] = {}
        self._key_of: dict[int, tuple[int, tuple[int, ...]]] = {}
        self._node_of_page: dict[int, int] = {}
        self._next = ROOT + 1
        self.hits = self.queries = 0                          # tokens found, tokens asked for

    def __len__(self) -> int:
        return len(self._node)

    def match(self, tokens: Sequence[int]) -> tuple[list[int], int]:
        """Pages of the longest known chain of whole blocks at the start of `tokens`, always leaving at least one
        token unmatched, and the chain's last node."""
        p, node, pages = self.page_size, ROOT, []
        for i in range((len(tokens) - 1) // p):
            found = self._node.get((node, tuple(tokens[i * p:(i + 1) * p])))
            if found is None:
                break
            node = found
            pages.append(self._page_of[node])
        self.queries += len(tokens)
        self.hits += len(pages) * p
        return pages, node

    def extend(self, node: int, block: Sequence[int], page: int) -> tuple[int, bool]:
        """The node of `block` after `node`. If the block is new, `page` is entered for it (True: the caller must
        register the page with its pool); if it is known, the known node is returned and `page` stays private."""
        key = (node, tuple(block))
        found = self._node.get(key)
        if found is not None:
            return found, False
        new, self._next = self._next, self._next + 1
        self._node[key], self._page_of[new], self._key_of[new], self._node_of_page[page] = new, page, key, new
        return new, True

    def evicted(self, page: int) -> None:
        """The pool took a kept page for something else: its node is forgotten."""
        node = self._node_of_page.pop(page, None)
        if node is not None:
            del self._node[self._key_of.pop(node)]
            del self._page_of[node]

    def pages(self) -> set[int]:
        return set(self._node_of_page)
