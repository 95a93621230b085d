"""Accounting of one pool of pages on the host: which are free, who holds the others, which are kept for reuse.

A page has a set of holders (request slots). Without a prefix index every page has one holder; with one, a page whose
content is registered there may be held by several requests at once, and when its last holder lets go it is not
freed but kept, oldest first in line to be taken again when the free list is empty
(core/holon/core/memory.py:28-133; core/holon/core/prefix.py:135-152). Giving back a page that the giver does not
hold (freed twice, or never taken) is an error here as there (memory.py:104-123).
"""
from __future__ import annotations

from collections import OrderedDict
from collections.abc import Callable


class OutOfPages(RuntimeError):
    """A pool is too small for what is asked of it at start (one request of the longest length must fit)."""


class PageError(RuntimeError):
    """A page was given back by someone who does not hold it."""


class PagePool:
    def __init__(self, pages: int) -> None:
        self.pages = pages
        self._free = list(range(pages - 1, -1, -1))          # pop() hands out low numbers first
        self._holders: list[set[int]] = [set() for _ in range(pages)]
        self._registered: set[int] = set()                   # pages whose content a prefix index knows
        self._kept: OrderedDict[int, None] = OrderedDict()   # registered, no holder: reusable as they are, or evictable
        self.on_evict: Callable[[int], None] | None = None   # told when a kept page is taken for something else

    @property
    def available(self) -> int:
        """Pages that `take` can hand out: the free ones and the kept ones."""
        return len(self._free) + len(self._kept)

    def take(self, n: int, holder: int) -> list[int] | None:
        """`n` pages for `holder`, or None (and nothing taken) if fewer are available. Freed pages are used again
        first; when none is free, the page kept longest is evicted."""
        if n > self.available:
            return None
        out = []
        for _ in range(n):
            if self._free:
                page = self._free.pop()
            else:
                page, _ = self._kept.popitem(last=False)
                self._registered.discard(page)
                if self.on_evict is not None:
                    self.on_evict(page)
            self._holders[page].add(holder)
            out.append(page)
        return out

    def give(self, pages, holder: int) -> None:
        for page in pages:
            if not 0 <= page < self.pages or holder not in self._holders[page]:
                held = sorted(self._holders[page]) if 0 <= page < self.pages else "nobody (no such page)"
                raise PageError(f"page {page} given back by {holder}, held by {held or 'nobody'}")
            self._holders[page].remove(holder)
            if not self._holders[page]:
                if page in self._registered:
                    self._kept[page] = None                   # newest last
                else:
                    self._free.append(page)

    def share(self, page: int, holder: int) -> None:
        """`holder` joins the holders of a registered page (taking it out of the kept ones if it had none)."""
        if page not in self._registered:
            raise PageError(f"page {page} is not registered: it cannot be shared")
        if holder in self._holders[page]:
            raise PageError(f"page {page} is held by {holder} already")
        self._kept.pop(page, None)
        self._holders[page].add(holder)

    def register(self, page: int) -> None:
        """The page's content is known to a prefix index from now on (it must be held)."""
        if not self._holders[page]:
            raise PageError(f"page {page} has no holder: it cannot be registered")
        self._registered.add(page)

    def registered(self, page: int) -> bool:
        return page in self._registered

    def holders(self, page: int) -> set[int]:
        return self._holders[page]

    def holder(self, page: int) -> int:
        """The one holder of a page that is not shared (-1: none)."""
        return next(iter(self._holders[page]), -1)

    def held_by(self, holder: int) -> list[int]:
        return [p for p, h in enumerate(self._holders) if holder in h]

    def check(self) -> None:
        """Every page is free, kept or held, and only one of these."""
        free, kept = set(self._free), set(self._kept)
        assert len(free) == len(self._free), "a page is twice in the free list"
        held = {p for p, h in enumerate(self._holders) if h}
        assert not free & kept and not free & held and not kept & held, "a page is in two states at once"
        assert len(free) + len(kept) + len(held) == self.pages, "a page is neither free, kept nor held"
        assert kept <= self._registered and not free & self._registered
