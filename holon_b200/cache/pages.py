"""Accounting of one pool of pages on the host: which are free, who holds the others.

The reference counts references on its units because a prefix cache shares them
(core/holon/core/memory.py:28-133); without sharing a page has one holder, and giving back a page that the giver
does not hold (freed twice, or never taken) is an error here as there (memory.py:104-123).
"""
from __future__ import annotations


class OutOfPages(RuntimeError):
    """A pool is too small for what is asked of it at start (one request of the longest length must fit)."""


class PageError(RuntimeError):
    """A page was given back by someone who does not hold it."""


class PagePool:
    FREE = -1

    def __init__(self, pages: int) -> None:
        self.pages = pages
        self._free = list(range(pages - 1, -1, -1))          # pop() hands out low numbers first
        self._holder = [self.FREE] * pages

    @property
    def available(self) -> int:
        return len(self._free)

    def take(self, n: int, holder: int) -> list[int] | None:
        """`n` pages for `holder`, or None (and nothing taken) if fewer are free. Freed pages are used again first."""
        if n > len(self._free):
            return None
        out = [self._free.pop() for _ in range(n)]
        for page in out:
            self._holder[page] = holder
        return out

    def give(self, pages, holder: int) -> None:
        for page in pages:
            if not 0 <= page < self.pages or self._holder[page] != holder:
                raise PageError(f"page {page} given back by {holder}, held by "
                                f"{self._holder[page] if 0 <= page < self.pages else 'nobody (no such page)'}")
            self._holder[page] = self.FREE
            self._free.append(page)

    def holder(self, page: int) -> int:
        return self._holder[page]

    def held_by(self, holder: int) -> list[int]:
        return [p for p, h in enumerate(self._holder) if h == holder]
