"""Fixed pool of cache pages with a free list."""
from __future__ import annotations

from typing import Iterable, List


class OutOfPages(RuntimeError):
    """The pool cannot supply the pages asked for; nothing was taken."""


class PagePool:
    """``num_pages`` page ids handed out and taken back.  The page freed last is
    handed out first, so a recycled page is reused at once (stale content in a
    recycled page must never matter: readers are bounded by lengths, as the
    reference bounds attention by ``span``, hostfog/hfee internal/llm/forward.go:162)."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"num_pages must be positive, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() gives 0 first
        self._held = [False] * num_pages

    @property
    def free_pages(self) -> int:
        return len(self._free)

    def take(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cannot take a negative number of pages")
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} of {self.num_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def give_back(self, pages: Iterable[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is not of this pool")
            if not self._held[p]:
                raise ValueError(f"page {p} is given back twice")
            self._held[p] = False
            self._free.append(p)

    def is_held(self, page: int) -> bool:
        return self._held[page]
