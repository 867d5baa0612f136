"""Free list of fixed-size pages (host side).  The reference's pool is a LIFO stack that
hands out low ids first and refuses a double free (memory/src/kv_cache.cpp:17-47); this one
keeps the same behaviour and adds all-or-nothing allocation of several pages."""
from __future__ import annotations

from typing import List, Optional


class PageError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))   # pop() yields 0, 1, 2, ...
        self._held = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self, n: int) -> Optional[List[int]]:
        """n pages, or None (and nothing taken) if fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if n > len(self._free):
            return None
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            self._held[p] = True
        return pages

    def free(self, pages) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise PageError(f"page {p} does not belong to this pool of {self.num_pages}")
            if not self._held[p]:
                raise PageError(f"page {p} is freed twice")
            self._held[p] = False
            self._free.append(p)

    def is_held(self, page: int) -> bool:
        return self._held[page]
