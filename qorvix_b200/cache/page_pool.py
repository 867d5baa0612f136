"""Free list of fixed-size pages.  The reference's pool is a LIFO stack that hands out low ids
first and refuses a double free (memory/src/kv_cache.cpp:17-47); this one keeps that behaviour
and adds all-or-nothing allocation of several pages.  The list itself lives in C++
(csrc/host_runtime.cpp); this class is its Python face."""
from __future__ import annotations

from typing import List, Optional

from . import native


class PageError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._lib = native.lib()
        self._h = self._lib.qvh_pool_create(self.num_pages)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.qvh_pool_destroy(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return self._lib.qvh_pool_num_free(self._h)

    @property
    def num_held(self) -> int:
        return self.num_pages - self.num_free

    def alloc(self, n: int) -> Optional[List[int]]:
        """n pages, or None (and nothing taken) if fewer are free."""
        if n < 0:
            raise ValueError("cannot allocate a negative number of pages")
        out = (native.c_int * max(n, 1))()
        if not self._lib.qvh_pool_alloc(self._h, n, out):
            return None
        return list(out[:n])

    def free(self, pages) -> None:
        pages = list(pages)
        rc = self._lib.qvh_pool_free(self._h, native.ints(pages) if pages else None, len(pages))
        if rc == -1:
            raise PageError(f"a page of {pages} does not belong to this pool of {self.num_pages}")
        if rc == -2:
            raise PageError(f"a page of {pages} is freed twice")

    def is_held(self, page: int) -> bool:
        return bool(self._lib.qvh_pool_is_held(self._h, page))
