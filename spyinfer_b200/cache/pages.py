"""A pool of page ids with a last-in-first-out free list.

Same behaviour as the reference's BlockManager (spymaster2h/spyinfer
src/engine/block_manager.cpp:5-42: ids ``0..N-1``, ``allocate`` pops one, ``free`` pushes
back), which makes a page that was just given back the next one handed out.  Double frees
and foreign ids are errors here instead of silent corruption.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """Same condition as the reference's "Out of memory: No free blocks available."
    (src/engine/block_manager.cpp:20-23)."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, found {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))  # page 0 is handed out first
        self._is_free = [True] * num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("Out of memory: No free blocks available.")
        page = self._free.pop()
        self._is_free[page] = False
        return page

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page {page} is not of this pool (0..{self.num_pages - 1})")
        if self._is_free[page]:
            raise ValueError(f"page {page} is freed twice")
        self._is_free[page] = True
        self._free.append(page)

    def is_free(self, page: int) -> bool:
        return self._is_free[page]
