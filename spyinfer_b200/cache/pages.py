"""A pool of page ids with a last-in-first-out free list.

Same behaviour as the reference's BlockManager (spymaster2h/spyinfer
src/engine/block_manager.cpp:5-42: ids ``0..N-1``, ``allocate`` pops one, ``free`` pushes
back), which makes a page that was just given back the next one handed out.  Double frees
and foreign ids are errors here instead of silent corruption.  The pool itself lives in the
C++ engine core; this class is its handle.
"""
from __future__ import annotations

import ctypes

from . import core
from .core import OutOfPages

__all__ = ["OutOfPages", "PagePool"]


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, found {num_pages}")
        self.num_pages = num_pages
        self._lib = core.lib()
        self._h = self._lib.spy_pool_create(num_pages)

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.spy_pool_destroy(self._h)
            self._h = None

    @property
    def num_free(self) -> int:
        return self._lib.spy_pool_num_free(self._h)

    def allocate(self) -> int:
        page = ctypes.c_int()
        core.check(self._lib.spy_pool_allocate(self._h, ctypes.byref(page)))
        return page.value

    def free(self, page: int) -> None:
        core.check(self._lib.spy_pool_free(self._h, int(page)))

    def is_free(self, page: int) -> bool:
        return bool(self._lib.spy_pool_is_free(self._h, int(page)))
