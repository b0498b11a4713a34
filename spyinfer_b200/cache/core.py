"""ctypes face of the host-side engine core (``csrc/engine_core.cpp``): page pools, the
cache's bookkeeping, batch assembly and the scheduler's decisions, in C++.

The library is built with the host compiler at first use (no GPU and no nvcc needed), so the
CPU tests exercise the same code that serving runs.
"""
from __future__ import annotations

import ctypes
from typing import Optional

from ..csrc import build

c_int_p = ctypes.POINTER(ctypes.c_int)
c_i32_p = ctypes.POINTER(ctypes.c_int32)
c_i64_p = ctypes.POINTER(ctypes.c_int64)

_lib: Optional[ctypes.CDLL] = None


class OutOfPages(RuntimeError):
    """Same condition as the reference's "Out of memory: No free blocks available."
    (spymaster2h/spyinfer src/engine/block_manager.cpp:20-23)."""


class NoFreeSlot(RuntimeError):
    pass


_ERRORS = {1: OutOfPages, 2: ValueError, 3: AssertionError, 4: NoFreeSlot, 5: KeyError}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = build.load("engine_core")
        L.spy_pool_create.restype = ctypes.c_void_p
        L.spy_pool_create.argtypes = [ctypes.c_int]
        L.spy_pool_destroy.argtypes = [ctypes.c_void_p]
        L.spy_pool_destroy.restype = None
        for name in ("spy_pool_num_free",):
            getattr(L, name).argtypes = [ctypes.c_void_p]
        L.spy_pool_is_free.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.spy_pool_allocate.argtypes = [ctypes.c_void_p, c_int_p]
        L.spy_pool_free.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.spy_cache_create.restype = ctypes.c_void_p
        L.spy_cache_create.argtypes = [ctypes.c_int, c_int_p, c_int_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.spy_cache_destroy.argtypes = [ctypes.c_void_p]
        L.spy_cache_destroy.restype = None
        for name in ("spy_cache_width", "spy_cache_min_free_pages", "spy_cache_num_free_slots", "spy_cache_num_live", "spy_cache_check"):
            getattr(L, name).argtypes = [ctypes.c_void_p]
        L.spy_cache_num_free_pages.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.spy_cache_live.argtypes = [ctypes.c_void_p, c_i64_p]
        L.spy_cache_tables.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.spy_cache_tables.restype = c_i32_p
        L.spy_cache_has_request.argtypes = [ctypes.c_void_p, ctypes.c_int64]
        L.spy_cache_add_request.argtypes = [ctypes.c_void_p, ctypes.c_int64, c_int_p]
        L.spy_cache_request.argtypes = [ctypes.c_void_p, ctypes.c_int64, c_int_p, c_int_p, c_int_p]
        L.spy_cache_pages_needed.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, c_int_p]
        L.spy_cache_can_reserve.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, c_int_p]
        L.spy_cache_reserve.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        L.spy_cache_commit.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
        L.spy_cache_free_request.argtypes = [ctypes.c_void_p, ctypes.c_int64]
        L.spy_cache_advance.argtypes = [ctypes.c_void_p, ctypes.c_int, c_i64_p, c_i32_p]
        L.spy_cache_gather.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, c_i64_p, ctypes.c_int, c_i32_p, ctypes.c_int]
        L.spy_cache_fill_batch.argtypes = [ctypes.c_void_p, ctypes.c_int, c_i64_p, c_i32_p, c_i32_p, c_i32_p, c_i32_p, ctypes.c_int] + [c_i32_p] * 7 + [c_int_p] * 3
        L.spy_sched_step.argtypes = ([ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, c_i64_p, c_i32_p, c_i32_p, ctypes.c_int, c_i64_p, c_i32_p]
                                     + [c_i64_p, c_i32_p, c_i32_p, c_i32_p, c_int_p, c_i64_p, c_int_p, c_int_p, c_i64_p])
        _lib = L
    return _lib


def check(code: int) -> None:
    """Raises the Python exception that a non-zero return code of the core stands for."""
    if code != 0:
        raise _ERRORS.get(code, RuntimeError)(build.last_error("engine_core"))


def i32(a):
    return a.ctypes.data_as(c_i32_p)


def i64(a):
    return a.ctypes.data_as(c_i64_p)
