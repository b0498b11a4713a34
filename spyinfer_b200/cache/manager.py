"""The cache manager: pages of keys and values with a block table per request, grouped by
what the layers need, and slots for per-request state of fixed size.

* Every entry of the model's run order that owns a cache declares its need.  Entries with
  equal paged needs (same heads, head size and window) form a *group*: one pool of page
  ids, one block table per request, one device tensor
  ``[entries, pages, 2 (K, V), kv_heads, page_size, head_dim]``.  A page id addresses the
  same token range in every entry of its group.
* A request holds, per group, the pages of the positions it has stored.  In a windowed group
  the pages that lie wholly behind the window of every future query are given back when a
  step is committed; their block-table entries become -1.
* A request also holds one *state slot* (an index below ``max_num_seqs``) from admission to
  its end.  Entries with a ``StateCacheNeed`` keep ``[entries, slots, *shape]`` tensors that
  are indexed by it; a slot's state is zeroed when the slot is handed out.  An architecture
  without such layers (Qwen3) still gets the slot: the batch carries it.
* All bookkeeping is host-side, in the C++ engine core (``csrc/engine_core.cpp``), and works
  without a GPU (``device=None``), which is how the CPU tests drive it; this class owns the
  device tensors and the views.

The reference's counterpart is one free list for all layers and a per-sequence vector
(spymaster2h/spyinfer src/engine/block_manager.cpp, src/engine/sequence.hpp:29,
src/engine/scheduler.cpp:24-35, 77-82); it frees only in remove_request
(src/engine/llm_engine.cpp:149-157) and has no groups, windows or state.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..config.spec import PagedCacheNeed, StateCacheNeed
from . import core
from .core import NoFreeSlot, OutOfPages

__all__ = ["CacheManager", "CacheView", "NoFreeSlot", "OutOfPages"]


@dataclass
class CacheView:
    """What one run-order entry's mixer sees of the cache during a step."""

    kind: str                      # "paged", "state" or "none"
    group: int = -1
    pages: Optional[torch.Tensor] = None        # [pages, 2, kv_heads, page_size, head_dim] of this entry
    block_table: Optional[torch.Tensor] = None  # [S, width] int32 on the device, set for each step
    page_size: int = 0
    window: Optional[int] = None
    writes: bool = True            # False: the entry reads another entry's cache
    state: Optional[torch.Tensor] = None        # [slots, *shape] of this entry


class _PagedGroup:
    """A group's need, the run-order entries it serves, its device tensor and a view of its block
    tables (``[max_num_seqs, width]``, row = state slot), which live in the engine core."""

    def __init__(self, need: PagedCacheNeed):
        self.need = need
        self.entries: List[int] = []
        self.tables: Optional[np.ndarray] = None
        self.pages: Optional[torch.Tensor] = None


class CacheManager:
    def __init__(self, needs: Sequence, page_size: int, num_pages: int, max_num_seqs: int, max_model_len: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, cache_of: Optional[Sequence[Optional[int]]] = None,
                 max_step_tokens: Optional[int] = None):
        """``needs[i]`` is the cache need of run-order entry ``i`` (None for an entry that keeps
        nothing); ``cache_of[i]`` names the earlier entry whose cache entry ``i`` reads instead
        of owning one.  ``num_pages`` is the size of the pool of a group that keeps every key.
        With ``max_step_tokens`` (the most tokens one step brings) a windowed group gets only the
        pages its requests can hold at once: each at most its window, the tokens of one step
        (their pages are taken before the step and the ones behind the window given back after
        it) and two pages of rounding; without it, ``num_pages`` as well."""
        if page_size <= 0 or max_num_seqs <= 0 or max_model_len <= 0:
            raise ValueError("page_size, max_num_seqs and max_model_len must be positive")
        self.page_size, self.num_pages, self.max_num_seqs, self.max_model_len = page_size, num_pages, max_num_seqs, max_model_len
        self.width = (max_model_len + page_size - 1) // page_size
        self.dtype, self.device = dtype, device
        self.groups: List[_PagedGroup] = []
        self.state_tensors: List[Optional[torch.Tensor]] = []
        self._views: List[CacheView] = []
        cache_of = list(cache_of) if cache_of is not None else [None] * len(needs)
        by_key: Dict[Hashable, int] = {}
        self._entry_slot_in_group: List[int] = []
        for i, need in enumerate(needs):
            if cache_of[i] is not None:
                src = self._views[cache_of[i]]
                self._views.append(CacheView(kind=src.kind, group=src.group, page_size=src.page_size, window=src.window, writes=False))
                self._entry_slot_in_group.append(self._entry_slot_in_group[cache_of[i]])
                self.state_tensors.append(None)
                continue
            if need is None:
                self._views.append(CacheView(kind="none"))
                self._entry_slot_in_group.append(-1)
                self.state_tensors.append(None)
            elif isinstance(need, PagedCacheNeed):
                key = need.group_key()
                if key not in by_key:
                    by_key[key] = len(self.groups)
                    self.groups.append(_PagedGroup(need))
                g = by_key[key]
                self._entry_slot_in_group.append(len(self.groups[g].entries))
                self.groups[g].entries.append(i)
                self._views.append(CacheView(kind="paged", group=g, page_size=page_size, window=need.window))
                self.state_tensors.append(None)
            elif isinstance(need, StateCacheNeed):
                t = None
                if device is not None:
                    t = torch.zeros((max_num_seqs,) + tuple(need.shape), dtype=getattr(torch, need.dtype), device=device)
                self._views.append(CacheView(kind="state", state=t))
                self._entry_slot_in_group.append(-1)
                self.state_tensors.append(t)
            else:
                raise TypeError(f"run-order entry {i}: unknown cache need {need!r}")
        # the bookkeeping (pools, block tables, slots, requests) lives in the C++ engine core
        self._lib = core.lib()
        windows = (ctypes.c_int * max(1, len(self.groups)))(*[(-1 if g.need.window is None else int(g.need.window)) for g in self.groups])
        self.group_pages = [self.pages_of_group(g.need.window, page_size, num_pages, max_num_seqs, max_step_tokens) for g in self.groups]
        sizes = (ctypes.c_int * max(1, len(self.groups)))(*self.group_pages)
        self._h = self._lib.spy_cache_create(len(self.groups), windows, sizes, page_size, num_pages, max_num_seqs, max_model_len)
        if not self._h:
            raise ValueError(core.build.last_error("engine_core"))
        for gi, g in enumerate(self.groups):
            g.tables = np.ctypeslib.as_array(self._lib.spy_cache_tables(self._h, gi), shape=(max_num_seqs, self.width))
        if device is not None:
            for g, pool_pages in zip(self.groups, self.group_pages):
                n = g.need
                # one page more than the pool hands out: the spare page (the id after the pool's last) takes
                # the writes of the padding rows of a fixed-size (captured) decode batch
                g.pages = torch.zeros((len(g.entries), pool_pages + 1, 2, n.num_kv_heads, page_size, n.head_dim), dtype=dtype, device=device)
        for i, v in enumerate(self._views):
            if v.kind == "paged" and self.groups[v.group].pages is not None:
                v.pages = self.groups[v.group].pages[self._entry_slot_in_group[i]]
            if v.kind == "state" and not v.writes and cache_of[i] is not None:
                v.state = self._views[cache_of[i]].state
        self._handles: Dict[Hashable, int] = {}    # request ids that are no small integers -> handles of the core
        self._names: Dict[int, Hashable] = {}

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.spy_cache_destroy(self._h)
            self._h = None

    # ---- request ids ------------------------------------------------------------------------
    def handle(self, rid) -> int:
        """The 64-bit handle the core knows a request by: the id itself when it is an integer
        below 2^62, else a number above that, given out at first use."""
        if isinstance(rid, int) and not isinstance(rid, bool) and 0 <= rid < (1 << 62):
            return rid
        h = self._handles.get(rid)
        if h is None:
            h = (1 << 62) + len(self._handles)
            self._handles[rid] = h
            self._names[h] = rid
        return h

    def _record(self, rid):
        slot, length, reserved = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        rc = self._lib.spy_cache_request(self._h, self.handle(rid), ctypes.byref(slot), ctypes.byref(length), ctypes.byref(reserved))
        if rc != 0:
            raise KeyError(rid)
        return slot.value, length.value, reserved.value

    # ---- sizes -------------------------------------------------------------------------
    @staticmethod
    def pages_of_group(window: Optional[int], page_size: int, num_pages: int, max_num_seqs: int, max_step_tokens: Optional[int]) -> int:
        """The pool size of a group with this window (None: every key is kept)."""
        if window is None or max_step_tokens is None:
            return num_pages
        per_request = (int(window) + int(max_step_tokens) + page_size - 1) // page_size + 2
        return max(1, min(num_pages, max_num_seqs * per_request))

    @staticmethod
    def bytes_per_page(needs: Sequence, page_size: int, dtype: torch.dtype) -> int:
        """Device bytes that one more page costs in every group that keeps every key (windowed
        groups are bounded by their window, see ``pages_of_group``; with only such groups, in every group)."""
        elt = torch.empty((), dtype=dtype).element_size()
        paged = [n for n in needs if isinstance(n, PagedCacheNeed)]
        full = [n for n in paged if n.window is None] or paged
        return sum(2 * n.num_kv_heads * page_size * n.head_dim * elt for n in full)

    def most_tokens_alone(self) -> int:
        """The most tokens of ONE request that the pools can hold (beyond ``max_model_len`` if only
        windowed groups exist: their pages come back as the window passes)."""
        full = [p for g, p in zip(self.groups, self.group_pages) if g.need.window is None]
        return min(full) * self.page_size if full else max(self.max_model_len, self.num_pages * self.page_size)

    def pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    # ---- requests ----------------------------------------------------------------------
    def has_request(self, rid) -> bool:
        return bool(self._lib.spy_cache_has_request(self._h, self.handle(rid)))

    def live_requests(self) -> List:
        n = self._lib.spy_cache_num_live(self._h)
        out = np.empty(max(1, n), dtype=np.int64)
        n = self._lib.spy_cache_live(self._h, core.i64(out))
        return [self._names.get(int(h), int(h)) for h in out[:n]]

    def num_free_slots(self) -> int:
        return self._lib.spy_cache_num_free_slots(self._h)

    def num_free_pages(self, group: int = 0) -> int:
        return self._lib.spy_cache_num_free_pages(self._h, group)

    def min_free_pages(self) -> int:
        return self._lib.spy_cache_min_free_pages(self._h)

    def add_request(self, rid) -> int:
        slot = ctypes.c_int()
        rc = self._lib.spy_cache_add_request(self._h, self.handle(rid), ctypes.byref(slot))
        if rc == 2:
            raise ValueError(f"request {rid!r} is already live")
        core.check(rc)
        self.zero_state(slot.value)
        return slot.value

    def zero_state(self, slot: int) -> None:
        """A slot that has just been handed out starts from zero state."""
        for t in self.state_tensors:
            if t is not None:
                t[slot].zero_()

    def slot(self, rid) -> int:
        return self._record(rid)[0]

    def length(self, rid) -> int:
        return self._record(rid)[1]

    def pages_needed(self, rid, new_length: int) -> int:
        """Pages (the most over the groups) that ``reserve(rid, new_length)`` would take."""
        pages = ctypes.c_int()
        if self._lib.spy_cache_pages_needed(self._h, self.handle(rid), int(new_length), ctypes.byref(pages)) != 0:
            raise KeyError(rid)
        return pages.value

    def can_reserve(self, rid, new_length: int) -> bool:
        yes = ctypes.c_int()
        if self._lib.spy_cache_can_reserve(self._h, self.handle(rid), int(new_length), ctypes.byref(yes)) != 0:
            raise KeyError(rid)
        return bool(yes.value)

    def reserve(self, rid, new_length: int) -> None:
        """Gives the request the pages its positions ``[reserved, new_length)`` will be stored
        in, in every group.  All or nothing: raises OutOfPages without taking any."""
        rc = self._lib.spy_cache_reserve(self._h, self.handle(rid), int(new_length))
        if rc == 5:
            raise KeyError(rid)
        if rc == 2:
            raise ValueError(f"request {rid!r}: {new_length} tokens exceed max_model_len {self.max_model_len}")
        core.check(rc)

    def commit(self, rid, new_length: int) -> None:
        """The step that stored positions up to ``new_length`` has been issued: the request's
        length advances and windowed groups give back the pages no later query can see."""
        rc = self._lib.spy_cache_commit(self._h, self.handle(rid), int(new_length))
        if rc == 5:
            raise KeyError(rid)
        core.check(rc)

    def advance(self, rids: Sequence, counts: Sequence[int]) -> None:
        """A step has been issued: every request of it is committed at its length plus the tokens it brought."""
        handles = np.asarray([self.handle(r) for r in rids] or [0], dtype=np.int64)
        counts = np.asarray(list(counts) or [0], dtype=np.int32)
        rc = self._lib.spy_cache_advance(self._h, len(rids), core.i64(handles), core.i32(counts))
        if rc == 5:
            raise KeyError(core.build.last_error("engine_core"))
        core.check(rc)

    def free_request(self, rid) -> None:
        """Everything the request holds goes back: pages of every group and the slot."""
        rc = self._lib.spy_cache_free_request(self._h, self.handle(rid))
        if rc == 5:
            raise KeyError(rid)
        core.check(rc)

    def spare_page(self, group: int = 0) -> int:
        """Id of the page of ``group`` that no request ever holds (see the pages tensor's allocation)."""
        return self.group_pages[group]

    def block_table(self, rid, group: int = 0) -> np.ndarray:
        return self.groups[group].tables[self.slot(rid)]

    def gather_block_tables(self, rids: Sequence, group: int, width: Optional[int] = None, out: Optional[np.ndarray] = None) -> np.ndarray:
        """The block-table rows of ``rids`` in group ``group``, ``width`` entries each (default: all),
        into ``out[:len(rids), :width]`` when it is given."""
        width = self.width if width is None else width
        handles = np.asarray([self.handle(r) for r in rids], dtype=np.int64)
        if out is None:
            out = np.empty((len(rids), width), dtype=np.int32)
        rc = self._lib.spy_cache_gather(self._h, group, len(rids), core.i64(handles), width, core.i32(out), out.strides[0] // 4)
        if rc == 5:
            raise KeyError(core.build.last_error("engine_core"))
        core.check(rc)
        return out[:len(rids), :width]

    # ---- the batch arrays of a step -----------------------------------------------------------
    def assemble(self, rids: Sequence, token_lists: Sequence[Sequence[int]], want_lists: Sequence[Sequence[int]], vocab_size: int):
        """The flat arrays of one step, made by the engine core (``spy_cache_fill_batch``): request
        ``rids[i]`` brings ``token_lists[i]`` and wants logits at the places ``want_lists[i]`` among
        them.  Requests that are new get a slot (zero state), pages for the new tokens are reserved,
        token ids and wanted places are checked (ValueError names the request).  Returns
        ``token_ids[T], positions[T], seq_of_token[T], q_start[S + 1], ctx_len[S], state_slot[S],
        logit_rows[R]`` (numpy int32) and the longest context."""
        n = len(rids)
        fresh = [r for r in rids if not self.has_request(r)]
        counts = np.asarray([len(t) for t in token_lists] or [0], dtype=np.int32)
        T = int(counts[:n].sum())
        try:
            tokens = np.fromiter((int(t) for ts in token_lists for t in ts), dtype=np.int32, count=T) if T else np.zeros(1, np.int32)
        except OverflowError:
            raise ValueError(f"a token id of this step is outside the vocabulary of {vocab_size}") from None
        want_start = np.zeros(n + 1, dtype=np.int32)
        np.cumsum([len(w) for w in want_lists], out=want_start[1:])
        R = int(want_start[n])
        want = np.fromiter((int(w) for ws in want_lists for w in ws), dtype=np.int32, count=R) if R else np.zeros(1, np.int32)
        handles = np.asarray([self.handle(r) for r in rids] or [0], dtype=np.int64)
        token_ids, positions, seq_of_token = (np.empty(max(1, T), dtype=np.int32) for _ in range(3))
        q_start, ctx_len, slots, logit_rows = np.empty(n + 1, np.int32), np.empty(max(1, n), np.int32), np.empty(max(1, n), np.int32), np.empty(max(1, R), np.int32)
        t_out, r_out, longest = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        rc = self._lib.spy_cache_fill_batch(self._h, n, core.i64(handles), core.i32(counts), core.i32(tokens), core.i32(want_start), core.i32(want),
                                            int(vocab_size), core.i32(token_ids), core.i32(positions), core.i32(seq_of_token), core.i32(q_start),
                                            core.i32(ctx_len), core.i32(slots), core.i32(logit_rows), ctypes.byref(t_out), ctypes.byref(r_out),
                                            ctypes.byref(longest))
        for r in fresh:                       # slots handed out by this call start from zero state
            if self.has_request(r):
                self.zero_state(self.slot(r))
        if rc == 2:
            message = core.build.last_error("engine_core")
            k = int(message.split()[1].rstrip(":")) if message.startswith("entry ") else -1
            raise ValueError((f"request {rids[k]!r}: " if 0 <= k < n else "") + message)
        core.check(rc)
        return token_ids[:T], positions[:T], seq_of_token[:T], q_start, ctx_len[:n], slots[:n], logit_rows[:R], longest.value

    # ---- views for the model --------------------------------------------------------------
    def view(self, entry: int) -> CacheView:
        return self._views[entry]

    def num_groups(self) -> int:
        return len(self.groups)

    # ---- checks ------------------------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page is lost, held twice, or both free and held; slots likewise."""
        core.check(self._lib.spy_cache_check(self._h))
