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
* All bookkeeping is host-side and works without a GPU (``device=None``), which is how the
  CPU tests drive it.

The reference's counterpart is one free list for all layers and a per-sequence vector
(spymaster2h/spyinfer src/engine/block_manager.cpp, src/engine/sequence.hpp:29,
src/engine/scheduler.cpp:24-35, 77-82); it frees only in remove_request
(src/engine/llm_engine.cpp:149-157) and has no groups, windows or state.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..config.spec import PagedCacheNeed, StateCacheNeed
from .pages import OutOfPages, PagePool


class NoFreeSlot(RuntimeError):
    pass


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
    def __init__(self, need: PagedCacheNeed, num_pages: int, max_num_seqs: int, width: int):
        self.need = need
        self.pool = PagePool(num_pages)
        self.entries: List[int] = []
        self.tables = np.full((max_num_seqs, width), -1, dtype=np.int32)  # row = state slot
        self.pages: Optional[torch.Tensor] = None


class _Request:
    def __init__(self, slot: int):
        self.slot = slot
        self.length = 0      # tokens stored (committed)
        self.reserved = 0    # tokens that have pages


class CacheManager:
    def __init__(self, needs: Sequence, page_size: int, num_pages: int, max_num_seqs: int, max_model_len: int,
                 dtype: torch.dtype = torch.bfloat16, device=None, cache_of: Optional[Sequence[Optional[int]]] = None):
        """``needs[i]`` is the cache need of run-order entry ``i`` (None for an entry that keeps
        nothing); ``cache_of[i]`` names the earlier entry whose cache entry ``i`` reads instead
        of owning one.  ``num_pages`` is the size of every group's pool."""
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
                    self.groups.append(_PagedGroup(need, num_pages, max_num_seqs, self.width))
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
        if device is not None:
            for g in self.groups:
                n = g.need
                # one page more than the pool hands out: the spare page (id num_pages) takes the
                # writes of the padding rows of a fixed-size (captured) decode batch
                g.pages = torch.zeros((len(g.entries), num_pages + 1, 2, n.num_kv_heads, page_size, n.head_dim), dtype=dtype, device=device)
        for i, v in enumerate(self._views):
            if v.kind == "paged" and self.groups[v.group].pages is not None:
                v.pages = self.groups[v.group].pages[self._entry_slot_in_group[i]]
            if v.kind == "state" and not v.writes and cache_of[i] is not None:
                v.state = self._views[cache_of[i]].state
        self._free_slots: List[int] = list(range(max_num_seqs - 1, -1, -1))
        self._requests: Dict[Hashable, _Request] = {}

    # ---- sizes -------------------------------------------------------------------------
    @staticmethod
    def bytes_per_page(needs: Sequence, page_size: int, dtype: torch.dtype) -> int:
        """Device bytes that one more page in every group costs."""
        elt = torch.empty((), dtype=dtype).element_size()
        return sum(2 * n.num_kv_heads * page_size * n.head_dim * elt for n in needs if isinstance(n, PagedCacheNeed))

    def pages_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    # ---- requests ----------------------------------------------------------------------
    def has_request(self, rid) -> bool:
        return rid in self._requests

    def live_requests(self) -> List:
        return list(self._requests)

    def num_free_slots(self) -> int:
        return len(self._free_slots)

    def num_free_pages(self, group: int = 0) -> int:
        return self.groups[group].pool.num_free if self.groups else self.num_pages

    def min_free_pages(self) -> int:
        return min((g.pool.num_free for g in self.groups), default=self.num_pages)

    def add_request(self, rid) -> int:
        if rid in self._requests:
            raise ValueError(f"request {rid!r} is already live")
        if not self._free_slots:
            raise NoFreeSlot(f"all {self.max_num_seqs} request slots are taken")
        slot = self._free_slots.pop()
        self._requests[rid] = _Request(slot)
        for t in self.state_tensors:
            if t is not None:
                t[slot].zero_()
        return slot

    def slot(self, rid) -> int:
        return self._requests[rid].slot

    def length(self, rid) -> int:
        return self._requests[rid].length

    def _first_needed_page(self, g: _PagedGroup, length: int) -> int:
        """Lowest logical page that a query at position ``length`` or later can still see."""
        if g.need.window is None:
            return 0
        return max(0, length - g.need.window + 1) // self.page_size

    def pages_needed(self, rid, new_length: int) -> int:
        """Pages (the most over the groups) that ``reserve(rid, new_length)`` would take."""
        r = self._requests[rid]
        have = self.pages_for(r.reserved)
        return max(0, self.pages_for(new_length) - have)

    def can_reserve(self, rid, new_length: int) -> bool:
        need = self.pages_needed(rid, new_length)
        return new_length <= self.max_model_len and all(g.pool.num_free >= need for g in self.groups)

    def reserve(self, rid, new_length: int) -> None:
        """Gives the request the pages its positions ``[reserved, new_length)`` will be stored
        in, in every group.  All or nothing: raises OutOfPages without taking any."""
        r = self._requests[rid]
        if new_length > self.max_model_len:
            raise ValueError(f"request {rid!r}: {new_length} tokens exceed max_model_len {self.max_model_len}")
        if new_length <= r.reserved:
            return
        need = self.pages_needed(rid, new_length)
        for g in self.groups:
            if g.pool.num_free < need:
                raise OutOfPages("Out of memory: No free blocks available.")
        first, last = self.pages_for(r.reserved), self.pages_for(new_length)
        for g in self.groups:
            row = g.tables[r.slot]
            for lp in range(first, last):
                row[lp] = g.pool.allocate()
        r.reserved = new_length

    def commit(self, rid, new_length: int) -> None:
        """The step that stored positions up to ``new_length`` has been issued: the request's
        length advances and windowed groups give back the pages no later query can see."""
        r = self._requests[rid]
        if new_length > r.reserved:
            raise ValueError(f"request {rid!r}: commit of {new_length} tokens, only {r.reserved} have pages")
        if new_length < r.length:
            raise ValueError(f"request {rid!r}: length cannot shrink from {r.length} to {new_length}")
        r.length = new_length
        for g in self.groups:
            if g.need.window is None:
                continue
            row = g.tables[r.slot]
            for lp in range(self._first_needed_page(g, new_length)):
                if row[lp] >= 0:
                    g.pool.free(int(row[lp]))
                    row[lp] = -1

    def free_request(self, rid) -> None:
        """Everything the request holds goes back: pages of every group and the slot."""
        r = self._requests.pop(rid)
        for g in self.groups:
            row = g.tables[r.slot]
            for lp in np.nonzero(row >= 0)[0]:
                g.pool.free(int(row[lp]))
            row[:] = -1
        self._free_slots.append(r.slot)

    @property
    def spare_page(self) -> int:
        """Id of the page that no request ever holds (see the pages tensor's allocation)."""
        return self.num_pages

    def block_table(self, rid, group: int = 0) -> np.ndarray:
        return self.groups[group].tables[self._requests[rid].slot]

    def gather_block_tables(self, rids: Sequence, group: int, width: Optional[int] = None) -> np.ndarray:
        slots = [self._requests[r].slot for r in rids]
        t = self.groups[group].tables[slots]
        return t if width is None else t[:, :width]

    # ---- views for the model --------------------------------------------------------------
    def view(self, entry: int) -> CacheView:
        return self._views[entry]

    def num_groups(self) -> int:
        return len(self.groups)

    # ---- checks ------------------------------------------------------------------------------
    def check_invariants(self) -> None:
        """No page is lost, held twice, or both free and held; slots likewise."""
        for gi, g in enumerate(self.groups):
            held = []
            for rid, r in self._requests.items():
                held += [int(p) for p in g.tables[r.slot] if p >= 0]
            if len(held) != len(set(held)):
                raise AssertionError(f"group {gi}: a page is held twice: {sorted(held)}")
            free = list(g.pool._free)
            if len(free) != len(set(free)):
                raise AssertionError(f"group {gi}: a page is on the free list twice")
            if set(free) & set(held):
                raise AssertionError(f"group {gi}: pages both free and held: {sorted(set(free) & set(held))}")
            if len(free) + len(held) != g.pool.num_pages:
                raise AssertionError(f"group {gi}: {g.pool.num_pages - len(free) - len(held)} pages are lost")
            live_slots = {r.slot for r in self._requests.values()}
            for s in range(self.max_num_seqs):
                if s not in live_slots and (g.tables[s] >= 0).any():
                    raise AssertionError(f"group {gi}: slot {s} has no request but still names pages")
        slots = [r.slot for r in self._requests.values()]
        if len(slots) != len(set(slots)) or set(slots) & set(self._free_slots) or len(slots) + len(self._free_slots) != self.max_num_seqs:
            raise AssertionError("state slots are lost or held twice")
