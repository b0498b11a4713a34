"""Continuous batching above the step function: admits requests, cuts prompts into portions
under a token budget, decodes, and decides what happens when pages run out.

Every step:

1. each running request that is decoding (one token left to run) gets its token, in the
   order of admission; if its next position needs a page and none is free, the request
   admitted last is preempted (its pages and slot are given back, it returns to the front
   of the waiting queue and is recomputed from its tokens so far) until a page is free; a
   request is never preempted in favour of a request admitted after it;
2. running requests still in their prompt get a portion of ``min(rest, chunk_size, budget left)``
   tokens (``chunk_size`` is optional: without it the budget alone cuts);
3. waiting requests are admitted first-come-first-served while a slot is free, the number of
   live requests is below ``max_num_seqs``, token budget is left and pages for the first
   portion are free; the first that does not fit stops admission (as in the reference).

The reference's scheduler (spymaster2h/spyinfer src/engine/scheduler.cpp:17-122) admits by
block count, always runs a prompt whole (no budget, no portions: :59-70), and when a
decoding sequence finds no block it skips it with half-written batch arrays (:77-87); it has
no preemption.  A request whose stated length (prompt plus ``max_new_tokens``) could never
be held by the pool even alone is refused at submission here.  A request without
``max_new_tokens`` may grow to ``max_model_len``; when the pool is smaller than that, the
request ends with the reason ``"out_of_pages"`` at the last token the pool can hold
(``Scheduler.most_tokens_alone``), as it would end at ``max_model_len``.  And whatever the
cause, the only running request is never preempted: if it cannot go on, nothing would change
by recomputing it, so it is ended with that reason (``ended_without_token``).
"""
from __future__ import annotations

import ctypes
from collections import deque
from dataclasses import dataclass
from typing import Deque, List

import numpy as np

from ..cache import CacheManager, core
from ..config.engine_config import EngineConfig
from .sequence import Sequence, SequenceStatus


@dataclass
class ScheduledPortion:
    seq: Sequence
    start: int          # position of the first token run
    num_tokens: int
    samples: bool       # the portion reaches the request's last token: its logits are sampled


class RequestTooLarge(ValueError):
    pass


class Scheduler:
    def __init__(self, config: EngineConfig, cache: CacheManager):
        self.config, self.cache = config, cache
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.num_preemptions = 0
        self.ended_without_token: List[Sequence] = []   # requests that schedule() had to end; the caller reports and clears them

    def most_tokens_alone(self) -> int:
        """The most tokens of one request that the pool can hold when the request is alone."""
        return self.cache.most_tokens_alone()

    def check_fits(self, seq: Sequence, max_new_tokens: int) -> None:
        """Refuses a request that could never run to its end even alone in the pool."""
        if len(seq) >= self.config.max_model_len:
            raise RequestTooLarge(f"a prompt of {len(seq)} tokens leaves no room to generate within max_model_len {self.config.max_model_len}")
        final = min(len(seq) + max_new_tokens, self.config.max_model_len)
        if final > self.cache.most_tokens_alone():
            raise RequestTooLarge(f"{final} tokens need {self.cache.pages_for(final)} pages of {self.cache.page_size}; the pool has "
                                  f"{self.cache.most_tokens_alone() // self.cache.page_size}")

    def add_sequence(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def finish(self, seq: Sequence, reason: str) -> None:
        """The request is over: it leaves the running list and gives back what it holds."""
        seq.status, seq.finish_reason = SequenceStatus.FINISHED, reason
        if seq in self.running:
            self.running.remove(seq)
        if self.cache.has_request(seq.id):
            self.cache.free_request(seq.id)

    def schedule(self) -> List[ScheduledPortion]:
        """The portions of the next step.  Pages for them are reserved; the caller runs them
        through the step function and reports sampled tokens back.

        The decision itself (the three rules of the module's header, preemption included) is
        ``spy_sched_step`` of the C++ engine core, which sees the two queues as arrays of
        (request, tokens so far, tokens already run) and works on the cache's bookkeeping
        directly; what it decided is applied to the request records and the queues here."""
        while True:
            portions, stuck = self._decide()
            if stuck is None:
                return portions
            self.ended_without_token.append(stuck)
            self.finish(stuck, "out_of_pages")

    def _decide(self):
        lib, cache = core.lib(), self.cache
        run, wait = list(self.running), list(self.waiting)
        n_run, n_wait = len(run), len(wait)
        run_ids = np.asarray([cache.handle(q.id) for q in run] or [0], dtype=np.int64)
        run_len = np.asarray([len(q) for q in run] or [0], dtype=np.int32)
        run_done = np.asarray([q.num_computed for q in run] or [0], dtype=np.int32)
        wait_ids = np.asarray([cache.handle(q.id) for q in wait] or [0], dtype=np.int64)
        wait_len = np.asarray([len(q) for q in wait] or [0], dtype=np.int32)
        cap = n_run + n_wait + 1
        out_ids, preempted = np.empty(cap, dtype=np.int64), np.empty(cap, dtype=np.int64)
        out_start, out_count, out_samples = (np.empty(cap, dtype=np.int32) for _ in range(3))
        n_out, n_pre, n_adm, stuck = ctypes.c_int(), ctypes.c_int(), ctypes.c_int(), ctypes.c_int64(-1)
        core.check(lib.spy_sched_step(cache._h, int(self.config.max_num_batched_tokens), int(self.config.chunk_size or 0), int(self.config.max_num_seqs), n_run, core.i64(run_ids),
                                      core.i32(run_len), core.i32(run_done), n_wait, core.i64(wait_ids), core.i32(wait_len), core.i64(out_ids),
                                      core.i32(out_start), core.i32(out_count), core.i32(out_samples), ctypes.byref(n_out), core.i64(preempted),
                                      ctypes.byref(n_pre), ctypes.byref(n_adm), ctypes.byref(stuck)))
        by_handle = {cache.handle(q.id): q for q in run + wait}
        for h in preempted[:n_pre.value]:          # in the order of preemption, each to the very front of the queue
            seq = by_handle[int(h)]
            self.running.remove(seq)
            seq.num_computed = 0
            seq.status = SequenceStatus.WAITING
            seq.num_preemptions += 1
            self.num_preemptions += 1
            self.waiting.appendleft(seq)
        for _ in range(n_adm.value):               # the first of the queue as it now stands
            seq = self.waiting.popleft()
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            cache.zero_state(cache.slot(seq.id))
        portions = [ScheduledPortion(by_handle[int(out_ids[i])], int(out_start[i]), int(out_count[i]), bool(out_samples[i])) for i in range(n_out.value)]
        return portions, (by_handle[stuck.value] if stuck.value >= 0 else None)
