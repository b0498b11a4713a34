"""Continuous batching above the step function: admits requests, cuts prompts into portions
under a token budget, decodes, and decides what happens when pages run out.

Every step:

1. each running request that is decoding (one token left to run) gets its token, in the
   order of admission; if its next position needs a page and none is free, the request
   admitted last is preempted (its pages and slot are given back, it returns to the front
   of the waiting queue and is recomputed from its tokens so far) until a page is free; a
   request is never preempted in favour of a request admitted after it;
2. running requests still in their prompt get a portion of ``min(rest, budget left)`` tokens;
3. waiting requests are admitted first-come-first-served while a slot is free, the number of
   live requests is below ``max_num_seqs``, token budget is left and pages for the first
   portion are free; the first that does not fit stops admission (as in the reference).

The reference's scheduler (spymaster2h/spyinfer src/engine/scheduler.cpp:17-122) admits by
block count, always runs a prompt whole (no budget, no portions: :59-70), and when a
decoding sequence finds no block it skips it with half-written batch arrays (:77-87); it has
no preemption.  A request that could never finish in the pool even alone is refused at
submission here.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass
from typing import Deque, List

from ..cache import CacheManager
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

    def check_fits(self, seq: Sequence, max_new_tokens: int) -> None:
        """Refuses a request that could never run to its end even alone in the pool."""
        if len(seq) >= self.config.max_model_len:
            raise RequestTooLarge(f"a prompt of {len(seq)} tokens leaves no room to generate within max_model_len {self.config.max_model_len}")
        final = min(len(seq) + max_new_tokens, self.config.max_model_len)
        if self.cache.pages_for(final) > self.cache.num_pages:
            raise RequestTooLarge(f"{final} tokens need {self.cache.pages_for(final)} pages of {self.cache.page_size}; the pool has "
                                  f"{self.cache.num_pages}")

    def add_sequence(self, seq: Sequence) -> None:
        seq.status = SequenceStatus.WAITING
        self.waiting.append(seq)

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running)

    def _preempt(self, seq: Sequence) -> None:
        self.running.remove(seq)
        self.cache.free_request(seq.id)
        seq.num_computed = 0
        seq.status = SequenceStatus.WAITING
        seq.num_preemptions += 1
        self.num_preemptions += 1
        self.waiting.appendleft(seq)

    def finish(self, seq: Sequence, reason: str) -> None:
        """The request is over: it leaves the running list and gives back what it holds."""
        seq.status, seq.finish_reason = SequenceStatus.FINISHED, reason
        if seq in self.running:
            self.running.remove(seq)
        if self.cache.has_request(seq.id):
            self.cache.free_request(seq.id)

    def schedule(self) -> List[ScheduledPortion]:
        """The portions of the next step.  Pages for them are reserved; the caller runs them
        through the step function and reports sampled tokens back."""
        while True:
            out = self._schedule_once()
            if out or not self.running:
                return out
            # live requests, yet none can run (prompts in progress hold every page): the
            # request admitted last gives its pages back and is recomputed later
            self._preempt(self.running[-1])

    def _schedule_once(self) -> List[ScheduledPortion]:
        budget = self.config.max_num_batched_tokens
        cache, ps = self.cache, self.cache.page_size
        out: List[ScheduledPortion] = []
        # 1. decoding requests, oldest first
        for seq in list(self.running):
            if seq not in self.running or seq.remaining != 1 or budget <= 0:
                continue
            while not cache.can_reserve(seq.id, len(seq)) and self.running[-1] is not seq:
                victim = self.running[-1]
                out = [p for p in out if p.seq is not victim]   # a victim that already got its token this step loses it
                self._preempt(victim)
            if not cache.can_reserve(seq.id, len(seq)):
                continue                                        # it is the newest itself: it waits (or is preempted above)
            cache.reserve(seq.id, len(seq))
            out.append(ScheduledPortion(seq, seq.num_computed, 1, True))
            budget -= 1
        # 2. prompts of running requests, in portions
        for seq in self.running:
            if seq.remaining <= 1 or budget <= 0:
                continue
            fit = (cache.pages_for(seq.num_computed) + cache.min_free_pages()) * ps - seq.num_computed
            n = min(seq.remaining, budget, fit)
            if n <= 0:
                continue
            cache.reserve(seq.id, seq.num_computed + n)
            out.append(ScheduledPortion(seq, seq.num_computed, n, seq.num_computed + n == len(seq)))
            budget -= n
        # 3. admission, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.config.max_num_seqs and cache.num_free_slots() > 0:
            seq = self.waiting[0]
            n = min(seq.remaining, budget)
            if cache.pages_for(n) > cache.min_free_pages():
                fit = cache.min_free_pages() * ps
                if self.running or fit <= 0:
                    break                       # wait for running requests to finish and free pages
                n = min(n, fit)                 # nothing else is running: start with what fits
            self.waiting.popleft()
            cache.add_request(seq.id)
            cache.reserve(seq.id, n)
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            out.append(ScheduledPortion(seq, 0, n, n == len(seq)))
            budget -= n
        return out
