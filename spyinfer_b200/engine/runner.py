"""The step function: runs one batch of (request, its next tokens) through the model, from
the cache that earlier steps left, and returns logits at the wanted places.

``ModelRunner.step`` is the one entry that generation, the scheduler and trace replay all
use.  For every entry it reserves pages for the new positions, lays the batch out, runs the
model on exactly the given tokens, and commits the new lengths (which lets windowed groups
give pages back).  Counterpart in the reference: spymaster2h/spyinfer
src/engine/model_runner.cpp:49-157, which also samples and finishes inside; that lives in
the engine above this class here.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache import CacheManager
from ..config.engine_config import EngineConfig
from .batch import BatchStager, StepBatch, StepEntry
from .model import Model


class StepError(RuntimeError):
    pass


class ModelRunner:
    def __init__(self, model: Model, config: EngineConfig, cache: Optional[CacheManager] = None):
        kernels.require_cuda()
        self.model, self.config = model, config
        self.device = model.ctx.device
        needs, cache_of = model.cache_needs()
        if cache is None:
            num_pages = config.num_kvcache_blocks
            if num_pages is None:
                num_pages = self._pages_from_free_memory(needs)
            cache = CacheManager(needs, config.kvcache_block_size, num_pages, config.max_num_seqs, config.max_model_len,
                                 dtype=model.ctx.dtype, device=self.device, cache_of=cache_of)
        self.cache = cache
        self.stager = BatchStager(self.device, config.max_num_batched_tokens, config.max_num_seqs, cache.width, max(1, cache.num_groups()))
        self.vocab_size = model.spec.vocab_size
        self.steps = 0
        self.tokens_run = 0

    def _pages_from_free_memory(self, needs) -> int:
        per_page = CacheManager.bytes_per_page(needs, self.config.kvcache_block_size, self.model.ctx.dtype)
        if per_page == 0:
            return 1
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - int(total * (1.0 - self.config.gpu_memory_utilization)) - (2 << 30)  # room for activations
        pages = budget // per_page
        most = self.config.max_num_seqs * ((self.config.max_model_len + self.config.kvcache_block_size - 1) // self.config.kvcache_block_size)
        if pages <= 0:
            raise StepError("no device memory is left for the cache after the weights; lower gpu_memory_utilization's complement or the model size")
        return int(min(pages, most))

    # ---- the step ----------------------------------------------------------------------------
    def build_batch(self, entries: Sequence[StepEntry], pad_tokens: int = 0, pad_seqs: int = 0) -> StepBatch:
        cache = self.cache
        seen = set()
        token_ids: List[int] = []
        positions: List[int] = []
        seq_of_token: List[int] = []
        logit_rows: List[int] = []
        q_start, ctx_len, slots = [0], [], []
        for s, e in enumerate(entries):
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r} brings no tokens to this step")
            if not cache.has_request(e.request):
                cache.add_request(e.request)
            start = cache.length(e.request)
            cache.reserve(e.request, start + n)
            base = len(token_ids)
            for t in e.tokens:
                if not 0 <= int(t) < self.vocab_size:
                    raise StepError(f"request {e.request!r}: token id {t} is outside the vocabulary of {self.vocab_size}")
            token_ids += [int(t) for t in e.tokens]
            positions += range(start, start + n)
            seq_of_token += [s] * n
            for wpos in e.want:
                if not 0 <= int(wpos) < n:
                    raise StepError(f"request {e.request!r}: wanted place {wpos} is not among its {n} tokens")
                logit_rows.append(base + int(wpos))
            q_start.append(base + n)
            ctx_len.append(start + n)
            slots.append(cache.slot(e.request))
        rids = [e.request for e in entries]
        width = max(1, cache.pages_for(max(ctx_len))) if not pad_seqs else cache.width
        tables = [cache.gather_block_tables(rids, g, width) for g in range(cache.num_groups())]
        i32 = lambda a: np.asarray(a, dtype=np.int32)
        return self.stager.stage(i32(token_ids), i32(positions), i32(seq_of_token), i32(q_start), i32(ctx_len), i32(slots),
                                 i32(logit_rows), tables, pad_tokens, pad_seqs)

    def commit(self, entries: Sequence[StepEntry]) -> None:
        for e in entries:
            self.cache.commit(e.request, self.cache.length(e.request) + len(e.tokens))

    def step(self, entries: Sequence[StepEntry]) -> Optional[torch.Tensor]:
        """Runs the entries as one batch.  Returns float32 logits ``[wanted, vocab]`` on the
        device, rows in the order of the entries and of each entry's ``want``; None when
        nothing is wanted."""
        if not entries:
            return None
        batch = self.build_batch(entries)
        logits = self.model.forward(batch, self.cache)
        self.commit(entries)
        self.steps += 1
        self.tokens_run += batch.num_tokens
        return logits

    def finish(self, request) -> None:
        """The request is over: its pages and its slot are given back."""
        if self.cache.has_request(request):
            self.cache.free_request(request)

    def check_status(self) -> None:
        """Raises if a kernel of an earlier step met an index that would have left its buffers
        (it skipped the access).  Synchronises with the device."""
        code, detail = self.stager.status.tolist()
        if code != 0:
            self.stager.status.zero_()
            raise StepError("a kernel refused " + kernels.STATUS_MESSAGES.get(code, f"status {code}").format(detail=detail))
