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
                                 dtype=model.ctx.dtype, device=self.device, cache_of=cache_of,
                                 max_step_tokens=max(config.max_num_batched_tokens, config.max_num_seqs))
        self.cache = cache
        self.stager = BatchStager(self.device, max(config.max_num_batched_tokens, config.max_num_seqs), config.max_num_seqs, cache.width, max(1, cache.num_groups()))
        self.vocab_size = model.spec.vocab_size
        self.steps = 0
        self.tokens_run = 0
        self.graph_steps = 0
        self._host_tokens = [None, None]
        self._tokens_copied = [torch.cuda.Event(), torch.cuda.Event()]
        self._read_turn = 0
        self._graphs = {}          # decode batch size (padded) -> (graph, logits, kernel launches it holds)
        self._use_graphs = bool(config.use_cuda_graphs) and model.graph_safe()
        #: set to a list to have every step append a pair of CUDA events (timing enabled) recorded
        #: before its first and after its last launch: the sum of the pairs' times against the span
        #: from the first to the last event is the share of the time the device was at work
        self.step_events: Optional[list] = None

    def _pages_from_free_memory(self, needs) -> int:
        """The pool size that the free device memory allows: windowed groups take what their windows
        need (``CacheManager.pages_of_group``), the rest goes to the groups that keep every key."""
        from ..config.spec import PagedCacheNeed
        cfg = self.config
        page, step = cfg.kvcache_block_size, max(cfg.max_num_batched_tokens, cfg.max_num_seqs)
        per_page = CacheManager.bytes_per_page(needs, page, self.model.ctx.dtype)
        if per_page == 0:
            return 1
        paged = [n for n in needs if isinstance(n, PagedCacheNeed)]
        windowed = [n for n in paged if n.window is not None] if any(n.window is None for n in paged) else []
        fixed = sum(CacheManager.pages_of_group(n.window, page, 1 << 30, cfg.max_num_seqs, step) * CacheManager.bytes_per_page([n], page, self.model.ctx.dtype)
                    for n in windowed)
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - int(total * (1.0 - cfg.gpu_memory_utilization)) - (2 << 30) - fixed  # room for activations
        pages = budget // per_page
        most = cfg.max_num_seqs * ((cfg.max_model_len + page - 1) // page)
        if pages <= 0:
            raise StepError("no device memory is left for the cache after the weights; lower gpu_memory_utilization's complement or the model size")
        return int(min(pages, most))

    # ---- the step ----------------------------------------------------------------------------
    def _fill(self, entries: Sequence[StepEntry]):
        """The step's flat arrays (``CacheManager.assemble``, which is the C++ engine core's work)."""
        rids = [e.request for e in entries]
        try:
            return (rids,) + self.cache.assemble(rids, [e.tokens for e in entries], [e.want for e in entries], self.vocab_size)
        except ValueError as e:
            raise StepError(str(e)) from None

    def build_batch(self, entries: Sequence[StepEntry], pad_tokens: int = 0, pad_seqs: int = 0) -> StepBatch:
        cache = self.cache
        rids, token_ids, positions, seq_of_token, q_start, ctx_len, slots, logit_rows, longest = self._fill(entries)
        width = max(1, cache.pages_for(longest)) if not pad_seqs else cache.width
        tables = [cache.gather_block_tables(rids, g, width) for g in range(cache.num_groups())]
        return self.stager.stage(token_ids, positions, seq_of_token, q_start, ctx_len, slots, logit_rows, tables, pad_tokens, pad_seqs)

    def commit(self, entries: Sequence[StepEntry]) -> None:
        self.cache.advance([e.request for e in entries], [len(e.tokens) for e in entries])

    # ---- decoding through a captured graph -----------------------------------------------------
    def _decode_bucket(self, n: int) -> int:
        b = 1
        while b < n:
            b *= 2
        return min(b, self.config.max_num_seqs)

    def _build_decode_batch(self, entries: Sequence[StepEntry], bucket: int) -> StepBatch:
        """A batch of ``bucket`` one-token rows at fixed device offsets: the entries first, then
        padding rows that read and write only the cache's spare page."""
        cache, S = self.cache, len(entries)
        for e in entries:
            if len(e.tokens) != 1:
                raise StepError(f"request {e.request!r}: a decode step brings one token, found {len(e.tokens)}")
        rids, tok, pos, _, _, ctx, slot, _, _ = self._fill(entries)
        token_ids = np.zeros(bucket, np.int32)
        positions = np.zeros(bucket, np.int32)
        ctx_len = np.ones(bucket, np.int32)
        slots = np.zeros(bucket, np.int32)
        token_ids[:S], positions[:S], ctx_len[:S], slots[:S] = tok, pos, ctx, slot
        tables = []
        for g in range(cache.num_groups()):
            t = np.full((bucket, cache.width), -1, np.int32)
            cache.gather_block_tables(rids, g, out=t)
            t[S:, 0] = cache.spare_page(g)
            tables.append(t)
        ar = np.arange(bucket + 1, dtype=np.int32)
        return self.stager.stage(token_ids, positions, ar[:bucket], ar, ctx_len, slots, ar[:bucket], tables, bucket, bucket)

    def _step_graph(self, entries: Sequence[StepEntry], tokens_from: Optional[torch.Tensor] = None) -> torch.Tensor:
        S = len(entries)
        bucket = self._decode_bucket(S)
        batch = self._build_decode_batch(entries, bucket)
        if tokens_from is not None:
            batch.token_ids[:S].copy_(tokens_from[:S])   # behind the staging copy on the stream, ahead of the kernels
        held = self._graphs.get(bucket)
        if held is None:
            # the first step of this size runs eagerly (it also makes every lazy allocation);
            # the graph is captured from the second on
            self._graphs[bucket] = "warm"
            logits = self.model.forward(batch, self.cache)
        elif held == "warm":
            torch.cuda.synchronize()
            before = kernels.launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_logits = self.model.forward(batch, self.cache)
            self._graphs[bucket] = (graph, static_logits, kernels.launch_count() - before)
            kernels.count_launches(-(kernels.launch_count() - before))   # captured, not run
            graph.replay()
            kernels.count_launches(self._graphs[bucket][2])
            logits = static_logits
            self.graph_steps += 1
        else:
            graph, static_logits, launches = held
            graph.replay()
            kernels.count_launches(launches)
            logits = static_logits
            self.graph_steps += 1
        self.commit(entries)
        self.steps += 1
        self.tokens_run += S
        return logits[:S]

    def step(self, entries: Sequence[StepEntry], tokens_from: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the entries as one batch.  Returns float32 logits ``[wanted, vocab]`` on the
        device, rows in the order of the entries and of each entry's ``want``; None when
        nothing is wanted.  A batch in which every request brings one token and wants its
        logits (a decode step) is replayed from a CUDA graph captured for its size; the
        returned tensor is then the graph's own output buffer, valid until the next step.

        ``tokens_from`` (int32 on the device, one per entry; every entry brings one token): the token
        ids are taken from it on the device instead of from the entries, whose tokens only stand in.
        This is how a decode step is launched before the host knows what the last one sampled."""
        if not entries:
            return None
        if self.step_events is None:
            return self._step(entries, tokens_from)
        pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
        pair[0].record()
        logits = self._step(entries, tokens_from)
        pair[1].record()
        self.step_events.append(pair)
        return logits

    def _step(self, entries: Sequence[StepEntry], tokens_from: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        if tokens_from is not None and any(len(e.tokens) != 1 for e in entries):
            raise StepError("tokens_from needs entries of one token each")
        if self._use_graphs and all(len(e.tokens) == 1 and len(e.want) == 1 and int(e.want[0]) == 0 for e in entries):
            if len({e.request for e in entries}) != len(entries):
                raise StepError("a request appears twice in one step")
            return self._step_graph(entries, tokens_from)
        batch = self.build_batch(entries)
        if tokens_from is not None:
            batch.token_ids.copy_(tokens_from[:batch.num_tokens])
        logits = self.model.forward(batch, self.cache)
        self.commit(entries)
        self.steps += 1
        self.tokens_run += batch.num_tokens
        return logits

    def finish(self, request) -> None:
        """The request is over: its pages and its slot are given back."""
        if self.cache.has_request(request):
            self.cache.free_request(request)

    def start_read(self, tokens: torch.Tensor):
        """Queues, behind the kernels launched so far, the copy of a step's sampled tokens and of the
        status word into pinned memory.  Returns what ``finish_read`` needs.  Two steps may be in
        flight at a time (the buffers alternate)."""
        n = tokens.shape[0]
        self._read_turn ^= 1
        host, event = self._host_tokens[self._read_turn], self._tokens_copied[self._read_turn]
        if host is None or host.shape[0] < n + 2:
            host = self._host_tokens[self._read_turn] = torch.empty(max(n + 2, self.config.max_num_seqs + 2), dtype=torch.int32, pin_memory=True)
        host[:n].copy_(tokens, non_blocking=True)
        host[n:n + 2].copy_(self.stager.status, non_blocking=True)
        event.record()
        return host, event, n

    def finish_read(self, pending) -> List[int]:
        """Waits for a copy queued by ``start_read``; raises if a kernel had refused an index."""
        host, event, n = pending
        event.synchronize()
        out = host[:n + 2].tolist()
        if out[n] != 0:
            self._raise_status(out[n], out[n + 1])
        return out[:n]

    def read_tokens(self, tokens: torch.Tensor) -> List[int]:
        """The sampled tokens of a step on the host, and the status word checked, with one wait for the device."""
        return self.finish_read(self.start_read(tokens))

    def check_status(self) -> None:
        """Raises if a kernel of an earlier step met an index that would have left its buffers
        (it skipped the access).  Synchronises with the device."""
        code, detail = self.stager.status.tolist()
        if code != 0:
            self._raise_status(code, detail)

    def _raise_status(self, code: int, detail: int) -> None:
        """The status word was set: it is cleared, and what a kernel that gave up may have left
        behind is put right, before the error is raised; the engine can go on with other steps."""
        self.stager.status.zero_()
        if code == kernels.STATUS_WAIT_TIMEOUT:
            kernels.gemm_tcgen05_reset()
            raise StepError("a kernel gave up: " + kernels.STATUS_MESSAGES[code].format(detail=detail) + "; the results of the step are not valid")
        raise StepError("a kernel refused " + kernels.STATUS_MESSAGES.get(code, f"status {code}").format(detail=detail))
