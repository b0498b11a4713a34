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


def padded_step_sizes(tokens: int, requests: int, wanted: int, max_requests: int, max_tokens: int, limit: int, head: int = 0):
    """The sizes (tokens, requests, wanted rows, one-token requests at the head) that a step is padded to before it is
    replayed from a CUDA graph: tokens to a multiple of 32 (up to 128) or 64, requests to a power of two with room for the
    request that holds the padding tokens, wanted rows to a power of two that is at least the requests'; ``head`` (the
    requests at the head of the batch that bring one token and go through the decode kernel; 0: none do) to a power of two,
    the padding being one-token requests of their own.  None: the step is not padded (more than ``limit`` tokens, nothing
    wanted, or no room left for the padding), it runs on launches one by one."""
    if wanted <= 0 or tokens <= 0 or tokens > limit:
        return None
    Hb = 0
    if head > 0:
        Hb = 1
        while Hb < head:
            Hb *= 2
    tokens, requests = tokens + (Hb - head), requests + (Hb - head)
    Tb = (tokens + 31) // 32 * 32 if tokens <= 128 else (tokens + 63) // 64 * 64
    need = requests + (1 if Tb > tokens else 0)           # the padding tokens are a request of their own
    Sb = 1
    while Sb < need:
        Sb *= 2
    Sb = min(Sb, max_requests)
    Rb = 1
    while Rb < wanted:
        Rb *= 2
    Rb = max(min(Rb, Tb), min(Sb, Tb))                    # at least a row a request: fewer distinct sizes, and the extra rows cost next to nothing
    if Sb < need or Rb < wanted or Tb > max_tokens:
        return None
    return Tb, Sb, Rb, Hb


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
        self._graphs = {}          # padded sizes of a step -> (graph, logits, kernel launches it holds); decode steps: the batch size
        self._use_graphs = bool(config.use_cuda_graphs) and model.graph_safe()
        self._graph_pool = None
        self._capture_stream = None
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

    #: From this many one-token requests beside prompt portions on, their attention runs through the decode kernel (the
    #: batch says so in ``one_token_head``), which reads a cache two to three times faster for one token than a 256-row
    #: block of the kernel for portions does ...
    ONE_TOKEN_HEAD_MIN = 4
    #: ... or from this many keys of the longest of them on: such a block walks a long cache alone, tile after tile (77 us for
    #: 8,192 keys where the decode kernel, which shares a pair's tiles out over all blocks, needs 14)
    ONE_TOKEN_HEAD_KEYS = 1024

    def _lay_out(self, entries: Sequence[StepEntry]):
        """The arrays of a step that is no decode step, with the requests that bring one token laid out first.  Returns
        ``(filled, head)``: ``filled`` as ``_fill`` gives it, the wanted rows in the order of ``entries`` as given; ``head``,
        how many requests at the head bring one token each and should go through the decode kernel (0: none, or not worth a
        launch of its own)."""
        n = len(entries)
        ones = sum(1 for e in entries if len(e.tokens) == 1)
        if ones == 0 or ones == n:
            return self._fill(entries), 0
        order = sorted(range(n), key=lambda i: len(entries[i].tokens) != 1)       # stable: one-token requests first
        laid_out = [entries[i] for i in order]
        rids, token_ids, positions, seq_of_token, q_start, ctx_len, slots, logit_rows, longest = self._fill(laid_out)
        if len(logit_rows):                                                       # the wanted rows, entry by entry in the caller's order
            ends = np.cumsum([len(e.want) for e in laid_out])
            rows_of = {i: logit_rows[end - len(entries[i].want):end] for i, end in zip(order, ends)}
            logit_rows = np.concatenate([rows_of[i] for i in range(n)]).astype(np.int32)
        head = ones if ones >= self.ONE_TOKEN_HEAD_MIN or int(ctx_len[:ones].max()) >= self.ONE_TOKEN_HEAD_KEYS else 0
        return (rids, token_ids, positions, seq_of_token, q_start, ctx_len, slots, logit_rows, longest), head

    def _batch_as_laid_out(self, filled, head: int) -> StepBatch:
        cache = self.cache
        rids, token_ids, positions, seq_of_token, q_start, ctx_len, slots, logit_rows, longest = filled
        width = max(1, cache.pages_for(longest))
        tables = [cache.gather_block_tables(rids, g, width) for g in range(cache.num_groups())]
        batch = self.stager.stage(token_ids, positions, seq_of_token, q_start, ctx_len, slots, logit_rows, tables)
        batch.one_token_head = head
        return batch

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

    # A step of other shapes (prompt portions, mixes) of up to ``EngineConfig.graph_step_tokens`` tokens is padded to one of a
    # few sizes and replayed from a graph as well: below that size the host takes longer to launch the step's kernels one by
    # one than the device takes to run them (the default, 384, is where the two meet at the 8B shape).
    #: graphs of padded steps kept at a time (the least recently used one goes first)
    GRAPH_STEP_LIMIT = 24
    #: a padded step's graph is made for a padded number of one-token requests at its head; with more of them than this
    #: the step is launched one by one instead
    GRAPH_STEP_ONE_TOKEN_REQUESTS = 16

    def _step_graph(self, entries: Sequence[StepEntry], tokens_from: Optional[torch.Tensor] = None) -> torch.Tensor:
        S = len(entries)
        bucket = self._decode_bucket(S)
        batch = self._build_decode_batch(entries, bucket)
        if tokens_from is not None:
            batch.token_ids[:S].copy_(tokens_from[:S])   # behind the staging copy on the stream, ahead of the kernels
        logits = self._run_through_graph(bucket, batch)
        self.commit(entries)
        self.steps += 1
        self.tokens_run += S
        return logits[:S]

    def _run_through_graph(self, key, batch: StepBatch) -> torch.Tensor:
        """The forward pass of a batch whose arrays lie at the fixed offsets of its padded sizes ``key``: eagerly the
        first time (which also makes every lazy allocation), captured the second, replayed from then on."""
        held = self._graphs.get(key)
        if held is None:
            self._graphs[key] = "warm"
            return self.model.forward(batch, self.cache)
        if held == "warm":
            before = kernels.launch_count()
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
                self._capture_stream = torch.cuda.Stream(device=self.device)
            # One memory pool for all step graphs: they never run at the same time, none reads what another wrote, and the
            # logits each returns stay allocated while the graph is held, so their activations may share the same memory.
            # Captured on a stream of its own between two joins with the current one.  (torch.cuda.graph() would also
            # collect garbage and hand all cached device memory back first, after which the next large step allocates anew:
            # with a large model in memory that cost most of a second at every new size.)
            current = torch.cuda.current_stream(self.device)
            self._capture_stream.wait_stream(current)
            with torch.cuda.stream(self._capture_stream):
                graph.capture_begin(pool=self._graph_pool)
                try:
                    static_logits = self.model.forward(batch, self.cache)
                finally:
                    graph.capture_end()
            current.wait_stream(self._capture_stream)
            launches = kernels.launch_count() - before
            self._graphs[key] = (graph, static_logits, launches)
            kernels.count_launches(-launches)   # captured, not run
        else:
            self._graphs[key] = self._graphs.pop(key)   # most recently used last
        graph, static_logits, launches = self._graphs[key]
        graph.replay()
        kernels.count_launches(launches)
        self.graph_steps += 1
        return static_logits

    def _padded_batch(self, filled, head: int, Tb: int, Sb: int, Rb: int, Hb: int) -> StepBatch:
        """The batch laid out for ``Tb`` tokens, ``Sb`` requests, ``Rb`` wanted rows and ``Hb`` one-token requests at the head:
        the ``head`` real one-token requests, one-token requests of padding up to ``Hb``, the other requests, then one
        request that holds the padding tokens; further requests are empty.  All padding sits at position 0 and reads and
        writes only the cache's spare page; the padding rows of the logits repeat the first wanted row."""
        cache = self.cache
        rids, tok, pos, seq_of, q_start, ctx, slot, rows, _ = filled
        T, S, R, extra = len(tok), len(ctx), len(rows), Hb - head
        token_ids, positions = np.zeros(Tb, np.int32), np.zeros(Tb, np.int32)
        seq_of_token = np.full(Tb, S + extra, np.int32)                          # what is left over belongs to the request of padding tokens
        token_ids[:head], positions[:head], seq_of_token[:head] = tok[:head], pos[:head], seq_of[:head]
        seq_of_token[head:Hb] = np.arange(head, Hb, dtype=np.int32)
        token_ids[Hb:T + extra], positions[Hb:T + extra], seq_of_token[Hb:T + extra] = tok[head:], pos[head:], seq_of[head:] + extra
        starts = np.full(Sb + 1, Tb, np.int32)
        starts[:Hb + 1] = np.arange(Hb + 1, dtype=np.int32)
        starts[Hb:S + extra + 1] = q_start[head:] + extra
        ctx_len, slots = np.ones(Sb, np.int32), np.zeros(Sb, np.int32)
        ctx_len[:head], slots[:head] = ctx[:head], slot[:head]
        ctx_len[Hb:S + extra], slots[Hb:S + extra] = ctx[head:], slot[head:]
        logit_rows = np.full(Rb, 0, np.int32)
        logit_rows[:R] = np.where(rows >= head, rows + extra, rows)
        logit_rows[R:] = logit_rows[0]
        tables = []
        for g in range(cache.num_groups()):
            t = np.full((Sb, cache.width), -1, np.int32)
            real = cache.gather_block_tables(rids, g, cache.width)
            t[:head], t[Hb:S + extra] = real[:head], real[head:]
            t[head:Hb, 0] = cache.spare_page(g)
            t[S + extra:, 0] = cache.spare_page(g)
            tables.append(t)
        batch = self.stager.stage(token_ids, positions, seq_of_token, starts, ctx_len, slots, logit_rows, tables, Tb, Sb)
        batch.one_token_head = Hb
        return batch

    def step(self, entries: Sequence[StepEntry], tokens_from: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """Runs the entries as one batch.  Returns float32 logits ``[wanted, vocab]`` on the
        device, rows in the order of the entries and of each entry's ``want``; None when
        nothing is wanted.  A batch in which every request brings one token and wants its
        logits (a decode step) is replayed from a CUDA graph captured for its size, and so is any
        other batch of up to ``EngineConfig.graph_step_tokens`` tokens, padded to one of a few sizes; the
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
        if tokens_from is not None:
            batch = self.build_batch(entries)
            batch.token_ids.copy_(tokens_from[:batch.num_tokens])
            logits = self.model.forward(batch, self.cache)
        else:
            if len({e.request for e in entries}) != len(entries):
                raise StepError("a request appears twice in one step")
            filled, head = self._lay_out(entries)
            wanted = len(filled[7])
            sizes = None
            if self._use_graphs and head <= self.GRAPH_STEP_ONE_TOKEN_REQUESTS:
                sizes = padded_step_sizes(len(filled[1]), len(entries), wanted, self.config.max_num_seqs, self.stager.max_tokens,
                                          self.config.graph_step_tokens, head)
            if sizes is not None:
                logits = self._run_through_graph(("step",) + sizes, self._padded_batch(filled, head, *sizes))[:wanted]
                mixed = [k for k in self._graphs if isinstance(k, tuple)]
                if len(mixed) > self.GRAPH_STEP_LIMIT:
                    del self._graphs[mixed[0]]
            else:
                logits = self.model.forward(self._batch_as_laid_out(filled, head), self.cache)
        self.commit(entries)
        self.steps += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
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
