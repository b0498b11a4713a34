"""Grouped-query softmax attention over the paged cache, with optional per-head q/k RMSNorm,
a position encoding of its own, and an optional window.

Order of operations (spymaster2h/spyinfer src/models/qwen3.hpp:136-213): q, k, v projections
(fused into one matrix here), RMSNorm over head_dim on q and k with one shared weight each,
position encoding on q and k, keys and values stored into the cache, attention, output
projection.  kv head = head * nkv / nh, score = q.k / sqrt(head_dim), causal on absolute
positions (src/backends/cpu/cpu_attention.cpp:59, :96, :100-110).  A windowed layer sees
the last ``window`` keys, the query's own included.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..config.spec import PagedCacheNeed
from ..weights.loader import WeightDecl
from .base import Mixer
from .linear import Linear
from .registry import build_part, register_part


@register_part("attention")
class Attention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``qk_norm_eps``
    (None: no q/k norm), ``position`` (a PartSpec or None), ``window`` (None: all keys),
    ``scale`` (None: 1/sqrt(head_dim)), ``prefix``, ``qkv_bias`` and ``o_bias`` (default false: the
    projections have bias tensors ``{q,k,v}_proj.bias`` / ``o_proj.bias``)."""

    graph_safe = True

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(params["hidden_size"])
        self.nh, self.nkv, self.hd = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        if self.nh % self.nkv:
            raise ValueError(f"attention: {self.nh} heads do not group over {self.nkv} key/value heads")
        if self.hd % 4 or self.hd > 512:
            raise ValueError(f"attention: head_dim {self.hd} must be a multiple of 4 and at most 512")
        self.qk_norm_eps = params.get("qk_norm_eps")
        self.window = params.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError(f"attention: window {self.window} must be positive")
        self.scale = float(params["scale"]) if params.get("scale") is not None else 1.0 / math.sqrt(float(self.hd))
        self.prefix = params.get("prefix", "")
        self.qkv_bias, self.o_bias = bool(params.get("qkv_bias", False)), bool(params.get("o_bias", False))
        pos = params.get("position")
        self.position = build_part(pos, ctx) if pos is not None else None
        self.qkv = self.o = self.q_norm = self.k_norm = self.rope_table = None
        # which attention kernels take these sizes (the page size, known at the first step, decides between them)
        self.tc = kernels.attention_tc_takes(self.nh, self.nkv, self.hd, ctx.dtype)        # tcgen05, pages that are one TMA box
        self.mma = kernels.attention_mma_takes(self.nh, self.nkv, self.hd, ctx.dtype)      # mma.sync, any page size
        self._split_plans = {}

    def weight_decls(self):
        p, nh, nkv, hd, H = self.prefix, self.nh, self.nkv, self.hd, self.hidden
        decls = [WeightDecl(p + "q_proj.weight", (nh * hd, H)), WeightDecl(p + "k_proj.weight", (nkv * hd, H)),
                 WeightDecl(p + "v_proj.weight", (nkv * hd, H)), WeightDecl(p + "o_proj.weight", (H, nh * hd))]
        if self.qk_norm_eps is not None:
            decls += [WeightDecl(p + "q_norm.weight", (hd,), init="one_plus_normal"),
                      WeightDecl(p + "k_norm.weight", (hd,), init="one_plus_normal")]
        if self.qkv_bias:
            decls += [WeightDecl(p + "q_proj.bias", (nh * hd,)), WeightDecl(p + "k_proj.bias", (nkv * hd,)), WeightDecl(p + "v_proj.bias", (nkv * hd,))]
        if self.o_bias:
            decls += [WeightDecl(p + "o_proj.bias", (H,))]
        return decls

    def bind(self, tensors):
        p = self.prefix
        qkv = [tensors[p + n] for n in ("q_proj.weight", "k_proj.weight", "v_proj.weight")]
        if len({t.dtype for t in qkv}) > 1:
            qkv = [t.float() for t in qkv]
        bias = None
        if self.qkv_bias:
            bias = torch.cat([tensors[p + n].float() for n in ("q_proj.bias", "k_proj.bias", "v_proj.bias")]).contiguous()
        self.qkv = Linear(torch.cat(qkv, dim=0).contiguous(), self.ctx.dtype, bias=bias)
        self.o = Linear(tensors[p + "o_proj.weight"], self.ctx.dtype, bias=tensors[p + "o_proj.bias"] if self.o_bias else None)
        if self.qk_norm_eps is not None:
            self.q_norm, self.k_norm = tensors[p + "q_norm.weight"], tensors[p + "k_norm.weight"]
            if self.q_norm.dtype != self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    def modules(self):
        mods = ["qk_rope_store"] + (["attention_tc", "attention_decode"] if self.tc else []) + (["attention_mma"] if self.mma else ["attention_generic"]) + self.qkv.modules() + self.o.modules()
        if self.position is not None:
            mods += self.position.modules()
        return mods

    def linears(self):
        return [self.qkv, self.o]

    def cache_need(self):
        return PagedCacheNeed(self.nkv, self.hd, int(self.window) if self.window is not None else None)

    def split_plan(self, num_seqs: int):
        """(split_keys, max_splits) for decoding ``num_seqs`` requests: the keys of every request
        are cut into ranges so that (requests x key/value heads x ranges) blocks fill whole waves
        of the GPU's block slots (two a SM) as evenly as possible; at most 16 ranges, ranges of at
        least 256 keys and a multiple of 64.  The plan depends on the (padded) batch size only."""
        plan = self._split_plans.get(num_seqs)
        if plan is None:
            slots, per_split, best = 2 * torch.cuda.get_device_properties(self.ctx.device).multi_processor_count, num_seqs * self.nkv, None
            most = max(1, min(16, self.ctx.max_model_len // 256))
            for splits in range(1, most + 1):
                blocks = per_split * splits
                waves = -(-blocks // slots)
                fill = min(blocks, slots) / slots if waves == 1 else blocks / (waves * slots)
                keys = self.ctx.max_model_len / splits
                score = (fill * keys / (keys + 200.0), -splits)       # a block's fixed cost is worth about 200 keys
                if best is None or score > best[0]:
                    best = (score, splits)
            splits = best[1]
            split_keys = max(256, (-(-self.ctx.max_model_len // splits) + 63) // 64 * 64)
            plan = (split_keys, -(-self.ctx.max_model_len // split_keys))
            self._split_plans[num_seqs] = plan
        return plan

    def forward(self, x, batch, cache):
        if self.rope_table is None and self.position is not None:
            self.rope_table = self.position.rotation_table()   # built by the first step (an eager one)
        qkv = self.qkv(x, defer=True)
        q = None
        if qkv.dim() == 3:   # split-K partial products: summed inside the next kernel, q gets a buffer of its own
            q = torch.empty((x.shape[0], self.nh * self.hd), dtype=x.dtype, device=x.device)
        q = kernels.qk_rope_store(qkv, self.nh, self.nkv, self.hd, self.q_norm, self.k_norm, float(self.qk_norm_eps or 0.0),
                                  self.rope_table, batch.positions, batch.seq_of_token, cache.block_table, cache.pages,
                                  store=cache.writes, status=batch.status, q_out=q,
                                  pairing=self.position.pairing if self.position is not None else "half")
        out = torch.empty((x.shape[0], self.nh * self.hd), dtype=x.dtype, device=x.device)
        decoding = batch.one_token_each         # every request brings one token
        boxes = self.tc and cache.page_size in kernels.ATTENTION_TMA_PAGE_SIZES        # a page is one TMA box
        if (boxes and decoding and batch.num_seqs <= kernels.ATTENTION_DECODE_MAX_SEQS and batch.num_seqs * self.nkv <= kernels.ATTENTION_DECODE_MAX_PAIRS
                and kernels.attention_decode_takes(self.nh, self.nkv, self.hd, cache.page_size, x.dtype)):
            # memory-bound: one persistent block per SM, the batch's key tiles shared out evenly, pages by TMA
            kernels.attention_decode(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.q_start,
                                     batch.num_seqs, self.scale, window=self.window, status=batch.status)
        elif decoding and self.mma:
            # page sizes that are no TMA box, or very many requests: keys split across blocks by a plan per batch size
            split_keys, max_splits = self.split_plan(batch.num_seqs)
            kernels.attention_mma(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.q_start,
                                  batch.num_seqs, self.scale, window=self.window, split_keys=split_keys, max_splits=max_splits,
                                  status=batch.status)
        elif boxes:
            # prompt portions on blocks of 256 query rows; requests that decode beside them (laid out first in the batch)
            # go through the decode kernel, which reads a cache two to three times faster for one token than a 256-row block does
            head = batch.one_token_head      # the step function says whether a launch of the decode kernel pays for them
            if not (0 < head <= kernels.ATTENTION_DECODE_MAX_SEQS and head * self.nkv <= kernels.ATTENTION_DECODE_MAX_PAIRS
                    and kernels.attention_decode_takes(self.nh, self.nkv, self.hd, cache.page_size, x.dtype)):
                head = 0
            if head:
                kernels.attention_decode(q, self.nh, self.hd, out, cache.pages, cache.block_table[:head], batch.positions, batch.q_start[:head + 1],
                                         head, self.scale, window=self.window, status=batch.status)
            kernels.attention_tc(q, self.nh, self.hd, out, cache.pages, cache.block_table[head:], batch.positions, batch.q_start[head:],
                                 batch.num_seqs - head, self.scale, window=self.window, status=batch.status)
        elif self.mma:
            kernels.attention_mma(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.q_start,
                                  batch.num_seqs, self.scale, window=self.window, status=batch.status)
        else:
            # the float32 path, head sizes above 128 or no multiple of 8, more than 16 query heads a key/value head
            kernels.attention_generic(q, self.nh, self.hd, out, cache.pages, cache.block_table, batch.positions, batch.seq_of_token,
                                      self.scale, window=self.window, status=batch.status)
        return self.o(out, defer=self.defer_output)
