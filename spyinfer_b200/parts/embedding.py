"""Token embedding and output head.

``token_embedding``: ``h[t] = E[ids[t]]`` into the 32-bit residual stream, no scaling
(spymaster2h/spyinfer src/models/qwen3.hpp:114-119).  ``lm_head``: ``logits = x @ W^T`` in
32-bit out, ``W`` the embedding table when tied (qwen3.hpp:46, 295-301).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import Part
from .linear import Linear
from .registry import register_part


@register_part("token_embedding")
class TokenEmbedding(Part):
    graph_safe = True
    """params: ``vocab_size``, ``hidden_size``, ``weight`` (full tensor name)."""

    kernel_modules = ("embedding",)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab, self.hidden, self.weight_name = int(params["vocab_size"]), int(params["hidden_size"]), params["weight"]
        self.table = None

    def weight_decls(self):
        return [WeightDecl(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.table = tensors[self.weight_name]

    def forward(self, token_ids, status=None):
        out = torch.empty((token_ids.shape[0], self.hidden), dtype=torch.float32, device=token_ids.device)
        return kernels.embedding(self.table, token_ids, out, status)


@register_part("lm_head")
class LMHead(Part):
    graph_safe = True
    """params: ``vocab_size``, ``hidden_size``, ``tied``, ``weight`` (full name when untied),
    ``tied_to`` (full name of the embedding table when tied)."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab, self.hidden, self.tied = int(params["vocab_size"]), int(params["hidden_size"]), bool(params["tied"])
        self.weight_name = params["tied_to"] if self.tied else params["weight"]
        self.ignorable = [params["weight"]] if self.tied else []
        self.linear = None

    def weight_decls(self):
        return [] if self.tied else [WeightDecl(self.weight_name, (self.vocab, self.hidden))]

    def bind(self, tensors):
        self.linear = Linear(tensors[self.weight_name], self.ctx.dtype)

    def modules(self):
        return self.linear.modules()

    def linears(self):
        return [self.linear]

    def forward(self, x):
        return self.linear(x, out_dtype=torch.float32)
