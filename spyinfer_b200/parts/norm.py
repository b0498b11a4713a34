"""RMSNorm: ``x * (1 / sqrt(mean(x^2) + eps)) * weight``, statistics in 32-bit, plain weight.

Formula: spymaster2h/spyinfer src/backends/cpu/x64/kernels.cpp:168-180; used before the
mixer, before the feed-forward and before the head (src/models/qwen3.hpp:127-133, 224-230,
287-293).  The residual sum of the block is fused into the same kernel.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import Norm
from .registry import register_part


@register_part("rms_norm")
class RMSNorm(Norm):
    graph_safe = True
    """params: ``size``, ``eps``, ``weight`` (the tensor's relative name)."""

    kernel_modules = ("rmsnorm",)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.size, self.eps, self.weight_name = int(params["size"]), float(params["eps"]), params.get("weight", "weight")
        self.weight = None

    def weight_decls(self):
        return [WeightDecl(self.weight_name, (self.size,), init="one_plus_normal")]

    def bind(self, tensors):
        self.weight = tensors[self.weight_name]

    def forward(self, x, out_dtype=None):
        out = torch.empty(x.shape, dtype=out_dtype or self.ctx.dtype, device=x.device)
        return kernels.rmsnorm(x, self.weight, self.eps, out)

    def forward_add(self, residual, delta, rows=None, out_dtype=None):
        n = residual.shape[0] if rows is None else rows.shape[0]
        out = torch.empty((n, self.size), dtype=out_dtype or self.ctx.dtype, device=residual.device)
        return kernels.rmsnorm(residual, self.weight, self.eps, out, delta=delta, rows=rows, write_back=delta is not None and rows is None)
