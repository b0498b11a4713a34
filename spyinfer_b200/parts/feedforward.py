"""Dense gated feed-forward: ``down(act(gate(x)) * up(x))``, no biases.

spymaster2h/spyinfer src/models/qwen3.hpp:233-263 with SiLU as the activation (SwiGLU:
src/backends/cpu/x64/kernels.cpp:242-247).  The gate and up projections are fused into one
matrix at load; on the bfloat16 path their rows are interleaved and the activation runs in
the product's epilogue, so the gate and up activations never reach memory.  The output may
come back as a stack of split-K partial products, which the next norm adds to the residual.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import FeedForward
from .linear import Linear
from .registry import register_part


@register_part("gated_mlp")
class GatedMLP(FeedForward):
    graph_safe = True
    """params: ``hidden_size``, ``intermediate_size``, ``activation`` ("silu"), ``prefix``."""

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden, self.inter = int(params["hidden_size"]), int(params["intermediate_size"])
        if params.get("activation", "silu") != "silu":
            raise ValueError(f"gated_mlp: activation {params['activation']!r} is not implemented (only \"silu\")")
        self.prefix = params.get("prefix", "")
        self.gate_up = self.down = None
        self.fused = False

    def weight_decls(self):
        p = self.prefix
        return [WeightDecl(p + "gate_proj.weight", (self.inter, self.hidden)),
                WeightDecl(p + "up_proj.weight", (self.inter, self.hidden)),
                WeightDecl(p + "down_proj.weight", (self.hidden, self.inter))]

    def bind(self, tensors):
        p = self.prefix
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        if gate.dtype != up.dtype:
            gate, up = gate.float(), up.float()
        self.fused = (self.ctx.dtype == torch.bfloat16 and gate.dtype == torch.bfloat16
                      and kernels.tensor_core_gemm_takes(2 * self.inter, self.hidden))
        if self.fused:
            # rows alternate gate_i, up_i: the tensor-core product applies SwiGLU in its epilogue
            self.gate_up = Linear(torch.stack([gate, up], dim=1).reshape(2 * self.inter, self.hidden).contiguous(), self.ctx.dtype)
        else:
            self.gate_up = Linear(torch.cat([gate, up], dim=0).contiguous(), self.ctx.dtype)
        self.down = Linear(tensors[p + "down_proj.weight"], self.ctx.dtype)
        self.gate_up.hint_next = not self.fused       # fused: the down product follows at once

    def linears(self):
        return [self.gate_up, self.down]

    def modules(self):
        return ([] if self.fused else ["swiglu"]) + self.gate_up.modules() + self.down.modules()

    def forward(self, x):
        if self.fused:
            return self.down(self.gate_up(x, epilogue="swiglu"), defer=self.defer_output)
        gu = self.gate_up(x)
        z = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        kernels.swiglu(gu, z)
        return self.down(z)
