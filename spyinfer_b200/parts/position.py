"""Position encodings that a mixer applies to its queries and keys.

``rotary_half``: pairs ``(j, j + r)`` with ``r = rotary_dim / 2``, ``freq_j = theta^(-j/r)``,
``angle = position * freq_j``, all in 32-bit; spymaster2h/spyinfer
src/utils/constant_table.hpp:28-41 (table) and src/backends/cpu/cpu_operator.cpp:397-408
(rotation).  ``no_position``: nothing is applied.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import PositionEncoding
from .registry import register_part

_TABLES = {}


@register_part("rotary_half")
class RotaryHalf(PositionEncoding):
    """params: ``theta``, ``rotary_dim`` (even, at most the head size)."""

    kernel_modules = ("qk_rope_store",)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.theta, self.rotary_dim = float(params["theta"]), int(params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be a positive even number, found {self.rotary_dim}")

    def inverse_frequencies(self) -> torch.Tensor:
        r = self.rotary_dim // 2
        j = torch.arange(r, dtype=torch.float32)
        return torch.pow(torch.tensor(self.theta, dtype=torch.float32), -j / float(r))

    def rotation_table(self):
        key = (self.theta, self.rotary_dim, self.ctx.max_model_len, str(self.ctx.device))
        if key not in _TABLES:
            inv = self.inverse_frequencies().to(self.ctx.device)
            _TABLES[key] = kernels.build_rope_table(inv, self.ctx.max_model_len)
        return _TABLES[key]


@register_part("no_position")
class NoPosition(PositionEncoding):
    pass
