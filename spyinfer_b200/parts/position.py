"""Position encodings that a mixer applies to its queries and keys.

``rotary_half``: pairs ``(j, j + r)`` with ``r = rotary_dim / 2``, ``freq_j = theta^(-j/r)``,
``angle = position * freq_j``, all in 32-bit; spymaster2h/spyinfer
src/utils/constant_table.hpp:28-41 (table) and src/backends/cpu/cpu_operator.cpp:397-408
(rotation).  ``rotary_interleaved``: the same angles on the pairs ``(2j, 2j + 1)`` (the
rule the reference's doc/op.md:58-95 describes and its code does not use).  Both take an
optional ``frequency_scale`` (every frequency divided by it: positions stretched linearly)
or explicit ``inverse_frequencies`` (one per pair: any other frequency function), so a
scaled rotary encoding is a parameter, not a new kernel.  ``no_position``: nothing is applied.
"""
from __future__ import annotations

import torch

from .. import kernels
from .base import PositionEncoding
from .registry import register_part

_TABLES = {}


@register_part("rotary_half")
class RotaryHalf(PositionEncoding):
    graph_safe = True
    """params: ``theta``, ``rotary_dim`` (even, at most the head size); optional
    ``frequency_scale`` (default 1) and ``inverse_frequencies`` (a list of ``rotary_dim / 2``
    numbers that replaces ``theta^(-j/r)``)."""

    kernel_modules = ("qk_rope_store",)

    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.theta, self.rotary_dim = float(params["theta"]), int(params["rotary_dim"])
        if self.rotary_dim <= 0 or self.rotary_dim % 2:
            raise ValueError(f"rotary_dim must be a positive even number, found {self.rotary_dim}")
        self.frequency_scale = float(params.get("frequency_scale", 1.0))
        if not self.frequency_scale > 0.0:
            raise ValueError(f"frequency_scale must be positive, found {self.frequency_scale}")
        self.given = params.get("inverse_frequencies")
        if self.given is not None and len(self.given) != self.rotary_dim // 2:
            raise ValueError(f"inverse_frequencies must name {self.rotary_dim // 2} frequencies, found {len(self.given)}")

    def inverse_frequencies(self) -> torch.Tensor:
        r = self.rotary_dim // 2
        if self.given is not None:
            inv = torch.tensor([float(f) for f in self.given], dtype=torch.float32)
        else:
            j = torch.arange(r, dtype=torch.float32)
            inv = torch.pow(torch.tensor(self.theta, dtype=torch.float32), -j / float(r))
        return inv / self.frequency_scale if self.frequency_scale != 1.0 else inv

    def rotation_table(self):
        key = (self.theta, self.rotary_dim, self.frequency_scale, tuple(self.given) if self.given is not None else None,
               self.ctx.max_model_len, str(self.ctx.device))
        if key not in _TABLES:
            inv = self.inverse_frequencies().to(self.ctx.device)
            _TABLES[key] = kernels.build_rope_table(inv, self.ctx.max_model_len)
        return _TABLES[key]


@register_part("rotary_interleaved")
class RotaryInterleaved(RotaryHalf):
    """As ``rotary_half`` with the pairs ``(2j, 2j + 1)``."""

    pairing = "interleaved"


@register_part("no_position")
class NoPosition(PositionEncoding):
    graph_safe = True
    pass
