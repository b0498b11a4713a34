"""Block arrangements around the 32-bit residual stream.

``pre_norm``: ``h += mixer(norm(h)); h += ffn(norm(h))`` (spymaster2h/spyinfer
src/models/qwen3.hpp:127-133, 216-230, 272-277).  Each residual sum is fused into the norm
that follows it: a block receives the previous block's output as ``delta``, still to be
added, and hands its own feed-forward output on in the same way.
"""
from __future__ import annotations

from .base import Block

_BLOCKS = {}


def register_block(kind: str):
    def wrap(cls):
        cls.kind = kind
        _BLOCKS[kind] = cls
        return cls

    return wrap


def build_block(kind: str, parts) -> Block:
    """``parts``: role -> built part (``LayerSpec.roles()`` with every ``PartSpec`` built)."""
    if kind not in _BLOCKS:
        raise KeyError(f"unknown block arrangement {kind!r}; registered: {', '.join(sorted(_BLOCKS))}")
    return _BLOCKS[kind](dict(parts))


@register_block("pre_norm")
class PreNormBlock(Block):
    graph_safe = True

    def forward(self, hidden, delta, batch, cache):
        x = self.mixer_norm.forward_add(hidden, delta)
        a = self.mixer.forward(x, batch, cache)
        x = self.ffn_norm.forward_add(hidden, a)
        return hidden, self.feed_forward.forward(x)
