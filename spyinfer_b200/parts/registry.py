"""The registry of parts: a ``PartSpec.kind`` names a class here, and ``build_part`` makes it.

A model is put together only through this registry, so a new mixer, feed-forward, norm,
position encoding or block arrangement is added by registering a class, from anywhere
(a test included), without touching the engine:

    @register_part("my_mixer")
    class MyMixer(Mixer): ...
"""
from __future__ import annotations

from typing import Dict, Type

from ..config.spec import PartSpec

_PARTS: Dict[str, Type] = {}


def register_part(kind: str):
    def wrap(cls):
        cls.kind = kind
        _PARTS[kind] = cls
        return cls

    return wrap


def known_parts():
    return sorted(_PARTS)


def build_part(spec: PartSpec, ctx):
    """``ctx`` is the ``BuildContext`` (dtype, device, limits) every part is built with."""
    if spec.kind not in _PARTS:
        raise KeyError(f"unknown part kind {spec.kind!r}; registered: {', '.join(known_parts())}")
    return _PARTS[spec.kind](dict(spec.params), ctx)
