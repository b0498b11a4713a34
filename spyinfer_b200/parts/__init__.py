"""The parts a model is put together from, and their registry."""
from .base import Block, BuildContext, FeedForward, Mixer, Norm, Part, PositionEncoding
from .block import PreNormBlock, build_block, register_block
from .registry import build_part, known_parts, register_part
from . import attention, embedding, feedforward, norm, position  # noqa: F401  (register the built-in parts)
from .linear import Linear

__all__ = ["Block", "BuildContext", "FeedForward", "Mixer", "Norm", "Part", "PositionEncoding", "PreNormBlock", "build_block",
           "register_block", "build_part", "known_parts", "register_part", "Linear"]
