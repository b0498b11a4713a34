"""Interfaces of the parts a model is put together from.

A part is built from its own sizes and constants (``params``) and a ``BuildContext``; it
declares the tensors it needs by names relative to its layer's prefix, gets them bound, and
then only computes.  No part knows which model it is in, which layer it is, or what other
parts the model has.

* ``Norm``: ``forward(x)`` and ``forward_add(residual, delta)`` (residual sum fused in).
* ``PositionEncoding``: owned by a mixer; hands out what the mixer's kernel needs.
* ``Mixer``: ``forward(x, batch, cache)``; declares what it keeps between steps through
  ``cache_need()`` (pages of keys and values, a fixed-size state per request, or nothing).
* ``FeedForward``: ``forward(x)``.
* ``Block``: the arrangement of a layer's parts around the residual stream (for the usual
  pre-norm block two norms, a mixer and a feed-forward; an arrangement states the roles it
  needs): ``forward(hidden, delta, batch, cache) -> (hidden, delta)``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence

import torch

from ..weights.loader import WeightDecl


@dataclass
class BuildContext:
    """What every part is built with.  ``dtype`` is the storage type of activations and of
    the cache: bfloat16 (the serving path) or float32 (everything in true 32-bit)."""

    dtype: torch.dtype
    device: torch.device
    max_model_len: int


class Part:
    kind: str = ""
    #: kernel modules (``csrc/<name>.cu``) this part launches; built before the first step
    kernel_modules: Sequence[str] = ()
    #: True when ``forward`` launches the same kernels with the same arguments for every batch of the same sizes
    #: (tokens, requests, wanted rows): no look at the batch's content on the host, no wait for the device, no
    #: allocation that outlives the call.  A model whose parts all say so has its small steps captured in CUDA
    #: graphs and replayed; one part that does not keeps the whole model on launches one by one.
    graph_safe: bool = False

    def __init__(self, params: Dict[str, Any], ctx: BuildContext):
        self.params = params
        self.ctx = ctx

    def weight_decls(self) -> List[WeightDecl]:
        """Tensors this part needs, named relative to its layer's prefix."""
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receives the declared tensors (same relative names), already on the device."""

    def modules(self) -> List[str]:
        return list(self.kernel_modules)

    def linears(self) -> List:
        """The part's ``Linear`` products in the order ``forward`` runs them (the model tells each
        which weight is read next, so that it can ask for it ahead of time)."""
        return []


class Norm(Part):
    def forward(self, x: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        raise NotImplementedError

    def forward_add(self, residual: torch.Tensor, delta: Optional[torch.Tensor], rows: Optional[torch.Tensor] = None,
                    out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        """``residual += delta`` (32-bit, in place, skipped when ``delta`` is None), then the
        norm of the sum.  With ``rows`` only those rows are normed and nothing is written back.
        ``delta`` is ``[rows, size]``, or a stack ``[splits, rows, size]`` of float32 partial
        products (a mixer or feed-forward may hand its last product over unsummed); all are added."""
        raise NotImplementedError


class PositionEncoding(Part):
    #: which two elements of a head the table's angle ``j`` rotates: "half" ``(j, j + r)`` or
    #: "interleaved" ``(2j, 2j + 1)``
    pairing: str = "half"

    def rotation_table(self) -> Optional[torch.Tensor]:
        """For encodings that rotate pairs of each head's elements: float32 ``[positions, r, 2]``
        of (cos, sin) per position and pair, which the fused q/k kernel applies by the part's
        ``pairing`` rule; None for no rotation."""
        return None


class Mixer(Part):
    #: True: ``forward`` may hand its result over as a stack ``[splits, rows, size]`` of float32 partial
    #: products (its last product then skips its own reduction), which ``Norm.forward_add`` adds to the
    #: residual.  A block arrangement that does anything else with the result sets this to False on
    #: the part and always gets ``[rows, size]``.
    defer_output: bool = True

    def cache_need(self):
        """A ``PagedCacheNeed``, a ``StateCacheNeed`` or None."""
        return None

    def forward(self, x: torch.Tensor, batch, cache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    defer_output: bool = True     # as ``Mixer.defer_output``

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of a layer's parts.  ``required`` and ``optional`` name the roles it takes
    (``LayerSpec.roles()``); the parts arrive as ``self.parts[role]`` and as attributes of the
    same names (None for an optional role that the layer does not have)."""

    kind: str = ""
    graph_safe: bool = False      # as ``Part.graph_safe``, for the arrangement's own code
    required: Sequence[str] = ("mixer_norm", "mixer", "ffn_norm", "feed_forward")
    optional: Sequence[str] = ()

    def __init__(self, parts: Dict[str, Part]):
        missing = [r for r in self.required if r not in parts]
        unknown = [r for r in parts if r not in self.required and r not in self.optional]
        if missing or unknown:
            raise ValueError(f"block arrangement {self.kind!r} takes the roles {list(self.required)} (optional {list(self.optional)}): "
                             f"missing {missing}, unknown {unknown}")
        self.parts = dict(parts)
        for role in list(self.required) + list(self.optional):
            setattr(self, role, parts.get(role))

    def forward(self, hidden: torch.Tensor, delta: Optional[torch.Tensor], batch, cache):
        """``hidden`` is the 32-bit residual stream; ``delta`` the previous block's output
        that is still to be added to it (None for the first).  Returns the same pair."""
        raise NotImplementedError
