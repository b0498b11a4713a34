"""The data that describes a model to the engine: parts, layers, and the order they run in.

A model is a list of layers; a layer is a block arrangement over named parts (for the usual
pre-norm block: a norm before the mixer, the mixer, a norm before the feed-forward, the
feed-forward; an arrangement may name others, or fewer); each part is a
``PartSpec``: the registry key of its kind plus its sizes and constants.  The order in
which layers run is a list of ``RunEntry`` and may name a layer twice, or let an entry
read the cache that an earlier entry wrote.  Nothing here knows a model by name: an
architecture's typed configuration produces a ``ModelSpec`` and the engine builds from it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple


@dataclass(frozen=True)
class PartSpec:
    """One part: ``kind`` is a key of the part registry, ``params`` its sizes and constants."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: the arrangement (a key of the block registry), its parts by the role they play
    in it, and the prefix of its tensors' names in the checkpoint.

    The four roles of the usual block have fields of their own; an arrangement that needs other
    parts (norms after the mixer and the feed-forward, a second feed-forward, ...) names them in
    ``more``, and one that needs fewer leaves fields at None.  Which roles are required is the
    arrangement's statement (``Block.required`` / ``Block.optional``), checked when the layer is
    built.  The role ``mixer``, if present, is the part that owns the layer's cache."""

    block: str
    mixer_norm: Optional[PartSpec] = None
    mixer: Optional[PartSpec] = None
    ffn_norm: Optional[PartSpec] = None
    feed_forward: Optional[PartSpec] = None
    weight_prefix: str = ""
    more: Dict[str, PartSpec] = field(default_factory=dict)

    def roles(self) -> Dict[str, PartSpec]:
        """role -> part, in the order the parts' tensors are declared."""
        out = {r: getattr(self, r) for r in ("mixer_norm", "mixer", "ffn_norm", "feed_forward") if getattr(self, r) is not None}
        for r, p in self.more.items():
            if r in out:
                raise ValueError(f"layer role {r!r} is given twice")
            out[r] = p
        return out

    def __hash__(self):
        return hash((self.block, self.weight_prefix, tuple(self.roles().items())))


@dataclass(frozen=True)
class RunEntry:
    """One position in the run order.

    ``layer`` indexes ``ModelSpec.layers``.  Every entry owns a cache of its own unless
    ``cache_of`` names an earlier entry (by its index in the run order): then this entry's
    mixer reads that entry's cache and stores nothing.
    """

    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: List[LayerSpec]
    run_order: List[RunEntry]
    final_norm: PartSpec
    head: PartSpec
    max_position: int
    eos_token_id: int = -1
    bos_token_id: int = -1

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        for i, e in enumerate(self.run_order):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"run order entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"run order entry {i} reads the cache of entry {e.cache_of}, which is not an earlier entry")
                if self.run_order[e.cache_of].cache_of is not None:
                    raise ValueError(f"run order entry {i} reads the cache of entry {e.cache_of}, which owns none")


@dataclass(frozen=True)
class PagedCacheNeed:
    """A mixer that keeps keys and values of past tokens in pages.

    ``window`` is ``None`` when every past key is kept, else the number of most recent
    keys (the query's own included) that a query can see.  Entries of the run order with
    equal needs share one group of pages in the cache manager.
    """

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self) -> Tuple:
        return ("paged", self.num_kv_heads, self.head_dim, self.window)


@dataclass(frozen=True)
class StateCacheNeed:
    """A mixer that keeps a state of fixed size for each live request, in that request's slot."""

    shape: Tuple[int, ...]
    dtype: str = "float32"

    def group_key(self) -> Tuple:
        return ("state", tuple(self.shape), self.dtype)
