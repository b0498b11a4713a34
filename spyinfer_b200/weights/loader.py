"""Binding a checkpoint's tensors to a model's declared weights, by tensor name.

The model declares what it needs (``WeightDecl``: full name, shape, how a random model
fills it).  ``load_checkpoint`` reads a model folder and returns ``{name: tensor}`` on the
device, or raises ONE ``WeightError`` that lists every missing tensor, every unexpected
tensor and every wrong shape or unusable dtype.  (The reference reports a missing tensor
as a bare ``std::out_of_range`` and never compares shapes: spymaster2h/spyinfer
src/utils/weight_reader.hpp:19-26, src/utils/safetensors_reader.cpp:84-99.)

Storage: BF16 stays bfloat16; F32 stays float32; F16 is widened to float32 (exact);
integer tables become int32.
"""
from __future__ import annotations

import weakref
from collections.abc import Mapping
from dataclasses import dataclass
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile, shard_paths


@dataclass(frozen=True)
class WeightDecl:
    """One tensor a model needs.  ``init`` says how a random model fills it: ``"normal"``
    (zero mean), ``"one_plus_normal"`` (norm gains) or ``"zeros"``.  ``integer`` marks an
    index table, kept as int32."""

    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    integer: bool = False


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every difference."""

    def __init__(self, where: str, missing: Sequence[str], unexpected: Sequence[str], wrong: Sequence[str]):
        self.missing, self.unexpected, self.wrong = list(missing), list(unexpected), list(wrong)
        lines = [f"{where}: the checkpoint does not fit the model"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong:
            lines.append(f"  wrong shape or dtype ({len(self.wrong)}):")
            lines += ["    " + w for w in self.wrong]
        super().__init__("\n".join(lines))


def _store(t: torch.Tensor, decl: WeightDecl) -> torch.Tensor:
    if decl.integer:
        return t.to(torch.int32)
    if t.dtype == torch.float16:
        return t.to(torch.float32)
    return t


class LazyTensors(Mapping):
    """``name -> tensor`` whose tensors are made when they are asked for (read from the checkpoint and
    copied to the device, or drawn at random) and not kept: a model that binds its parts one after the
    other, each turning what it gets into the layout it computes with, then never holds the whole
    checkpoint beside the model.  A tensor that is asked for again while the first one is still in
    use (a tied head and its embedding table) is the same object, not a second copy."""

    def __init__(self, names: Iterable[str], make: Callable[[str], torch.Tensor], on_close: Optional[Callable[[], None]] = None):
        self._names = list(names)
        self._known = set(self._names)
        self._make = make
        self._alive = weakref.WeakValueDictionary()
        self._on_close = on_close

    def __getitem__(self, name: str) -> torch.Tensor:
        if name not in self._known:
            raise KeyError(name)
        t = self._alive.get(name)
        if t is None:
            t = self._make(name)
            self._alive[name] = t
        return t

    def __iter__(self):
        return iter(self._names)

    def __len__(self):
        return len(self._names)

    def close(self) -> None:
        if self._on_close is not None:
            self._on_close()
            self._on_close = None


def open_checkpoint(model_dir: str, decls: Iterable[WeightDecl], device, ignorable: Sequence[str] = ()) -> LazyTensors:
    """Checks the folder against the declarations (ONE ``WeightError`` that lists every missing,
    unexpected and wrong tensor) and returns its tensors as a ``LazyTensors``: each is read and
    copied to ``device`` when it is asked for.  ``stored_dtypes`` of the result tells how each
    tensor is stored.  Close it when the model is bound.
    ``ignorable`` names tensors that may be present without being used (the separate head
    of a checkpoint whose configuration ties it to the embedding)."""
    decls = list(decls)
    try:
        files = [SafetensorsFile(p) for p in shard_paths(model_dir)]
    except SafetensorsError as e:
        raise WeightError(str(e), [], [], []) from None

    def close():
        for f in files:
            f.close()

    where: Dict[str, SafetensorsFile] = {}
    for f in files:
        for name in f.names():
            where[name] = f
    missing, wrong = [], []
    wanted = {d.name for d in decls}
    for d in decls:
        f = where.get(d.name)
        if f is None:
            missing.append(d.name)
            continue
        if f.shape(d.name) != tuple(d.shape):
            wrong.append(f"{d.name}: expected shape {list(d.shape)}, found {list(f.shape(d.name))} in {f.path}")
        is_int = f.dtype(d.name) in (torch.int32, torch.int64)
        if is_int != d.integer:
            wrong.append(f"{d.name}: expected {'an integer' if d.integer else 'a floating-point'} tensor, found {f.dtype(d.name)} in {f.path}")
    unexpected = sorted(n for n in where if n not in wanted and n not in set(ignorable))
    if missing or unexpected or wrong:
        close()
        raise WeightError(model_dir, missing, unexpected, wrong)
    by_name = {d.name: d for d in decls}
    out = LazyTensors([d.name for d in decls], lambda n: _store(where[n].tensor(n), by_name[n]).to(device).contiguous(), close)
    out.stored_dtypes = {d.name: where[d.name].dtype(d.name) for d in decls}
    return out


def load_checkpoint(model_dir: str, decls: Iterable[WeightDecl], device, ignorable: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """Every declared tensor on ``device`` (see ``open_checkpoint`` for the checks and for a way
    that does not hold them all at once)."""
    lazy = open_checkpoint(model_dir, decls, device, ignorable)
    try:
        return {name: lazy[name] for name in lazy}
    finally:
        lazy.close()
