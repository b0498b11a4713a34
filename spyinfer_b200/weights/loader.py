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

from dataclasses import dataclass
from typing import Dict, Iterable, List, Sequence, Tuple

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


def load_checkpoint(model_dir: str, decls: Iterable[WeightDecl], device, ignorable: Sequence[str] = ()) -> Dict[str, torch.Tensor]:
    """``ignorable`` names tensors that may be present without being used (the separate head
    of a checkpoint whose configuration ties it to the embedding)."""
    decls = list(decls)
    try:
        files = [SafetensorsFile(p) for p in shard_paths(model_dir)]
    except SafetensorsError as e:
        raise WeightError(str(e), [], [], []) from None
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
    try:
        if missing or unexpected or wrong:
            raise WeightError(model_dir, missing, unexpected, wrong)
        out = {}
        for d in decls:
            out[d.name] = _store(where[d.name].tensor(d.name), d).to(device).contiguous()
        return out
    finally:
        for f in files:
            f.close()
