"""Random weights from a configuration and a seed: in memory on any device, or as a model
folder (config.json, model.safetensors) that the ordinary loader reads.

Every tensor has a generator of its own, seeded from the seed and the tensor's name, so a
tensor's values do not depend on which other tensors the model has or on their order.
Values are drawn in float32 and rounded to bfloat16, the storage type.  CPU and CUDA
generators are different streams: a folder written on the CPU and a model initialised on
the GPU from the same seed are two different (equally distributed) models.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Dict, Iterable, Iterator, Tuple

import torch

from .loader import WeightDecl
from .safetensors_io import write_safetensors


def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(decl: WeightDecl, seed: int, std: float, norm_std: float, device) -> torch.Tensor:
    if decl.integer:
        raise ValueError(f"{decl.name}: no rule for a random integer table")
    g = torch.Generator(device=device).manual_seed(_tensor_seed(seed, decl.name))
    if decl.init == "zeros":
        return torch.zeros(decl.shape, dtype=torch.bfloat16, device=device)
    x = torch.randn(decl.shape, generator=g, device=device, dtype=torch.float32)
    if decl.init == "normal":
        x.mul_(std)
    elif decl.init == "one_plus_normal":
        x.mul_(norm_std).add_(1.0)
    else:
        raise ValueError(f"{decl.name}: unknown init rule {decl.init!r}")
    return x.to(torch.bfloat16)


def random_tensors(decls: Iterable[WeightDecl], seed: int, std: float = 0.02, norm_std: float = 0.05,
                   device="cpu") -> Iterator[Tuple[str, torch.Tensor]]:
    for d in decls:
        yield d.name, random_tensor(d, seed, std, norm_std, device)


def write_model_folder(model_dir: str, config, seed: int, std: float = 0.02, norm_std: float = 0.05, shard_bytes: int = 0,
                       device="cpu") -> None:
    """``config`` is an ``ArchitectureConfig``; the folder gets its config.json and every tensor the
    model declares: in one model.safetensors, or, with ``shard_bytes``, in files of about that size
    (a tensor is never cut) named by a model.safetensors.index.json, as large checkpoints are
    stored.  ``device``: where the values are drawn (see the module's header: CPU and CUDA draw
    different values from one seed)."""
    from ..engine.model import declared_weights  # late: the engine imports this package

    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(config.to_json(), f, indent=1)
    decls = declared_weights(config.to_spec())

    def nbytes(d):
        n = 2
        for k in d.shape:
            n *= int(k)
        return n

    shards, size = [[]], 0
    for d in decls:
        if shard_bytes and shards[-1] and size + nbytes(d) > shard_bytes:
            shards.append([])
            size = 0
        shards[-1].append(d)
        size += nbytes(d)
    if len(shards) == 1:
        names = ["model.safetensors"]
    else:
        names = [f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors" for i in range(len(shards))]
        index = {"metadata": {"total_size": sum(nbytes(d) for d in decls)},
                 "weight_map": {d.name: name for name, part in zip(names, shards) for d in part}}
        with open(os.path.join(model_dir, "model.safetensors.index.json"), "w") as f:
            json.dump(index, f, indent=1)
    for name, part in zip(names, shards):
        layout = [(d.name, torch.bfloat16, tuple(d.shape)) for d in part]
        write_safetensors(os.path.join(model_dir, name), layout, random_tensors(part, seed, std, norm_std, device))
