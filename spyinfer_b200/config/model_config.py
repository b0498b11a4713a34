"""Registry from an architecture's name (config.json ``architectures[0]``) to its typed
configuration, and the entry points that read a model folder's config.json.  A config.json
without an ``architectures`` list is looked up by its ``model_type`` (the one key the
reference requires to name the model, spymaster2h/spyinfer src/models/model_config.hpp:32),
which an architecture may register beside its name.

An architecture registers one class with two methods: ``from_json(dict)`` reads and checks
the architecture's own config.json keys, ``to_spec()`` turns them into a ``ModelSpec``.
The engine never looks at the keys itself.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Type

from .spec import ModelSpec

_ARCHITECTURES: Dict[str, Type["ArchitectureConfig"]] = {}
_MODEL_TYPES: Dict[str, str] = {}      # config.json "model_type" -> architecture name


class ConfigError(ValueError):
    """config.json is missing a key, or holds a value the engine cannot run."""


class ArchitectureConfig:
    """Base of a typed configuration of one architecture."""

    architecture: str = ""

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "ArchitectureConfig":
        raise NotImplementedError

    def to_json(self) -> Dict[str, Any]:
        raise NotImplementedError

    def to_spec(self) -> ModelSpec:
        raise NotImplementedError


def register_architecture(name: str, model_type: str = None):
    """Class decorator: ``@register_architecture("Qwen3ForCausalLM", model_type="qwen3")``."""

    def wrap(cls):
        cls.architecture = name
        _ARCHITECTURES[name] = cls
        if model_type is not None:
            _MODEL_TYPES[model_type] = name
        return cls

    return wrap


def known_architectures():
    return sorted(_ARCHITECTURES)


def config_from_json(data: Dict[str, Any]) -> ArchitectureConfig:
    archs = data.get("architectures")
    if isinstance(archs, str):
        archs = [archs]
    if not archs or not isinstance(archs, list):
        name = _MODEL_TYPES.get(data.get("model_type"))
        if name is None:
            raise ConfigError(f"config.json has no \"architectures\" list and its model_type {data.get('model_type')!r} names no known model; "
                              "known architectures: " + ", ".join(known_architectures()) + "; known model types: " + ", ".join(sorted(_MODEL_TYPES)))
    else:
        name = archs[0]
    if name not in _ARCHITECTURES:
        raise ConfigError(f"unknown architecture {name!r}; known architectures: " + ", ".join(known_architectures()))
    return _ARCHITECTURES[name].from_json(data)


def load_model_config(model_dir: str) -> ArchitectureConfig:
    path = os.path.join(model_dir, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"{path}: no config.json in the model folder")
    with open(path) as f:
        try:
            data = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    return config_from_json(data)
