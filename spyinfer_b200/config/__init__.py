"""Typed configuration: the architecture registry, the model description and the engine's options."""
from .engine_config import EngineConfig
from .model_config import (ArchitectureConfig, ConfigError, config_from_json, known_architectures, load_model_config,
                           register_architecture)
from .spec import LayerSpec, ModelSpec, PagedCacheNeed, PartSpec, RunEntry, StateCacheNeed
from . import qwen3 as _qwen3  # registers "Qwen3ForCausalLM"
from .qwen3 import Qwen3Config

__all__ = ["EngineConfig", "ArchitectureConfig", "ConfigError", "config_from_json", "known_architectures",
           "load_model_config", "register_architecture", "LayerSpec", "ModelSpec", "PagedCacheNeed", "PartSpec",
           "RunEntry", "StateCacheNeed", "Qwen3Config"]
