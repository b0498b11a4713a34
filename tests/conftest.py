"""Shared fixtures: tiny configurations, model folders made in temporary folders, the plain
implementation's logits.  Tests marked ``gpu`` need a CUDA device; everything else runs on
the CPU."""
from __future__ import annotations

import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import plain_model  # noqa: E402


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny configurations that differ in every size and option.  A and B have the sizes of the
# two tiny reference workloads; C adds windows on some layers and a head size of 48; D has
# the head size (64) and group size (5 query heads per key/value head, no power of two) that
# put the bfloat16 path on its tensor-core attention kernel, a window, and a tied head.
TINY = {
    "a": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": 2,
                "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128,
                "vocab_size": 256, "rope_theta": 10000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
                "max_position_embeddings": 1024, "bos_token_id": 1, "eos_token_id": 2},
        seed=11, std=0.02, norm_std=0.05),
    "b": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": 3,
                "hidden_size": 96, "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 32, "intermediate_size": 224,
                "vocab_size": 384, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
                "max_position_embeddings": 2048, "bos_token_id": 0, "eos_token_id": 5},
        seed=22, std=0.03, norm_std=0.1),
    "c": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": 4,
                "hidden_size": 144, "num_attention_heads": 6, "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 200,
                "vocab_size": 517, "rope_theta": 50000.0, "rms_norm_eps": 3e-6, "tie_word_embeddings": False,
                "max_position_embeddings": 4096, "bos_token_id": 3, "eos_token_id": 4, "use_sliding_window": True,
                "sliding_window": 40, "layer_types": ["sliding_attention", "full_attention", "sliding_attention", "full_attention"]},
        seed=33, std=0.05, norm_std=0.2),
    "d": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": 2,
                "hidden_size": 200, "num_attention_heads": 10, "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 328,
                "vocab_size": 1187, "rope_theta": 300000.0, "rms_norm_eps": 2e-6, "tie_word_embeddings": True,
                "max_position_embeddings": 8192, "bos_token_id": 7, "eos_token_id": 8, "use_sliding_window": True,
                "sliding_window": 100, "layer_types": ["full_attention", "sliding_attention"]},
        seed=44, std=0.04, norm_std=0.1),
}


@pytest.fixture(scope="session")
def tiny_models(tmp_path_factory):
    """``name -> (model folder, config dict, weights dict)``; folders are written with the
    safetensors library from ``plain_model.random_weights``, not with the package's writer."""
    from safetensors.torch import save_file

    out = {}
    for name, case in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{name}")
        cfg = case["config"]
        with open(d / "config.json", "w") as f:
            json.dump(cfg, f)
        w = plain_model.random_weights(cfg, case["seed"], case["std"], case["norm_std"])
        save_file({k: v.contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
        out[name] = (str(d), cfg, w)
    return out


@pytest.fixture(scope="session")
def plain_logits_cache():
    """Memo of the plain implementation's whole-sequence logits, keyed by (model, tokens)."""
    cache = {}

    def get(name, cfg, weights, tokens):
        key = (name, tuple(tokens))
        if key not in cache:
            cache[key] = plain_model.forward_logits(weights, cfg, list(tokens))
        return cache[key]

    return get
