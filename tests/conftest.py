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
# put the bfloat16 path on its tensor-core attention kernel, a window, and a tied head.  E has
# biases on the q, k and v projections (made large, so that leaving them out shows).
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
    "e": dict(
        config={"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": 2,
                "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 104,
                "vocab_size": 300, "rope_theta": 20000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
                "max_position_embeddings": 1024, "bos_token_id": 1, "eos_token_id": 2, "attention_bias": True},
        seed=55, std=0.05, norm_std=0.1),
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


class GuardedAllocations:
    """Guard words around device buffers, in place of a memory checker (which this pool does not
    offer): while active, every CUDA tensor that ``torch.empty``, ``torch.full`` or ``torch.zeros``
    makes (in the test or inside the package) lies between two 256-byte zones filled with a
    pattern; ``check`` finds any zone that a kernel wrote into.  A write past the end of an
    output, before its start, or into a neighbouring buffer of the same test shows here even when
    the values that were checked are right."""

    ZONE = 256  # bytes on each side
    PATTERN = 0xA5

    def __init__(self, monkeypatch):
        self.held = []
        self._empty, self._full, self._zeros = torch.empty, torch.full, torch.zeros
        monkeypatch.setattr(torch, "empty", self.empty)
        monkeypatch.setattr(torch, "full", self.full)
        monkeypatch.setattr(torch, "zeros", self.zeros)

    def _plain(self, kwargs) -> bool:
        dev = kwargs.get("device")
        on_cuda = dev is not None and torch.device(dev).type == "cuda"
        return not on_cuda or kwargs.get("pin_memory") or kwargs.get("out") is not None or kwargs.get("layout") not in (None, torch.strided) \
            or torch.cuda.is_current_stream_capturing()

    def _guarded(self, size, kwargs):
        if len(size) == 1 and isinstance(size[0], (tuple, list, torch.Size)):
            size = tuple(size[0])
        dtype = kwargs.get("dtype") or torch.get_default_dtype()
        item = self._empty((), dtype=dtype).element_size()
        numel = 1
        for d in size:
            numel *= int(d)
        body = (numel * item + 255) // 256 * 256
        raw = self._empty(body + 2 * self.ZONE, dtype=torch.uint8, device=kwargs["device"])
        raw[:self.ZONE] = self.PATTERN
        raw[self.ZONE + numel * item:] = self.PATTERN
        self.held.append((raw, numel * item))
        return raw[self.ZONE:self.ZONE + numel * item].view(dtype).view(tuple(int(d) for d in size))

    def empty(self, *size, **kwargs):
        return self._empty(*size, **kwargs) if self._plain(kwargs) else self._guarded(size, kwargs)

    def full(self, size, fill_value, **kwargs):
        if self._plain(kwargs):
            return self._full(size, fill_value, **kwargs)
        if kwargs.get("dtype") is None:
            kwargs["dtype"] = torch.get_default_dtype() if isinstance(fill_value, float) else (torch.bool if isinstance(fill_value, bool) else torch.int64)
        return self._guarded((size,), kwargs).fill_(fill_value)

    def zeros(self, *size, **kwargs):
        return self._zeros(*size, **kwargs) if self._plain(kwargs) else self._guarded(size, kwargs).zero_()

    def check(self):
        torch.cuda.synchronize()
        for raw, nbytes in self.held:
            front, back = raw[:self.ZONE], raw[self.ZONE + nbytes:]
            assert bool((front == self.PATTERN).all()), f"a kernel wrote before the start of a {nbytes}-byte device buffer"
            assert bool((back == self.PATTERN).all()), f"a kernel wrote past the end of a {nbytes}-byte device buffer"
        return len(self.held)


@pytest.fixture
def guarded_allocations(monkeypatch):
    """See ``GuardedAllocations``; the zones are checked when the test ends."""
    g = GuardedAllocations(monkeypatch)
    yield g
    monkeypatch.undo()
    if torch.cuda.is_available():
        g.check()
