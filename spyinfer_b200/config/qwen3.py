"""Typed configuration of the Qwen3 dense decoder (``Qwen3ForCausalLM``).

Keys, defaults and meanings follow spymaster2h/spyinfer src/models/model_config.hpp:27-47:
``head_dim`` defaults to ``hidden_size / num_attention_heads``, ``rope_theta`` to 1e6,
``rms_norm_eps`` to 1e-6, ``max_position_embeddings`` to 16384, ``tie_word_embeddings`` to
false.  Unlike the reference, which lets -1 defaults flow through, every size is required and
checked.  ``model_type`` and ``hidden_act``, which the reference demands and then never uses
(:32-33; its activation is SiLU in code), default to ``"qwen3"`` and ``"silu"`` here; another
activation is refused.  ``rope_theta`` may also stand inside ``rope_parameters`` (newer
checkpoints write it there), and ``eos_token_id`` may be a list, whose first entry counts.

Read beyond the reference's keys: ``use_sliding_window``, ``sliding_window``, and which
layers have the window: ``layer_types`` (a layer of type ``"sliding_attention"`` sees the
last ``sliding_window`` keys, its own included; ``"full_attention"`` sees all) or, where that
list is absent, ``max_window_layers`` (layers ``0 .. max_window_layers - 1`` see every key,
the layers from ``max_window_layers`` on have the window).  ``use_sliding_window`` with
neither is refused: it would not say which layers are meant.  Where both are given the list
counts.  The reference reads none of these keys (every layer of its model sees all keys),
so their meaning here is this engine's statement, pinned by its own tests only.  ``attention_bias`` true gives the q, k and v projections bias
tensors (``self_attn.{q,k,v}_proj.bias``: the three the reference's model has slots for and
never binds, src/models/qwen3.hpp:39, 143-157; a checkpoint with further bias tensors is
refused by name at load).  Keys that would change the result and are not implemented are
refused: ``rope_scaling`` of any kind but the default.  A key that is not read at all and is not known to be without effect on
the logits (``_NO_EFFECT``) is named in a warning, never dropped silently.

The layer structure itself (pre-norm blocks of grouped-query attention with per-head q/k
RMSNorm and rotate-half RoPE, SwiGLU feed-forward, tied or untied head) restates
src/models/qwen3.hpp:19-54 (tensor names) and :122-308 (order of operations).
"""
from __future__ import annotations

import warnings
from dataclasses import asdict, dataclass, field
from typing import Any, Dict, List, Optional

from .model_config import ArchitectureConfig, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, RunEntry

# keys that checkpoints carry and that do not change what a forward pass computes
_NO_EFFECT = {"architectures", "torch_dtype", "dtype", "transformers_version", "use_cache", "attention_dropout", "initializer_range",
              "pad_token_id", "rope_scaling", "rope_parameters", "_name_or_path"}

_REQUIRED_INTS = ("hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "vocab_size")


@register_architecture("Qwen3ForCausalLM", model_type="qwen3")
@dataclass
class Qwen3Config(ArchitectureConfig):
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    vocab_size: int
    head_dim: int
    model_type: str = "qwen3"
    hidden_act: str = "silu"
    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 16384
    bos_token_id: int = -1
    eos_token_id: int = -1
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    layer_types: Optional[List[str]] = None
    max_window_layers: Optional[int] = None
    attention_bias: bool = False
    extra: Dict[str, Any] = field(default_factory=dict)

    @classmethod
    def from_json(cls, data: Dict[str, Any]) -> "Qwen3Config":
        problems = []
        data = dict(data)
        data.setdefault("model_type", "qwen3")
        data.setdefault("hidden_act", "silu")
        for key in ("model_type", "hidden_act"):
            if not isinstance(data[key], str):
                problems.append(f"{key!r} must be a string, found {data[key]!r}")
        for key in _REQUIRED_INTS:
            v = data.get(key)
            if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
                problems.append(f"{key!r} must be a positive integer, found {v!r}")
        if problems:
            raise ConfigError("Qwen3 config.json: " + "; ".join(problems))
        if data["hidden_act"] != "silu":
            raise ConfigError(f"Qwen3 config.json: hidden_act {data['hidden_act']!r} is not implemented (only \"silu\")")
        rope_parameters = data.get("rope_parameters") if isinstance(data.get("rope_parameters"), dict) else {}
        for key in ("rope_scaling", "rope_parameters"):
            scaling = data.get(key)
            if scaling in (None, {}):
                continue
            kind = scaling.get("rope_type", scaling.get("type", "default")) if isinstance(scaling, dict) else scaling
            if kind != "default":
                raise ConfigError(f"Qwen3 config.json: {key} of type {kind!r} is not implemented (only plain rotary positions); "
                                  "remove it or set it to null")
        if "rope_theta" not in data and "rope_theta" in rope_parameters:
            data["rope_theta"] = rope_parameters["rope_theta"]
        for key in ("bos_token_id", "eos_token_id"):
            if isinstance(data.get(key), list):
                data[key] = data[key][0] if data[key] else None
        if not isinstance(data.get("attention_bias", False), bool):
            raise ConfigError(f"Qwen3 config.json: attention_bias must be true or false, found {data['attention_bias']!r}")
        nh, nkv = data["num_attention_heads"], data["num_key_value_heads"]
        if nh % nkv != 0:
            raise ConfigError(f"Qwen3 config.json: num_attention_heads {nh} is not a multiple of num_key_value_heads {nkv}")
        head_dim = data.get("head_dim")
        if head_dim is None:
            if data["hidden_size"] % nh != 0:
                raise ConfigError("Qwen3 config.json: no head_dim, and hidden_size is not a multiple of num_attention_heads")
            head_dim = data["hidden_size"] // nh
        if not isinstance(head_dim, int) or head_dim <= 0 or head_dim % 2 != 0:
            raise ConfigError(f"Qwen3 config.json: head_dim must be a positive even integer, found {head_dim!r}")
        eps = float(data.get("rms_norm_eps", 1e-6))
        theta = float(data.get("rope_theta", 1000000.0))
        if not eps > 0.0 or not theta > 0.0:
            raise ConfigError("Qwen3 config.json: rms_norm_eps and rope_theta must be positive")
        use_window = bool(data.get("use_sliding_window", False))
        window = data.get("sliding_window")
        layer_types = data.get("layer_types")
        first_windowed = data.get("max_window_layers")
        if use_window:
            if not isinstance(window, int) or isinstance(window, bool) or window <= 0:
                raise ConfigError(f"Qwen3 config.json: use_sliding_window needs a positive sliding_window, found {window!r}")
            if layer_types is not None:
                if not isinstance(layer_types, list) or len(layer_types) != data["num_hidden_layers"]:
                    raise ConfigError("Qwen3 config.json: layer_types must name every layer")
                bad = sorted(set(layer_types) - {"full_attention", "sliding_attention"})
                if bad:
                    raise ConfigError(f"Qwen3 config.json: unknown layer_types {bad}")
            elif first_windowed is None:
                raise ConfigError("Qwen3 config.json: use_sliding_window without layer_types or max_window_layers does not say which "
                                  "layers have the window")
            elif not isinstance(first_windowed, int) or isinstance(first_windowed, bool) or not 0 <= first_windowed <= data["num_hidden_layers"]:
                raise ConfigError(f"Qwen3 config.json: max_window_layers must lie in 0..num_hidden_layers, found {first_windowed!r}")
        known = {f for f in cls.__dataclass_fields__ if f != "extra"}
        unread = sorted(k for k in data if k not in known and k not in _NO_EFFECT)
        if unread:
            warnings.warn(f"Qwen3 config.json: keys that this engine does not read: {unread}", stacklevel=2)
        return cls(
            hidden_size=data["hidden_size"], intermediate_size=data["intermediate_size"],
            num_hidden_layers=data["num_hidden_layers"], num_attention_heads=nh, num_key_value_heads=nkv,
            vocab_size=data["vocab_size"], head_dim=head_dim, model_type=data["model_type"], hidden_act=data["hidden_act"],
            rope_theta=theta, rms_norm_eps=eps, tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            max_position_embeddings=int(data.get("max_position_embeddings", 16384)),
            bos_token_id=int(data.get("bos_token_id", -1) if data.get("bos_token_id") is not None else -1),
            eos_token_id=int(data.get("eos_token_id", -1) if data.get("eos_token_id") is not None else -1),
            use_sliding_window=use_window, sliding_window=window if use_window else None,
            layer_types=list(layer_types) if (use_window and layer_types is not None) else None,
            max_window_layers=first_windowed if (use_window and layer_types is None) else None,
            attention_bias=bool(data.get("attention_bias", False)),
            extra={k: v for k, v in data.items() if k not in known and k not in ("architectures", "rope_parameters")},
        )

    def to_json(self) -> Dict[str, Any]:
        d = asdict(self)
        extra = d.pop("extra")
        d = {k: v for k, v in d.items() if v is not None}
        d["architectures"] = [self.architecture]
        for k, v in extra.items():
            d.setdefault(k, v)
        return d

    def layer_window(self, layer: int) -> Optional[int]:
        if not self.use_sliding_window:
            return None
        if self.layer_types is not None:
            return self.sliding_window if self.layer_types[layer] == "sliding_attention" else None
        return self.sliding_window if layer >= self.max_window_layers else None

    def to_spec(self) -> ModelSpec:
        H = self.hidden_size
        position = PartSpec("rotary_half", {"theta": self.rope_theta, "rotary_dim": self.head_dim})
        layers = []
        for i in range(self.num_hidden_layers):
            layers.append(LayerSpec(
                block="pre_norm",
                mixer_norm=PartSpec("rms_norm", {"size": H, "eps": self.rms_norm_eps, "weight": "input_layernorm.weight"}),
                mixer=PartSpec("attention", {
                    "hidden_size": H, "num_heads": self.num_attention_heads, "num_kv_heads": self.num_key_value_heads,
                    "head_dim": self.head_dim, "qk_norm_eps": self.rms_norm_eps, "position": position,
                    "window": self.layer_window(i), "scale": None, "prefix": "self_attn.", "qkv_bias": self.attention_bias,
                }),
                ffn_norm=PartSpec("rms_norm", {"size": H, "eps": self.rms_norm_eps, "weight": "post_attention_layernorm.weight"}),
                feed_forward=PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": self.intermediate_size,
                                                    "activation": "silu", "prefix": "mlp."}),
                weight_prefix=f"model.layers.{i}.",
            ))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=H, vocab_size=self.vocab_size,
            embedding=PartSpec("token_embedding", {"vocab_size": self.vocab_size, "hidden_size": H,
                                                   "weight": "model.embed_tokens.weight"}),
            layers=layers, run_order=[RunEntry(i) for i in range(self.num_hidden_layers)],
            final_norm=PartSpec("rms_norm", {"size": H, "eps": self.rms_norm_eps, "weight": "model.norm.weight"}),
            head=PartSpec("lm_head", {"vocab_size": self.vocab_size, "hidden_size": H, "tied": self.tie_word_embeddings,
                                      "weight": "lm_head.weight", "tied_to": "model.embed_tokens.weight"}),
            max_position=self.max_position_embeddings, eos_token_id=self.eos_token_id, bos_token_id=self.bos_token_id,
        )
        spec.validate()
        return spec
