"""Typed configuration and the architecture registry."""
import copy
import json

import pytest

from conftest import TINY
from spyinfer_b200.config import (ConfigError, EngineConfig, Qwen3Config, config_from_json, known_architectures, load_model_config)


def test_registry_maps_name_to_config():
    assert "Qwen3ForCausalLM" in known_architectures()
    cfg = config_from_json(TINY["b"]["config"])
    assert isinstance(cfg, Qwen3Config)
    assert (cfg.hidden_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim) == (96, 8, 2, 32)
    assert cfg.rms_norm_eps == 1e-5 and cfg.rope_theta == 1e6 and cfg.tie_word_embeddings is False


def test_unknown_architecture_lists_known_ones():
    data = dict(TINY["a"]["config"], architectures=["LlamaForCausalLM"])
    with pytest.raises(ConfigError) as e:
        config_from_json(data)
    assert "LlamaForCausalLM" in str(e.value) and "Qwen3ForCausalLM" in str(e.value)
    # without an architectures list the model_type names the model; an unknown one is an error that lists both
    by_type = config_from_json({k: v for k, v in TINY["a"]["config"].items() if k != "architectures"})
    assert by_type.architecture == "Qwen3ForCausalLM"
    with pytest.raises(ConfigError) as e:
        config_from_json({k: v for k, v in dict(data, model_type="llama").items() if k != "architectures"})
    assert "llama" in str(e.value) and "qwen3" in str(e.value)


def test_keys_as_newer_checkpoints_write_them():
    """``rope_theta`` inside ``rope_parameters``, a default-typed ``rope_scaling``, ``eos_token_id`` as a
    list, no ``model_type``/``hidden_act`` (the reference demands both and uses neither), and keys
    that change nothing (``torch_dtype``, ``use_cache``, ``attention_dropout``) are accepted."""
    data = {k: v for k, v in TINY["b"]["config"].items() if k not in ("rope_theta", "model_type", "hidden_act")}
    data.update(rope_parameters={"rope_theta": 12345.0, "rope_type": "default"}, rope_scaling={"rope_type": "default"},
                eos_token_id=[7, 9], torch_dtype="bfloat16", use_cache=True, attention_dropout=0.0, attention_bias=False,
                sliding_window=None, max_window_layers=28)
    cfg = config_from_json(data)
    assert cfg.rope_theta == 12345.0 and cfg.eos_token_id == 7 and cfg.hidden_act == "silu" and cfg.model_type == "qwen3"
    assert config_from_json(cfg.to_json()).to_spec().layers[0].mixer.params["position"].params["theta"] == 12345.0
    with pytest.raises(ConfigError):
        config_from_json(dict(data, rope_parameters={"rope_theta": 1e6, "rope_type": "yarn", "factor": 4.0}))


def test_defaults_follow_the_reference():
    data = {k: v for k, v in TINY["a"]["config"].items() if k not in ("head_dim", "rope_theta", "rms_norm_eps", "tie_word_embeddings",
                                                                     "max_position_embeddings")}
    cfg = config_from_json(data)
    assert cfg.head_dim == 64 // 4 and cfg.rope_theta == 1e6 and cfg.rms_norm_eps == 1e-6
    assert cfg.tie_word_embeddings is False and cfg.max_position_embeddings == 16384


@pytest.mark.parametrize("key", ["hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "num_key_value_heads", "vocab_size"])
def test_missing_keys_are_named(key):
    data = {k: v for k, v in TINY["a"]["config"].items() if k != key}
    with pytest.raises(ConfigError) as e:
        config_from_json(data)
    assert key in str(e.value)


@pytest.mark.parametrize("patch", [{"num_key_value_heads": 3}, {"hidden_act": "gelu"}, {"rope_scaling": {"type": "yarn"}},
                                   {"attention_bias": "yes"}, {"head_dim": 15}, {"vocab_size": -1},
                                   {"use_sliding_window": True, "sliding_window": None},
                                   {"use_sliding_window": True, "sliding_window": 8},
                                   {"use_sliding_window": True, "sliding_window": 8, "max_window_layers": 3},
                                   {"use_sliding_window": True, "sliding_window": 8, "max_window_layers": "1"},
                                   {"use_sliding_window": True, "sliding_window": 8, "layer_types": ["full_attention"]}])
def test_values_the_engine_cannot_run_are_refused(patch):
    with pytest.raises(ConfigError):
        config_from_json(dict(TINY["a"]["config"], **patch))


def test_spec_is_data_layer_by_layer():
    spec = config_from_json(TINY["c"]["config"]).to_spec()
    assert len(spec.layers) == 4 and [e.layer for e in spec.run_order] == [0, 1, 2, 3]
    windows = [l.mixer.params["window"] for l in spec.layers]
    assert windows == [40, None, 40, None]
    m = spec.layers[0].mixer.params
    assert (m["num_heads"], m["num_kv_heads"], m["head_dim"], m["qk_norm_eps"]) == (6, 3, 48, 3e-6)
    assert m["position"].kind == "rotary_half" and m["position"].params == {"theta": 50000.0, "rotary_dim": 48}
    assert spec.layers[1].feed_forward.params["intermediate_size"] == 200
    assert spec.head.params["tied"] is False and spec.vocab_size == 517
    # a window key without use_sliding_window changes nothing
    plain = dict(TINY["c"]["config"], use_sliding_window=False)
    assert [l.mixer.params["window"] for l in config_from_json(plain).to_spec().layers] == [None] * 4


def test_which_layers_have_the_window_in_both_spellings():
    """``layer_types`` names the layers one by one; without it ``max_window_layers`` says how many
    layers at the bottom see every key.  The plain implementation states the same rule on its own."""
    import plain_model
    base = {k: v for k, v in TINY["c"]["config"].items() if k != "layer_types"}
    for first, want in [(0, [40, 40, 40, 40]), (2, [None, None, 40, 40]), (4, [None] * 4)]:
        data = dict(base, max_window_layers=first)
        cfg = config_from_json(data)
        assert [cfg.layer_window(i) for i in range(4)] == want == plain_model.layer_windows(data)
        assert [l.mixer.params["window"] for l in config_from_json(cfg.to_json()).to_spec().layers] == want
    both = dict(TINY["c"]["config"], max_window_layers=1)              # the list counts where both are given
    assert [config_from_json(both).layer_window(i) for i in range(4)] == [40, None, 40, None] == plain_model.layer_windows(both)
    off = dict(base, use_sliding_window=False, max_window_layers=2)
    assert [config_from_json(off).layer_window(i) for i in range(4)] == [None] * 4 == plain_model.layer_windows(off)


def test_keys_that_are_not_read_are_named_in_a_warning():
    import warnings
    with pytest.warns(UserWarning, match="logit_cap.*mystery"):
        cfg = config_from_json(dict(TINY["a"]["config"], mystery=1, logit_cap=30.0))
    assert cfg.extra == {"logit_cap": 30.0, "mystery": 1}
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        for name in TINY:
            config_from_json(TINY[name]["config"])
        config_from_json(dict(TINY["a"]["config"], torch_dtype="bfloat16", use_cache=True, attention_dropout=0.0, transformers_version="x",
                              sliding_window=None, max_window_layers=28, use_sliding_window=False))


def test_attention_bias_gives_the_q_k_v_projections_bias_tensors():
    from spyinfer_b200.engine.model import declared_weights
    spec = config_from_json(TINY["e"]["config"]).to_spec()
    names = {d.name: d.shape for d in declared_weights(spec)}
    assert names["model.layers.1.self_attn.q_proj.bias"] == (5 * 16,) and names["model.layers.0.self_attn.v_proj.bias"] == (1 * 16,)
    assert "model.layers.0.self_attn.o_proj.bias" not in names
    assert not any(n.endswith(".bias") for n in {d.name for d in declared_weights(config_from_json(TINY["a"]["config"]).to_spec())})


def test_config_round_trips_through_json(tmp_path):
    cfg = config_from_json(TINY["c"]["config"])
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg.to_json(), f)
    again = load_model_config(str(tmp_path))
    assert again.to_json() == cfg.to_json()
    with pytest.raises(ConfigError):
        load_model_config(str(tmp_path / "nowhere"))


def test_run_order_is_checked():
    from spyinfer_b200.config import RunEntry
    spec = config_from_json(TINY["a"]["config"]).to_spec()
    spec.run_order = [RunEntry(0), RunEntry(1), RunEntry(1, cache_of=1), RunEntry(0)]
    spec.validate()
    bad = copy.copy(spec)
    bad.run_order = [RunEntry(0, cache_of=0)]
    with pytest.raises(ValueError):
        bad.validate()
    bad.run_order = [RunEntry(5)]
    with pytest.raises(ValueError):
        bad.validate()


def test_engine_config_names_and_checks():
    c = EngineConfig(max_num_batched_tokens=64, max_num_seqs=4, max_model_len=100, kvcache_block_size=8, num_kvcache_blocks=10, dtype="fp32")
    assert c.dtype == "float32"
    c.clamp_to_model(50)
    assert c.max_model_len == 50
    for bad in (dict(dtype="float16"), dict(kvcache_block_size=0), dict(num_kvcache_blocks=0), dict(gpu_memory_utilization=0.0)):
        with pytest.raises(ValueError):
            EngineConfig(**bad)
