"""The safetensors container, binding by name with one clear error, and random models."""
import json
import os
import struct

import pytest
import torch
from safetensors.torch import load_file, save_file

from conftest import TINY
from spyinfer_b200.config import config_from_json
from spyinfer_b200.engine.model import declared_weights
from spyinfer_b200.weights import (SafetensorsError, SafetensorsFile, WeightDecl, WeightError, load_checkpoint, random_tensors,
                                   write_model_folder, write_safetensors)


def test_reader_agrees_with_the_safetensors_library(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).reshape(2, 3),
         "d": torch.randn(2, 2).to(torch.float16)}
    save_file(t, str(tmp_path / "model.safetensors"))
    f = SafetensorsFile(str(tmp_path / "model.safetensors"))
    assert sorted(f.names()) == sorted(t)
    for k in t:
        assert torch.equal(f.tensor(k), t[k]) and f.shape(k) == tuple(t[k].shape)


def test_writer_is_read_by_the_safetensors_library(tmp_path):
    t = [("x", torch.randn(4, 3).to(torch.bfloat16)), ("y", torch.randn(5))]
    write_safetensors(str(tmp_path / "m.safetensors"), [(n, v.dtype, tuple(v.shape)) for n, v in t], iter(t))
    back = load_file(str(tmp_path / "m.safetensors"))
    assert all(torch.equal(back[n], v) for n, v in t)


def test_storage_types(tmp_path):
    t = {"w": torch.randn(2, 2).to(torch.bfloat16), "f": torch.randn(2, 2), "h": torch.randn(2, 2).to(torch.float16),
         "i": torch.arange(4, dtype=torch.int64)}
    save_file(t, str(tmp_path / "model.safetensors"))
    decls = [WeightDecl("w", (2, 2)), WeightDecl("f", (2, 2)), WeightDecl("h", (2, 2)), WeightDecl("i", (4,), integer=True)]
    got = load_checkpoint(str(tmp_path), decls, "cpu")
    assert got["w"].dtype == torch.bfloat16            # bfloat16 is kept
    assert got["f"].dtype == torch.float32             # a tensor stored in 32-bit stays so
    assert got["h"].dtype == torch.float32 and torch.equal(got["h"], t["h"].float())
    assert got["i"].dtype == torch.int32               # integer tables as int32


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path, tiny_models):
    folder, cfg, w = tiny_models["b"]
    decls = declared_weights(config_from_json(cfg).to_spec())
    broken = {k: v for k, v in w.items()}
    del broken["model.layers.1.mlp.up_proj.weight"]
    del broken["model.norm.weight"]
    broken["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(8, 96, dtype=torch.bfloat16)
    broken["model.layers.7.extra.weight"] = torch.zeros(3, dtype=torch.bfloat16)
    save_file({k: v.contiguous() for k, v in broken.items()}, str(tmp_path / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_checkpoint(str(tmp_path), decls, "cpu")
    err = e.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert len(err.wrong) == 1 and "q_proj" in err.wrong[0] and "[256, 96]" in err.wrong[0] and "[8, 96]" in err.wrong[0]
    msg = str(err)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shape or dtype (1)", "up_proj", "extra.weight"):
        assert needle in msg


def test_untied_model_needs_its_head_and_tied_model_ignores_one(tmp_path, tiny_models):
    _, cfg_b, w_b = tiny_models["b"]
    no_head = {k: v.contiguous() for k, v in w_b.items() if k != "lm_head.weight"}
    os.makedirs(tmp_path / "b")
    save_file(no_head, str(tmp_path / "b" / "model.safetensors"))
    with pytest.raises(WeightError) as e:
        load_checkpoint(str(tmp_path / "b"), declared_weights(config_from_json(cfg_b).to_spec()), "cpu")
    assert e.value.missing == ["lm_head.weight"]
    _, cfg_a, w_a = tiny_models["a"]
    with_head = {k: v.contiguous() for k, v in w_a.items()}
    with_head["lm_head.weight"] = w_a["model.embed_tokens.weight"].clone()
    os.makedirs(tmp_path / "a")
    save_file(with_head, str(tmp_path / "a" / "model.safetensors"))
    decls = declared_weights(config_from_json(cfg_a).to_spec())
    assert "lm_head.weight" not in {d.name for d in decls}
    load_checkpoint(str(tmp_path / "a"), decls, "cpu", ignorable=["lm_head.weight"])
    with pytest.raises(WeightError):
        load_checkpoint(str(tmp_path / "a"), decls, "cpu")


def test_truncated_and_malformed_files(tmp_path):
    p = tmp_path / "model.safetensors"
    save_file({"a": torch.randn(64, 64)}, str(p))
    raw = p.read_bytes()
    p.write_bytes(raw[:-100])
    with pytest.raises(WeightError) as e:
        load_checkpoint(str(tmp_path), [WeightDecl("a", (64, 64))], "cpu")
    assert "truncated" in str(e.value)
    p.write_bytes(struct.pack("<Q", 10 ** 9) + b"{}")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    p.write_bytes(struct.pack("<Q", 4) + b"nope")
    with pytest.raises(SafetensorsError):
        SafetensorsFile(str(p))
    os.remove(p)
    with pytest.raises(WeightError):
        load_checkpoint(str(tmp_path), [WeightDecl("a", (1,))], "cpu")


def test_sharded_folder(tmp_path):
    save_file({"a": torch.ones(2)}, str(tmp_path / "s1.safetensors"))
    save_file({"b": torch.zeros(3)}, str(tmp_path / "s2.safetensors"))
    with open(tmp_path / "model.safetensors.index.json", "w") as f:
        json.dump({"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}, f)
    got = load_checkpoint(str(tmp_path), [WeightDecl("a", (2,)), WeightDecl("b", (3,))], "cpu")
    assert got["a"].sum() == 2 and got["b"].shape == (3,)


def test_random_model_folder_is_seeded_and_loads(tmp_path):
    cfg = config_from_json(TINY["b"]["config"])
    write_model_folder(str(tmp_path / "m1"), cfg, seed=5, std=0.03, norm_std=0.1)
    write_model_folder(str(tmp_path / "m2"), cfg, seed=5, std=0.03, norm_std=0.1)
    write_model_folder(str(tmp_path / "m3"), cfg, seed=6, std=0.03, norm_std=0.1)
    a, b, c = (load_file(str(tmp_path / m / "model.safetensors")) for m in ("m1", "m2", "m3"))
    assert all(torch.equal(a[k], b[k]) for k in a) and any(not torch.equal(a[k], c[k]) for k in a)
    assert all(v.dtype == torch.bfloat16 for v in a.values())
    with open(tmp_path / "m1" / "config.json") as f:
        assert config_from_json(json.load(f)).to_json() == cfg.to_json()
    q = a["model.layers.0.self_attn.q_proj.weight"].float()
    n = a["model.layers.0.input_layernorm.weight"].float()
    assert abs(q.std().item() - 0.03) < 0.003 and abs(q.mean().item()) < 0.002
    assert abs(n.mean().item() - 1.0) < 0.05 and 0.05 < n.std().item() < 0.15
    decls = declared_weights(cfg.to_spec())
    assert set(a) == {d.name for d in decls}
    load_checkpoint(str(tmp_path / "m1"), decls, "cpu")
    # a tensor's values do not depend on the other tensors of the model
    alone = dict(random_tensors([d for d in decls if d.name == "model.norm.weight"], 5, 0.03, 0.1))
    assert torch.equal(alone["model.norm.weight"], a["model.norm.weight"])


def test_random_model_folder_in_shards_reads_back_as_the_single_file_does(tmp_path):
    """``write_model_folder`` with ``shard_bytes``: several files and an index, no tensor cut, and the
    loader finds in them exactly the tensors of the one-file folder of the same seed."""
    from spyinfer_b200.config import config_from_json
    from spyinfer_b200.engine.model import declared_weights
    from spyinfer_b200.weights import write_model_folder
    from conftest import TINY

    cfg = config_from_json(TINY["b"]["config"])
    write_model_folder(str(tmp_path / "one"), cfg, 3, 0.03, 0.1)
    write_model_folder(str(tmp_path / "many"), cfg, 3, 0.03, 0.1, shard_bytes=60000)
    files = sorted(p.name for p in (tmp_path / "many").iterdir())
    assert "model.safetensors.index.json" in files and len([f for f in files if f.endswith(".safetensors")]) > 3
    decls = declared_weights(cfg.to_spec())
    one = load_checkpoint(str(tmp_path / "one"), decls, "cpu")
    many = load_checkpoint(str(tmp_path / "many"), decls, "cpu")
    assert one.keys() == many.keys() and all(torch.equal(one[k], many[k]) for k in one)


def test_tensors_are_made_when_asked_for_and_not_kept(tmp_path):
    """``open_checkpoint``: a tensor is read when it is asked for; asked for again while the first is
    still in use it is the same object (a tied head and its table), and once nobody holds it a fresh one."""
    from spyinfer_b200.config import config_from_json
    from spyinfer_b200.engine.model import declared_weights
    from spyinfer_b200.weights import open_checkpoint, write_model_folder
    from conftest import TINY

    cfg = config_from_json(TINY["a"]["config"])
    write_model_folder(str(tmp_path), cfg, 1)
    lazy = open_checkpoint(str(tmp_path), declared_weights(cfg.to_spec()), "cpu")
    assert "model.embed_tokens.weight" in lazy and "nothing" not in lazy and len(lazy) == len(declared_weights(cfg.to_spec()))
    assert lazy.stored_dtypes["model.norm.weight"] == torch.bfloat16
    a = lazy["model.embed_tokens.weight"]
    assert lazy["model.embed_tokens.weight"] is a
    ident = id(a)
    keep = a.clone()
    del a
    b = lazy["model.embed_tokens.weight"]
    assert torch.equal(b, keep)
    with pytest.raises(KeyError):
        lazy["nothing"]
    lazy.close()


@pytest.mark.gpu
def test_loading_never_holds_the_checkpoint_beside_the_model(tmp_path):
    """Four layers at the 8B layer sizes (1.5 GB): the parts fuse q|k|v and gate|up into layouts of their
    own at load.  The most device memory in use during the load stays well below twice the model."""
    from spyinfer_b200 import LLMEngine
    from spyinfer_b200.config import config_from_json
    from spyinfer_b200.weights import write_model_folder
    cfg = config_from_json({"architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 4, "hidden_size": 4096, "num_attention_heads": 32,
                            "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 1000, "max_position_embeddings": 256})
    write_model_folder(str(tmp_path), cfg, 2, device="cuda:0")
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    before = torch.cuda.memory_allocated()
    engine = LLMEngine(str(tmp_path), dtype="bfloat16", max_num_seqs=2, max_model_len=64, num_kvcache_blocks=8, max_num_batched_tokens=64)
    held = torch.cuda.memory_allocated() - before
    peak = torch.cuda.max_memory_allocated() - before
    assert held > 1.5e9 and peak < 1.4 * held, f"held {held / 1e9:.2f} GB after the load, {peak / 1e9:.2f} GB at its peak"
    assert len(engine.generate([[1, 2, 3]])[0]) > 0
