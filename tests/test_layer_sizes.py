"""The engine at the layer sizes of Qwen3-8B, 14B and 32B (one layer each, a small vocabulary
that is no power of two, seeded random weights) against the plain implementation, in 32-bit
and in bfloat16, under every way of cutting the work: whole, most of it in one step and the
last 32 tokens one by one, portions of changing size, and mixed with page reuse.  These are
the shapes the fast kernels were built for: group sizes 4, 5 and 8, widths 4096 and 5120,
feed-forward widths 12288, 17408 and 25600."""
import json
import random

import numpy as np
import pytest

import plain_model
from trace_tools import TraceBuilder, mixed_trace, peak_pages, peak_tokens, run_trace

pytestmark = pytest.mark.gpu

SHAPES = {
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128, intermediate_size=12288),
    "14b": dict(hidden_size=5120, num_attention_heads=40, num_key_value_heads=8, head_dim=128, intermediate_size=17408),
    "32b": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, head_dim=128, intermediate_size=25600),
}
LENGTHS = [3, 40, 131, 300]   # 131 and 300 tokens: one row of 256-token tiles, and two
PORTIONS = (7, 2, 19, 3, 2, 33)
# the same bounds as the tiny models' replay tests
TOL = {"float32": dict(max_rel=3e-5, rms_rel=1e-5), "bfloat16": dict(max_rel=5e-2, rms_rel=2e-2)}


def config_of(name):
    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": 1, "vocab_size": 389,
           "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 4096,
           "bos_token_id": 0, "eos_token_id": 1}
    cfg.update(SHAPES[name])
    return cfg


@pytest.fixture(scope="module")
def layer_models(tmp_path_factory):
    from safetensors.torch import save_file

    memo = {}

    def get(name):
        if name not in memo:
            cfg = config_of(name)
            d = tmp_path_factory.mktemp(f"layer_{name}")
            with open(d / "config.json", "w") as f:
                json.dump(cfg, f)
            w = plain_model.random_weights(cfg, 100 + len(name), 0.02, 0.05)
            save_file({k: v.contiguous() for k, v in w.items()}, str(d / "model.safetensors"))
            rng = random.Random(len(name))
            reqs = {f"r{n}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in LENGTHS}
            want = {rid: plain_model.forward_logits(w, cfg, toks).numpy() for rid, toks in reqs.items()}
            memo[name] = (str(d), cfg, reqs, want)
        return memo[name]

    return get


def build(reqs):
    b = TraceBuilder()
    tokens_of = {}
    for rid, toks in reqs.items():
        b.whole("w_" + rid, toks)
        b.tail_one_by_one("t_" + rid, toks, tail=32)
        b.portions("p_" + rid, toks, PORTIONS)
        for prefix in "wtp":
            tokens_of[prefix + "_" + rid] = toks
    mixed = {"m_" + rid: toks for rid, toks in reqs.items()}
    mixed_trace(b, mixed, {rid: max(1, len(toks) - 12) for rid, toks in mixed.items()}, random.Random(5), max_live=3)
    tokens_of.update(mixed)
    return b, tokens_of


# (shape, page size): every shape in the program's own pages of 16, and the 8B shape in pages of 4,
# which are no TMA box: the bfloat16 run then takes the mma.sync attention kernel (split mode for
# decoding steps, tiles mode for portions) at head size 128, with the pool at the trace's exact peak
CASES = [(name, None) for name in SHAPES] + [("8b", 4)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", CASES, ids=[f"{n}-page{p or 16}" for n, p in CASES])
def test_layer_sizes_match_plain_under_every_cut(name, page_size, dtype, layer_models, tmp_path):
    folder, cfg, reqs, want = layer_models(name)
    b, tokens_of = build(reqs)
    options = [] if page_size is None else ["--page-size", page_size, "--num-pages", peak_pages(b, page_size)]
    rows = run_trace(folder, dtype, b, str(tmp_path), peak_tokens(b), cfg["vocab_size"], options=options)
    tol = TOL[dtype]
    for rid, toks in tokens_of.items():
        ref = want[rid[2:]]
        got = np.stack([rows[(rid, p)] for p in range(len(toks))])
        assert np.isfinite(got).all(), f"{name} {rid}: logits are not finite"
        err = np.abs(got - ref)
        scale, rms = np.abs(ref).max(), np.sqrt((ref ** 2).mean())
        bad = np.argwhere(err > tol["max_rel"] * scale)
        if len(bad):
            first = int(bad[:, 0].min())
            raise AssertionError(f"{name} {rid} ({len(toks)} tokens): first wrong position {first}, error {err[first].max():.3g} against a "
                                 f"largest logit of {scale:.3g} (allowed {tol['max_rel'] * scale:.3g})")
        assert np.sqrt((err ** 2).mean()) <= tol["rms_rel"] * rms, f"{name} {rid}: rms error {np.sqrt((err ** 2).mean()):.3g} vs rms logit {rms:.3g}"


def test_eight_layers_at_8b_sizes_in_bfloat16_stay_within_the_bound(tmp_path, capsys):
    """Depth: eight layers at the 8B layer sizes (the other tests run one to four), bfloat16, a
    prompt of 64 tokens in one step and eight more tokens one by one, every row against the plain
    implementation in 32-bit.  The error that eight layers of bfloat16 roundings build up is
    printed and held to the bound of the one-layer tests."""
    from safetensors.torch import save_file

    cfg = dict(config_of("8b"), num_hidden_layers=8)
    w = plain_model.random_weights(cfg, 808, 0.02, 0.05)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
    rng = random.Random(8)
    toks = [rng.randrange(cfg["vocab_size"]) for _ in range(72)]
    b = TraceBuilder()
    b.tail_one_by_one("x", toks, tail=8)
    rows = run_trace(str(tmp_path), "bfloat16", b, str(tmp_path / "out"), peak_tokens(b), cfg["vocab_size"])
    want = plain_model.forward_logits(w, cfg, toks).numpy()
    got = np.stack([rows[("x", p)] for p in range(len(toks))])
    assert np.isfinite(got).all()
    err = np.abs(got - want)
    scale, rms = np.abs(want).max(), np.sqrt((want ** 2).mean())
    worst, err_rms = err.max() / scale, np.sqrt((err ** 2).mean()) / rms
    with capsys.disabled():
        print(f"\n  eight 8B-sized layers in bfloat16: largest error {worst:.4f} of the largest logit, rms error {err_rms:.4f} of the rms logit "
              f"(decoded rows alone: {err[64:].max() / scale:.4f})")
    assert worst <= TOL["bfloat16"]["max_rel"] and err_rms <= TOL["bfloat16"]["rms_rel"]


@pytest.mark.parametrize("name,requests", [("8b", 200), ("14b", 100)])
def test_many_requests_decode_together(name, requests, layer_models):
    """A hundred and two hundred requests decoding at once in bfloat16 (the products then run on one token tile of 128, or on
    pairs of blocks with K ranges whose partial sums the next norm and the q/k kernel add up; the decode graph is the padded
    one of 128 or 256 rows): three new tokens each, every one held against the plain implementation given the same history."""
    from spyinfer_b200 import LLMEngine, SamplingParams
    folder, cfg, _, _ = layer_models(name)
    weights = plain_model.random_weights(cfg, 100 + len(name), 0.02, 0.05)
    rng = random.Random(requests)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(rng.randrange(2, 7))] for _ in range(requests)]
    engine = LLMEngine(folder, dtype="bfloat16", max_num_seqs=256, max_model_len=64, num_kvcache_blocks=512, max_num_batched_tokens=2048)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=3, ignore_eos=True))
    assert engine.runner.graph_steps >= 1
    for i, (p, o) in enumerate(zip(prompts, outs)):
        assert len(o) == 3
        if i % 5:
            continue                      # the plain implementation on every fifth request
        seq = list(p)
        for k, tok in enumerate(o):
            logits = plain_model.forward_logits(weights, cfg, seq)[-1]
            assert logits[tok].item() >= logits.max().item() - 0.05 * logits.abs().max().item(), f"request {i}, token {k}: engine chose {tok}, plain argmax {int(logits.argmax())}"
            seq.append(tok)
