"""The plain implementation against the reference's own compiled CPU path.

``tests/golden/make_golden.py`` ran spymaster2h/spyinfer's CPU model code on two tiny seeded
models and stored its logits; this test rebuilds the same weights from the seed and compares
``plain_model.forward_logits`` with them.  The reference computes in float32 with another
order of sums, so equality holds to rounding: a few 1e-7 on logits of magnitude about 1."""
import json
import os

import numpy as np
import pytest
import torch

import plain_model

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_matches_reference_cpu_path(name):
    with open(os.path.join(GOLDEN, name + ".json")) as f:
        meta = json.load(f)
    cfg = meta["config"]
    golden = np.fromfile(os.path.join(GOLDEN, name + ".logits.f32"), dtype="<f4").reshape(-1, cfg["vocab_size"])
    weights = plain_model.random_weights(cfg, meta["seed"], meta["std"], meta["norm_std"])
    ours = torch.cat([plain_model.forward_logits(weights, cfg, p) for p in meta["prompts"]]).numpy()
    assert ours.shape == golden.shape
    assert np.abs(ours - golden).max() <= 5e-6 * max(1.0, meta["max_abs_logit"])
    # the reference's own whole-prompt and cut/mixed runs were bit-identical when the files were made
    assert meta["reference_whole_vs_cut_and_mixed_max_abs_diff"] == 0.0


def test_plain_float64_agrees_with_float32():
    with open(os.path.join(GOLDEN, "tiny_b.json")) as f:
        meta = json.load(f)
    cfg = meta["config"]
    weights = plain_model.random_weights(cfg, meta["seed"], meta["std"], meta["norm_std"])
    p = meta["prompts"][-1]
    a = plain_model.forward_logits(weights, cfg, p, compute=torch.float32)
    b = plain_model.forward_logits(weights, cfg, p, compute=torch.float64)
    assert (a.double() - b).abs().max() <= 1e-5 * b.abs().max()


def test_plain_window_limits_keys():
    torch.manual_seed(0)
    T, nh, hd = 12, 2, 8
    q, k, v = torch.randn(T, nh, hd), torch.randn(T, 1, hd), torch.randn(T, 1, hd)
    full = plain_model.causal_attention(q, k, v, range(T))
    win = plain_model.causal_attention(q, k, v, range(T), window=4)
    assert torch.allclose(full[:4], win[:4])          # the first 4 queries see everything they may see
    assert not torch.allclose(full[6:], win[6:])
    # a window of 1 returns the query's own value
    one = plain_model.causal_attention(q, k, v, range(T), window=1)
    assert torch.allclose(one, v.expand(T, nh, hd), atol=1e-6)
