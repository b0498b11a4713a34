"""Trace replay through ``bin/trace_run`` against the plain implementation, in 32-bit and in
bfloat16: each request alone and whole; most of it in one step and the last 32 tokens one by
one; in portions of changing size down to two tokens; and mixed, up to four live requests,
portions of some beside decoded tokens of others, in a pool so small that pages are used
again.  One process replays all of this for a (model, page size, dtype) triple; the tests
then compare every row with the plain implementation's row for the same request and
position.

Page sizes: every model at the program's own 16 (pool given by ``--max-tokens``), and the
reference workloads' own sizes, Tiny A at 4 and Tiny B at 8 (B with prompt portions of 5
beside decoding requests), and Tiny D at 4, with ``--num-pages`` set to the exact peak of
the trace in pages, so that every page given back is handed out again.  Pages of 4 are no
TMA box, so at D's head size of 64 the bfloat16 runs at that size go through the
``mma.sync`` attention kernel's split mode (decoding) and tiles mode (portions) inside the
engine, which pages of 16 never reach."""
import random

import numpy as np
import pytest
import torch

from conftest import TINY
from trace_tools import TraceBuilder, mixed_trace, peak_pages, peak_tokens, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = [1, 2, 7, 21, 43, 70, 150, 330]
PORTIONS = (7, 5, 3, 2, 2, 11, 2, 16, 17)

# float32: the engine and the plain implementation both compute in 32-bit with different
# orders of sums; the plain implementation differs from the reference's CPU path by a few
# 1e-7 on these models, so 3e-5 of the largest logit is two orders above rounding.
# bfloat16: ten roundings to 8 bits of mantissa per layer around a 32-bit residual stream.
TOL = {"float32": dict(max_rel=3e-5, rms_rel=1e-5), "bfloat16": dict(max_rel=5e-2, rms_rel=2e-2)}


def requests_of(name):
    rng = random.Random(TINY[name]["seed"])
    vocab = TINY[name]["config"]["vocab_size"]
    return {f"r{n}": [rng.randrange(vocab) for _ in range(n)] for n in LENGTHS}


# (model, page size); None: the program's default with the pool from --max-tokens
CASES = [("a", None), ("b", None), ("c", None), ("d", None), ("e", None), ("a", 4), ("b", 8), ("d", 4)]
CASE_IDS = [f"{n}-page{p or 16}" for n, p in CASES]


def build_all_modes(name, mixed_portions=(7, 5, 3, 2)):
    reqs = requests_of(name)
    b = TraceBuilder()
    tokens_of = {}
    for rid, toks in reqs.items():
        b.whole("w_" + rid, toks)
        tokens_of["w_" + rid] = toks
    for rid, toks in reqs.items():
        if len(toks) > 2:
            b.tail_one_by_one("t_" + rid, toks, tail=32)
            tokens_of["t_" + rid] = toks
            b.portions("p_" + rid, toks, PORTIONS)
            tokens_of["p_" + rid] = toks
    mixed = {"m_" + rid: toks for rid, toks in reqs.items()}
    prompt_lens = {rid: max(1, len(toks) - 12) for rid, toks in mixed.items()}
    mixed_trace(b, mixed, prompt_lens, random.Random(7), max_live=4, portion_sizes=mixed_portions)
    tokens_of.update(mixed)
    return b, tokens_of


@pytest.fixture(scope="module")
def replayed(tiny_models, tmp_path_factory):
    memo = {}

    def get(name, dtype, page_size=None):
        if (name, dtype, page_size) not in memo:
            folder, cfg, _ = tiny_models[name]
            # Tiny B's reference workload: prompt portions of 5 beside decoding requests
            b, tokens_of = build_all_modes(name, mixed_portions=(5,) if (name, page_size) == ("b", 8) else (7, 5, 3, 2))
            # the pool is the mixed part's peak (four live requests), so earlier requests' pages are
            # handed to later ones throughout the trace; with a page size given, the peak to the page
            options = [] if page_size is None else ["--page-size", page_size, "--num-pages", peak_pages(b, page_size)]
            out = run_trace(folder, dtype, b, str(tmp_path_factory.mktemp(f"trace_{name}_{dtype}_{page_size}")), peak_tokens(b), cfg["vocab_size"],
                            options=options)
            memo[(name, dtype, page_size)] = (out, tokens_of)
        return memo[(name, dtype, page_size)]

    return get


def compare(rows, tokens_of, prefix, name, tiny_models, plain_logits_cache, tol):
    _, cfg, weights = tiny_models[name]
    picked = {k: v for k, v in rows.items() if k[0].startswith(prefix)}
    assert picked, "the trace produced no rows for this mode"
    worst = None
    for rid in sorted({k[0] for k in picked}):
        want = plain_logits_cache(name, cfg, weights, tokens_of[rid]).numpy()
        got = np.stack([picked[(rid, p)] for p in range(len(tokens_of[rid]))])  # every position was asked for
        assert np.isfinite(got).all(), f"{rid}: logits are not finite"
        err = np.abs(got - want)
        scale, rms = np.abs(want).max(), np.sqrt((want ** 2).mean())
        bad = np.argwhere(err > tol["max_rel"] * scale)
        if len(bad):
            first = int(bad[:, 0].min())
            raise AssertionError(f"{rid} ({len(tokens_of[rid])} tokens): first wrong position {first}, error "
                                 f"{err[first].max():.3g} against a largest logit of {scale:.3g} (allowed {tol['max_rel'] * scale:.3g}); "
                                 f"page slot {first % 16}, page {first // 16}")
        assert np.sqrt((err ** 2).mean()) <= tol["rms_rel"] * rms, f"{rid}: rms error {np.sqrt((err ** 2).mean()):.3g} vs rms logit {rms:.3g}"
        worst = max(worst or 0.0, float(err.max() / scale))
    return worst


MODES = {"whole": "w_", "tail_one_by_one": "t_", "portions": "p_", "mixed": "m_"}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,page_size", CASES, ids=CASE_IDS)
@pytest.mark.parametrize("mode", list(MODES))
def test_replay_matches_plain(mode, name, page_size, dtype, replayed, tiny_models, plain_logits_cache):
    rows, tokens_of = replayed(name, dtype, page_size)
    compare(rows, tokens_of, MODES[mode], name, tiny_models, plain_logits_cache, TOL[dtype])


@pytest.mark.parametrize("name,page_size", CASES, ids=CASE_IDS)
def test_float32_does_not_depend_on_the_cut(name, page_size, replayed):
    """In 32-bit every token's arithmetic is arranged to be independent of the batch: the
    same request gives the same logits, to the last bit or nearly so, however it was cut."""
    rows, tokens_of = replayed(name, "float32", page_size)
    for rid in [r for r in tokens_of if r.startswith("w_")]:
        base = rid[2:]
        for other in ("t_", "p_", "m_"):
            if other + base not in tokens_of:
                continue
            for p in range(len(tokens_of[rid])):
                a, b = rows[(rid, p)], rows[(other + base, p)]
                assert np.abs(a - b).max() <= 2e-6 * max(1.0, np.abs(a).max()), f"{base} position {p}: whole vs {other} differ"


def test_float32_does_not_depend_on_the_page_size(replayed):
    """The same requests in pages of 16 and of 4: where a key lies in the cache changes nothing."""
    for name, small in (("a", 4), ("b", 8), ("d", 4)):
        rows16, tokens_of = replayed(name, "float32", None)
        rows_small, _ = replayed(name, "float32", small)
        for rid in [r for r in tokens_of if r.startswith(("w_", "p_"))]:
            for p in range(len(tokens_of[rid])):
                a, b = rows16[(rid, p)], rows_small[(rid, p)]
                assert np.abs(a - b).max() <= 2e-6 * max(1.0, np.abs(a).max()), f"{name} {rid} position {p}: pages of 16 and of {small} differ"


def test_random_model_from_a_configuration_and_a_seed(tiny_models, tmp_path):
    """``--random CONFIG --seed N`` in place of a model folder: the same seed gives the same model
    (two runs, cut differently, agree), it is the model that ``write_model_folder`` writes for that
    seed (checked through the plain implementation on the tensors of such a folder), and another
    seed gives another model."""
    import json

    from safetensors.torch import load_file

    from spyinfer_b200.config import config_from_json
    from spyinfer_b200.weights import write_model_folder

    import plain_model

    cfg = TINY["b"]["config"]
    with open(tmp_path / "tiny_b_config.json", "w") as f:       # a file name of its own, not config.json
        json.dump(cfg, f)
    toks = requests_of("b")["r43"]
    whole, cut = TraceBuilder(), TraceBuilder()
    whole.whole("x", toks)
    cut.portions("x", toks, (5, 2, 9))
    args = ["--random", str(tmp_path / "tiny_b_config.json"), "--weight-std", "0.03", "--norm-std", "0.1"]
    a = run_trace("", "float32", whole, str(tmp_path / "a"), 64, cfg["vocab_size"], model_args=args + ["--seed", "5"], options=["--page-size", 8])
    b = run_trace("", "float32", cut, str(tmp_path / "b"), 64, cfg["vocab_size"], model_args=args + ["--seed", "5"], options=["--page-size", 8])
    c = run_trace("", "float32", whole, str(tmp_path / "c"), 64, cfg["vocab_size"], model_args=args + ["--seed", "6"])
    write_model_folder(str(tmp_path / "model"), config_from_json(cfg), 5, 0.03, 0.1)
    want = plain_model.forward_logits(load_file(str(tmp_path / "model" / "model.safetensors")), cfg, toks).numpy()
    for p in range(len(toks)):
        assert np.abs(a[("x", p)] - b[("x", p)]).max() <= 2e-6 * max(1.0, np.abs(a[("x", p)]).max())
        assert np.abs(a[("x", p)] - want[p]).max() <= TOL["float32"]["max_rel"] * np.abs(want).max()
    assert np.abs(a[("x", 42)] - c[("x", 42)]).max() > 1e-3
