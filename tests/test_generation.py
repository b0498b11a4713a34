"""Generation through the Python entry point against the plain implementation: greedy
tokens, long decoding, the first tokens of a sequence, continuous batching with a pool so
small that requests are preempted and recomputed, and seeded temperature sampling."""
import numpy as np
import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu


def engine_for(folder, dtype, **kw):
    from spyinfer_b200 import LLMEngine
    opts = dict(dtype=dtype, max_num_seqs=4, max_model_len=512, kvcache_block_size=16, num_kvcache_blocks=64, max_num_batched_tokens=64)
    opts.update(kw)
    return LLMEngine(folder, **opts)


def all_pages_free(cache) -> bool:
    """Every group's pool is whole again (a windowed group's pool is smaller than the others')."""
    return all(cache.num_free_pages(g) == cache.group_pages[g] for g in range(cache.num_groups()))


def check_greedy(weights, cfg, prompt, out, dtype):
    """Every generated token is the plain implementation's argmax given the same history, or
    a token whose plain logit is within the dtype's reach of the best one."""
    seq = list(prompt)
    for i, tok in enumerate(out):
        logits = plain_model.forward_logits(weights, cfg, seq)[-1]
        best = logits.max().item()
        limit = 1e-4 * max(1.0, logits.abs().max().item()) if dtype == "float32" else 0.05 * logits.abs().max().item()
        assert logits[tok].item() >= best - limit, f"token {i}: engine chose {tok}, plain argmax {int(logits.argmax())}"
        seq.append(tok)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_greedy_generation_matches_plain(name, dtype, tiny_models):
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models[name]
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (1, 5, 9, 13, 31)]
    engine = engine_for(folder, dtype)
    outs = engine.generate(prompts, SamplingParams(max_new_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        check_greedy(weights, cfg, p, o, dtype)
    assert all_pages_free(engine.runner.cache) and max(engine.runner.cache.group_pages) == 64 and engine.runner.cache.num_free_slots() == 4
    engine.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(dtype, tiny_models):
    """A one-token prompt (the very first positions of a sequence), decoded for 200 tokens:
    across many pages and, in model c, far past its window of 40."""
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["c"]
    engine = engine_for(folder, dtype)
    out = engine.generate([[7]], SamplingParams(max_new_tokens=200, ignore_eos=True))[0]
    assert len(out) == 200
    # checking all 200 steps with the plain implementation is quadratic; check the first 24 and every 16th after
    seq = [7]
    for i, tok in enumerate(out):
        if i < 24 or i % 16 == 0 or i == 199:
            check_greedy(weights, cfg, seq, [tok], dtype)
        seq.append(tok)


def test_small_pool_preempts_and_still_gives_the_same_tokens(tiny_models):
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["b"]
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (20, 33, 7, 40, 12, 25)]
    sp = SamplingParams(max_new_tokens=30, ignore_eos=True)
    roomy = engine_for(folder, "float32", num_kvcache_blocks=64)
    want = roomy.generate(prompts, sp)
    del roomy
    tight = engine_for(folder, "float32", num_kvcache_blocks=9, max_num_batched_tokens=24)   # 144 tokens of cache for 6 requests of up to 70
    got = tight.generate(prompts, sp)
    assert tight.scheduler.num_preemptions > 0, "the pool was meant to be too small"
    assert got == want
    tight.runner.cache.check_invariants()
    assert tight.runner.cache.min_free_pages() == 9


def test_eos_and_max_model_len_finish_requests(tiny_models):
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["a"]
    engine = engine_for(folder, "float32", max_model_len=24)
    prompt = [3, 9, 27, 81]
    free_run = engine.generate([prompt], SamplingParams(max_new_tokens=10, ignore_eos=True))[0]
    # make the third generated token the end-of-sequence token
    engine.eos_token_id = free_run[2]
    rid = engine.add_request(prompt, SamplingParams(max_new_tokens=10))
    while not engine.is_request_finished(rid):
        engine.step()
    first_eos = free_run.index(free_run[2])
    assert engine.get_generated_tokens(rid) == free_run[:first_eos + 1] and engine.finish_reason(rid) == "eos"
    assert engine.get_output_tokens(rid) == prompt + free_run[:first_eos + 1]
    engine.remove_request(rid)
    engine.eos_token_id = -1
    rid = engine.add_request(prompt, SamplingParams(ignore_eos=True))
    while engine.has_unfinished_requests():
        engine.step()
    assert engine.finish_reason(rid) == "max_model_len" and len(engine.get_output_tokens(rid)) == 24
    with pytest.raises(ValueError):
        engine.add_request(list(range(24)))          # no room to generate
    with pytest.raises(ValueError):
        engine.add_request([cfg["vocab_size"]])      # outside the vocabulary


@pytest.mark.parametrize("lookahead", [True, False])
def test_requests_without_a_token_limit_end_where_the_pool_ends(lookahead, tiny_models):
    """The default ``SamplingParams()`` in a pool (3 pages of 16) smaller than ``max_model_len`` (512):
    the requests run to the pool's last token and end with the reason "out_of_pages"; the second one
    is preempted once for the first and recomputed.  ``generate`` returns, and the tokens are those of
    a roomy engine."""
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["a"]
    prompts = [[3, 9, 27, 81, 5, 6, 7], [2, 4, 8, 16]]
    roomy = engine_for(folder, "float32")
    want = roomy.generate(prompts, SamplingParams(max_new_tokens=48, ignore_eos=True))
    del roomy
    engine = engine_for(folder, "float32", num_kvcache_blocks=3, lookahead_decode=lookahead)
    got = engine.generate(prompts, SamplingParams(ignore_eos=True))
    assert [len(p) + len(o) for p, o in zip(prompts, got)] == [49, 49]          # 48 tokens in the cache and the one sampled from them
    assert got == [w[:len(g)] for w, g in zip(want, got)]
    assert engine.scheduler.num_preemptions == 1
    assert engine.runner.cache.min_free_pages() == 3 and engine.runner.cache.num_free_slots() == 4
    rid = engine.add_request(prompts[0])
    seen = []
    while engine.has_unfinished_requests():
        seen += engine.step()
    seen += engine.drain()
    assert engine.finish_reason(rid) == "out_of_pages" and [t for _, t, _ in seen] == got[0] and seen[-1][2]


def test_a_checkpoint_stored_in_32_bit_stays_so_and_the_bfloat16_engine_says_what_that_costs(tiny_models, tmp_path):
    import json
    import warnings

    from safetensors.torch import save_file

    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["d"]
    with open(tmp_path / "config.json", "w") as f:
        json.dump(cfg, f)
    save_file({k: v.float().contiguous() for k, v in weights.items()}, str(tmp_path / "model.safetensors"))
    with pytest.warns(UserWarning, match="stored in 32-bit.*CUDA-core kernel"):
        engine = engine_for(str(tmp_path), "bfloat16")
    assert engine.model.layers[0].mixer.o.weight.dtype == torch.float32 and not engine.model.layers[0].mixer.o.fast
    prompt = [9, 8, 7, 6, 5]
    out = engine.generate([prompt], SamplingParams(max_new_tokens=6, ignore_eos=True))[0]
    check_greedy(weights, cfg, prompt, out, "bfloat16")
    with warnings.catch_warnings():
        warnings.simplefilter("error")
        engine_for(folder, "bfloat16")                       # the bfloat16 checkpoint: no warning
        engine_for(str(tmp_path), "float32")                 # the 32-bit engine multiplies 32-bit matrices anyway


def test_temperature_sampling_is_seeded_and_follows_the_distribution(tiny_models):
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["a"]
    engine = engine_for(folder, "float32", max_num_seqs=64, num_kvcache_blocks=128, max_num_batched_tokens=512)
    prompt = [11, 22, 33]
    a = engine.generate([prompt] * 3, [SamplingParams(temperature=0.9, seed=s, max_new_tokens=8, ignore_eos=True) for s in (1, 1, 2)])
    assert a[0] == a[1] and a[0] != a[2]
    # the first generated token over many seeds follows softmax(logits / T) of the plain implementation
    n, temp = 4000, 1.5
    firsts = []
    for lo in range(0, n, 50):
        outs = engine.generate([prompt] * 50, [SamplingParams(temperature=temp, seed=s, max_new_tokens=1, ignore_eos=True) for s in range(lo, lo + 50)])
        firsts += [o[0] for o in outs]
    p = plain_model.softmax_probabilities(plain_model.forward_logits(weights, cfg, prompt)[-1], temp).numpy()
    freq = np.bincount(firsts, minlength=cfg["vocab_size"]) / n
    assert np.abs(freq - p).max() < 4 * np.sqrt(p.max() / n) + 2e-3


def test_top_k_of_one_is_greedy_and_top_k_limits_the_draws(tiny_models):
    """Through the entry point: with ``top_k=1`` a temperature draws the argmax; with ``top_k=3`` every first
    token over many seeds is one of the plain implementation's three most likely."""
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["b"]
    engine = engine_for(folder, "float32", max_num_seqs=64, num_kvcache_blocks=128, max_num_batched_tokens=512)
    prompt = [9, 8, 7, 6]
    greedy = engine.generate([prompt], SamplingParams(max_new_tokens=6, ignore_eos=True))[0]
    one = engine.generate([prompt] * 2, [SamplingParams(temperature=2.0, top_k=1, seed=s, max_new_tokens=6, ignore_eos=True) for s in (3, 4)])
    assert one[0] == greedy and one[1] == greedy
    outs = engine.generate([prompt] * 60, [SamplingParams(temperature=3.0, top_k=3, seed=s, max_new_tokens=1, ignore_eos=True) for s in range(60)])
    logits = plain_model.forward_logits(weights, cfg, prompt)[-1]
    top3 = set(torch.topk(logits, 3).indices.tolist())
    firsts = {o[0] for o in outs}
    assert firsts <= top3 and len(firsts) >= 2
    with pytest.raises(ValueError):
        SamplingParams(top_k=-1)


def test_step_raw_gives_the_plain_logits_and_leaves_the_scheduler_alone(tiny_models):
    """``LLMEngine.step_raw``: a prompt in two portions and a decoded token, logits against the plain
    implementation; afterwards the engine generates as if nothing had happened and every page is back."""
    from spyinfer_b200.engine import StepEntry
    folder, cfg, weights = tiny_models["a"]
    engine = engine_for(folder, "float32", max_num_seqs=4, num_kvcache_blocks=32, max_num_batched_tokens=64)
    free = engine.stats()["free_pages"]
    toks = [3, 14, 15, 92, 65, 35, 89]
    ref = plain_model.forward_logits(weights, cfg, toks).numpy()
    a = engine.step_raw([StepEntry("x", toks[:4], [3])])
    assert engine.step_raw([StepEntry("x", toks[4:6], [])]) is None
    b = engine.step_raw([StepEntry("x", toks[6:], [0])])
    np.testing.assert_allclose(a[0], ref[3], rtol=2e-4, atol=2e-5)
    np.testing.assert_allclose(b[0], ref[6], rtol=2e-4, atol=2e-5)
    engine.release_raw("x")
    assert engine.stats()["free_pages"] == free
    out = engine.generate([toks[:3]], SamplingParamsFor(4))[0]
    check_greedy(weights, cfg, toks[:3], out, "float32")


@pytest.mark.parametrize("dtype,name", [("float32", "b"), ("bfloat16", "d"), ("bfloat16", "c")])
def test_small_steps_of_any_shape_replayed_from_graphs_equal_eager_steps(tiny_models, dtype, name):
    """Small steps that are no decode steps (a prompt portion beside decoded tokens of others) are padded to a few
    sizes and replayed from CUDA graphs.  Seven steps of the same padded sizes but different shapes inside (the
    first runs eagerly, the second is captured, the rest are replays) give what an engine without graphs gives,
    row for row, and what the plain implementation gives; the padding leaves nothing behind in the cache."""
    from spyinfer_b200.engine import StepEntry
    folder, cfg, weights = tiny_models[name]
    rng = np.random.default_rng(11)
    V = cfg["vocab_size"]
    seqs = {r: rng.integers(1, V, size=60).tolist() for r in ("u", "v", "w0", "w1", "w2", "w3", "w4", "w5", "w6")}
    engines = [engine_for(folder, dtype, max_num_seqs=8, num_kvcache_blocks=64, max_num_batched_tokens=128, use_cuda_graphs=g) for g in (True, False)]
    free = [e.stats()["free_pages"] for e in engines]
    outs = [[], []]
    for i, engine in enumerate(engines):
        done = {"u": 0, "v": 0}
        for r, n in (("u", 9), ("v", 30)):                       # two requests under way
            engine.step_raw([StepEntry(r, seqs[r][:n], [])])
            done[r] = n
        for k in range(7):
            w, n = f"w{k}", 17 + k                                  # a new request's prompt of 17 ... 23 tokens beside two decoded tokens
            entries = [StepEntry("u", seqs["u"][done["u"]:done["u"] + 1], [0]), StepEntry(w, seqs[w][:n], [n - 1, 0] if k % 2 else [n - 1]),
                       StepEntry("v", seqs["v"][done["v"]:done["v"] + 1], [0])]
            outs[i].append(engine.step_raw(entries).copy())
            done["u"] += 1
            done["v"] += 1
            engine.release_raw(w)
        for r in ("u", "v"):
            engine.release_raw(r)
        assert engine.stats()["free_pages"] == free[i]
    assert engines[0].runner.graph_steps >= 5 and engines[1].runner.graph_steps == 0
    tol = dict(rtol=2e-4, atol=2e-5) if dtype == "float32" else dict(rtol=3e-2, atol=3e-2)
    for k, (a, b) in enumerate(zip(*outs)):
        assert a.shape == b.shape
        np.testing.assert_allclose(a, b, **(dict(rtol=1e-5, atol=1e-6) if dtype == "float32" else tol), err_msg=f"step {k}")
    # against the plain implementation: the new request's last row and u's decoded rows
    ref_u = plain_model.forward_logits(weights, cfg, seqs["u"][:16]).numpy()
    for k in range(7):
        n = 17 + k
        ref_w = plain_model.forward_logits(weights, cfg, seqs[f"w{k}"][:n]).numpy()
        scale = np.abs(ref_w).max()
        np.testing.assert_allclose(outs[0][k][0], ref_u[9 + k], rtol=tol["rtol"], atol=tol["atol"] * max(1.0, scale))
        np.testing.assert_allclose(outs[0][k][1], ref_w[n - 1], rtol=tol["rtol"], atol=tol["atol"] * max(1.0, scale))


@pytest.mark.parametrize("seed", [1, 2])
def test_random_engine_options_and_request_mixes(tiny_models, seed):
    """Forty engines with options drawn at random (page size, live requests, token budget, portion cap, pool from barely
    enough to ample, graphs for small steps on or off, both dtypes, every tiny model) generate for one to nine requests of
    random lengths each; a sample of every request's tokens is held against the plain implementation, every page comes
    back and the cache's invariants hold.  (The same loop ran for 3,300 engines and 250,000 tokens when it was written.)"""
    from spyinfer_b200 import LLMEngine, SamplingParams
    rng = np.random.default_rng(seed)
    for _ in range(40):
        name = str(rng.choice(sorted(tiny_models)))
        dtype = str(rng.choice(["bfloat16", "bfloat16", "float32"]))
        folder, cfg, weights = tiny_models[name]
        page, seqs, budget = int(rng.choice([4, 8, 16, 32])), int(rng.integers(1, 9)), int(rng.choice([16, 24, 64, 128, 300]))
        n_req = int(rng.integers(1, 10))
        prompts = [rng.integers(0, cfg["vocab_size"], int(rng.integers(1, 140))).tolist() for _ in range(n_req)]
        new = [int(rng.integers(1, 30)) for _ in range(n_req)]
        need = max((len(p) + n + page - 1) // page + 1 for p, n in zip(prompts, new))
        pages = int(rng.integers(need, need * max(2, n_req) + 1))
        chunk = None if rng.random() < 0.5 else int(rng.choice([3, 7, 16, 50]))
        what = dict(model=name, dtype=dtype, page=page, seqs=seqs, budget=budget, pages=pages, chunk=chunk, lens=[len(p) for p in prompts], new=new)
        engine = LLMEngine(folder, dtype=dtype, max_num_seqs=seqs, max_model_len=256, kvcache_block_size=page, num_kvcache_blocks=pages,
                           max_num_batched_tokens=budget, chunk_size=chunk, graph_step_tokens=int(rng.choice([0, 64, 384])))
        outs = engine.generate(prompts, [SamplingParams(max_new_tokens=n, ignore_eos=True) for n in new])
        for p, o, n in zip(prompts, outs, new):
            assert len(o) == n, what
            seq = list(p)
            for i, tok in enumerate(o):
                if i == 0 or i % 11 == 5 or i == n - 1:
                    check_greedy(weights, cfg, seq, [tok], dtype)
                seq.append(tok)
        assert all_pages_free(engine.runner.cache), what
        engine.runner.cache.check_invariants()


@pytest.mark.parametrize("decoders", [[1100], [30, 9, 60, 200, 45]])
def test_small_steps_with_decode_kernel_requests_replayed_from_graphs(tiny_models, decoders):
    """Small mixed steps whose one-token requests go through the decode kernel (one request holding more than a thousand keys,
    or five requests: the graph's head is then padded to eight with one-token requests of padding): six steps of the same
    padded sizes, each a new request's prompt beside the decoded tokens, give what an engine without graphs gives and what
    the plain implementation gives, rows in the order of the entries."""
    from spyinfer_b200.engine import StepEntry
    folder, cfg, weights = tiny_models["d"]
    rng = np.random.default_rng(len(decoders))
    V = cfg["vocab_size"]
    dec = {f"u{i}": rng.integers(1, V, size=n + 8).tolist() for i, n in enumerate(decoders)}
    news = [rng.integers(1, V, size=20 + k).tolist() for k in range(6)]
    outs = []
    for graphs in (True, False):
        engine = engine_for(folder, "bfloat16", max_num_seqs=16, max_model_len=2048, num_kvcache_blocks=256, max_num_batched_tokens=2048, use_cuda_graphs=graphs)
        done = {}
        for (r, toks), n in zip(dec.items(), decoders):
            engine.step_raw([StepEntry(r, toks[:n], [])])
            done[r] = n
        got = []
        for k, new in enumerate(news):
            names = list(dec)
            entries = ([StepEntry(r, dec[r][done[r]:done[r] + 1], [0]) for r in names[:1]] + [StepEntry(f"w{k}", new, [len(new) - 1])]
                       + [StepEntry(r, dec[r][done[r]:done[r] + 1], [0]) for r in names[1:]])
            got.append(engine.step_raw(entries).copy())
            for r in names:
                done[r] += 1
            engine.release_raw(f"w{k}")
        outs.append(got)
        if graphs:
            assert engine.runner.graph_steps >= 4
            keys = [k for k in engine.runner._graphs if isinstance(k, tuple)]
            assert keys and all(k[4] == (1 if len(decoders) == 1 else 8) for k in keys), keys
    for k, (a, b) in enumerate(zip(*outs)):
        np.testing.assert_allclose(a, b, rtol=3e-2, atol=3e-2, err_msg=f"step {k}")
    first = list(dec)[0]
    ref_first = plain_model.forward_logits(weights, cfg, dec[first][:decoders[0] + 6]).numpy()
    for k, new in enumerate(news):
        ref_new = plain_model.forward_logits(weights, cfg, new).numpy()
        scale = max(np.abs(ref_new).max(), np.abs(ref_first).max())
        np.testing.assert_allclose(outs[0][k][0], ref_first[decoders[0] + k], rtol=3e-2, atol=5e-2 * scale)
        np.testing.assert_allclose(outs[0][k][1], ref_new[-1], rtol=3e-2, atol=5e-2 * scale)


def test_one_long_request_decoding_beside_a_portion(tiny_models):
    """A single decoded token whose request holds more than a thousand keys, beside a prompt portion of another request: the
    decode kernel takes it (one 256-row block would walk its cache alone); logits as the plain implementation has them."""
    from spyinfer_b200.engine import StepEntry
    folder, cfg, weights = tiny_models["d"]
    rng = np.random.default_rng(41)
    long_one, other = rng.integers(1, cfg["vocab_size"], size=1300).tolist(), rng.integers(1, cfg["vocab_size"], size=500).tolist()
    engine = LLMEngine_for_long(folder)
    assert engine.step_raw([StepEntry("long", long_one[:-1], [])]) is None
    got = engine.step_raw([StepEntry("other", other, [499]), StepEntry("long", long_one[-1:], [0])])
    ref_long = plain_model.forward_logits(weights, cfg, long_one)[-1].numpy()
    ref_other = plain_model.forward_logits(weights, cfg, other)[-1].numpy()
    for row, ref in ((got[0], ref_other), (got[1], ref_long)):
        np.testing.assert_allclose(row, ref, rtol=3e-2, atol=5e-2 * np.abs(ref).max())


def LLMEngine_for_long(folder):
    return engine_for(folder, "bfloat16", max_num_seqs=4, max_model_len=2048, num_kvcache_blocks=160, max_num_batched_tokens=2048, graph_step_tokens=0)


@pytest.mark.parametrize("name,graphs", [("d", False), ("d", True), ("c", False), ("b", True)])
def test_decoded_tokens_beside_a_portion_take_the_decode_kernel(tiny_models, name, graphs):
    """A step that mixes many decoded tokens with prompt portions lays the one-token requests out first and runs their
    attention through the decode kernel, the portions through the kernel for portions.  The logits come back in the order
    of the entries as given (a portion first, decoded tokens around a second portion), every row as the plain
    implementation has it; with graphs on, twenty decoded tokens are too many for a padded graph and take the same path."""
    from spyinfer_b200.engine import StepEntry
    folder, cfg, weights = tiny_models[name]
    rng = np.random.default_rng(23)
    V = cfg["vocab_size"]
    n_dec = 20 if graphs else 7
    engine = engine_for(folder, "bfloat16", max_num_seqs=32, num_kvcache_blocks=256, max_num_batched_tokens=512, use_cuda_graphs=graphs)
    seqs = {f"r{i}": rng.integers(1, V, size=int(rng.integers(3, 150))).tolist() for i in range(n_dec)}
    for r, toks in seqs.items():                                     # the requests that will decode: all but their last token
        assert engine.step_raw([StepEntry(r, toks[:-1], [])]) is None
    p1, p2 = rng.integers(1, V, size=45).tolist(), rng.integers(1, V, size=133).tolist()
    engine.step_raw([StepEntry("p2", p2[:100], [])])
    names = list(seqs)
    entries = ([StepEntry("p1", p1, [0, 44])] + [StepEntry(r, seqs[r][-1:], [0]) for r in names[:3]] + [StepEntry("p2", p2[100:], [32, 5])]
               + [StepEntry(r, seqs[r][-1:], [0]) for r in names[3:]])
    got = engine.step_raw(entries)
    want = []
    for e in entries:
        full = p1 if e.request == "p1" else (p2 if e.request == "p2" else seqs[e.request])
        ref = plain_model.forward_logits(weights, cfg, full).numpy()
        start = len(full) - len(e.tokens)
        want += [ref[start + w] for w in e.want]
    want = np.stack(want)
    assert got.shape == want.shape
    scale = np.abs(want).max()
    np.testing.assert_allclose(got, want, rtol=3e-2, atol=5e-2 * scale)
    assert np.sqrt(((got - want) ** 2).mean()) <= 2e-2 * np.sqrt((want ** 2).mean())


def SamplingParamsFor(n):
    from spyinfer_b200 import SamplingParams
    return SamplingParams(max_new_tokens=n, ignore_eos=True)


def test_command_line_generates(tiny_models):
    import os, subprocess, sys
    folder, cfg, weights = tiny_models["a"]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bin", "spyinfer"), "-m", folder, "--dtype", "float32", "--prompt-tokens", "5,6,7",
           "--max-new-tokens", "5", "--ignore-eos", "--max-model-len", "64", "--num-kvcache-blocks", "8", "--stats"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = proc.stdout.strip().splitlines()
    tokens = [int(t) for t in lines[1].split()]
    assert len(tokens) == 5
    check_greedy(weights, cfg, [5, 6, 7], tokens, "float32")
    assert "steps" in lines[-1]
    # a seeded random prompt of a given length, pages named by the short options
    cmd = [sys.executable, os.path.join(root, "bin", "spyinfer"), "-m", folder, "--dtype", "float32", "--prompt-len", "9", "--seed", "3",
           "--max-new-tokens", "3", "--ignore-eos", "--max-model-len", "64", "--page-size", "4", "--num-pages", "16"]
    proc = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert len([int(t) for t in proc.stdout.strip().splitlines()[1].split()]) == 3
    bad = subprocess.run([sys.executable, os.path.join(root, "bin", "spyinfer"), "-m", folder, "-b", "cpu"], capture_output=True, text=True)
    assert bad.returncode == 1 and "Invalid backend type" in bad.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_steps_launched_ahead_give_the_same_tokens(dtype, tiny_models):
    """``lookahead_decode`` launches the next decode step before the last one's tokens are read (their ids
    stay on the device).  The tokens must be those of the engine that reads every step first: greedy
    and seeded temperature sampling, requests of different lengths that end at different steps, and a
    request that ends by its end-of-sequence token, whose one token too many is dropped.  Through
    ``step()`` every token is reported exactly once, a call later."""
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["d"]
    rng = np.random.default_rng(9)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (3, 17, 40)]
    params = [SamplingParams(max_new_tokens=25, ignore_eos=True), SamplingParams(max_new_tokens=9, ignore_eos=True),
              SamplingParams(temperature=0.8, seed=4, max_new_tokens=30, ignore_eos=True)]
    plain = engine_for(folder, dtype, lookahead_decode=False)
    ahead = engine_for(folder, dtype, lookahead_decode=True)
    want = plain.generate(prompts, params)
    assert ahead.generate(prompts, params) == want
    assert [len(w) for w in want] == [25, 9, 30]
    # end of sequence in the middle of decoding
    eos = want[0][10]
    first = want[0].index(eos)
    for engine in (plain, ahead):
        engine.eos_token_id = eos
        rid = engine.add_request(prompts[0], SamplingParams(max_new_tokens=25))
        seen = []
        while not engine.is_request_finished(rid):
            seen += [(tok, done) for r, tok, done in engine.step() if r == rid]
        assert [t for t, _ in seen] == want[0][:first + 1] and [d for _, d in seen] == [False] * first + [True]
        assert engine.get_generated_tokens(rid) == want[0][:first + 1] and engine.finish_reason(rid) == "eos"
        engine.remove_request(rid)
        assert all(r != rid for r, _, _ in engine.drain())     # what was launched ahead for it is dropped
        engine.runner.cache.check_invariants()
        assert engine.runner.cache.num_free_slots() == 4 and all_pages_free(engine.runner.cache)


def test_launching_ahead_gives_way_when_pages_run_out(tiny_models):
    """A pool so small that requests are preempted: the step launched ahead finds no page, the
    scheduler decides who gives way once the tokens are known, and the tokens are those of the engine
    that never launches ahead."""
    from spyinfer_b200 import SamplingParams
    folder, cfg, weights = tiny_models["b"]
    rng = np.random.default_rng(21)
    prompts = [rng.integers(0, cfg["vocab_size"], n).tolist() for n in (30, 11, 45, 8, 27, 19)]
    sp = [SamplingParams(max_new_tokens=n, ignore_eos=True, temperature=t, seed=3) for n, t in ((30, 0.0), (22, 0.7), (17, 0.0), (30, 0.0), (9, 1.1), (25, 0.0))]
    outs = []
    for ahead in (False, True):
        engine = engine_for(folder, "float32", num_kvcache_blocks=9, max_num_batched_tokens=24, lookahead_decode=ahead)
        outs.append(engine.generate(prompts, sp))
        assert engine.scheduler.num_preemptions > 0, "the pool was meant to be too small"
        engine.runner.cache.check_invariants()
        assert all_pages_free(engine.runner.cache) and engine.runner.cache.num_free_slots() == 4
    assert outs[0] == outs[1] and [len(o) for o in outs[0]] == [30, 22, 17, 30, 9, 25]
