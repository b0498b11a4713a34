"""Each part alone against the plain implementation's function for it, at sizes other than
the tiny models'; then arrangements that only a description can express: a run order that
names a layer twice and lets an entry read another entry's cache, and a toy mixer with a
state of its own that is defined here, registered, built and stepped without any change to
the package."""
import math

import numpy as np
import pytest
import torch

import plain_model

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def ctx_for(dtype, max_len=512):
    from spyinfer_b200.parts import BuildContext
    return BuildContext(dtype=dtype, device=torch.device(DEV), max_model_len=max_len)


def bound(part, std=0.05, seed=0):
    """Binds seeded random weights to a part; returns them by relative name (on the CPU)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for d in part.weight_decls():
        x = torch.randn(d.shape, generator=g)
        x = 1 + 0.1 * x if d.init == "one_plus_normal" else x * std
        w[d.name] = x.to(torch.bfloat16)
    part.bind({k: v.to(DEV) for k, v in w.items()})
    return w


def close(got, want, dtype):
    if dtype == torch.float32:
        torch.testing.assert_close(got.float().cpu(), want, rtol=1e-4, atol=1e-5 * max(1.0, want.abs().max().item()))
    else:
        err = (got.float().cpu() - want).abs().max().item()
        assert err <= 4e-2 * max(want.abs().max().item(), 1e-3), f"max error {err} against a largest value of {want.abs().max().item()}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_part(dtype):
    from spyinfer_b200.config import PartSpec
    from spyinfer_b200.parts import build_part
    part = build_part(PartSpec("rms_norm", {"size": 200, "eps": 1e-4, "weight": "n.weight"}), ctx_for(dtype))
    w = bound(part)
    x = torch.randn(9, 200)
    delta = torch.randn(9, 200).to(dtype)
    want = plain_model.rms_norm(x, w["n.weight"], 1e-4)
    close(part.forward(x.to(DEV)), want, dtype)
    res = x.to(DEV).clone()
    got = part.forward_add(res, delta.to(DEV))
    close(got, plain_model.rms_norm(x + delta.float(), w["n.weight"], 1e-4), dtype)
    torch.testing.assert_close(res.cpu(), x + delta.float())      # the residual stream holds the 32-bit sum


def test_rotary_half_table():
    from spyinfer_b200.config import PartSpec
    from spyinfer_b200.parts import build_part
    part = build_part(PartSpec("rotary_half", {"theta": 1e6, "rotary_dim": 48}), ctx_for(torch.float32, 300))
    table = part.rotation_table().cpu()
    cos, sin = plain_model.rotary_angles(range(300), 48, 1e6)
    torch.testing.assert_close(table[..., 0], cos, rtol=0, atol=3e-6)
    torch.testing.assert_close(table[..., 1], sin, rtol=0, atol=3e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_mlp_part(dtype):
    from spyinfer_b200.config import PartSpec
    from spyinfer_b200.parts import build_part
    part = build_part(PartSpec("gated_mlp", {"hidden_size": 72, "intermediate_size": 200, "activation": "silu", "prefix": "mlp."}), ctx_for(dtype))
    w = bound(part, std=0.2)
    x = torch.randn(11, 72).to(dtype)
    want = plain_model.feed_forward(x.float(), w, "")
    got = part.forward(x.to(DEV))
    close(got.sum(dim=0) if got.dim() == 3 else got, want, dtype)


def one_step_batch(cache, lens, device):
    """A batch that brings every sequence whole (positions 0..len-1)."""
    from spyinfer_b200.engine.batch import BatchStager
    stager = BatchStager(device, 1024, 8, cache.width, max(1, cache.num_groups()))
    tok, pos, seq, qs, cl, slots = [], [], [], [0], [], []
    for s, n in enumerate(lens):
        rid = f"s{s}"
        cache.add_request(rid)
        cache.reserve(rid, n)
        tok += [0] * n
        pos += range(n)
        seq += [s] * n
        qs.append(qs[-1] + n)
        cl.append(n)
        slots.append(cache.slot(rid))
    i32 = lambda a: np.asarray(a, dtype=np.int32)
    tables = [cache.gather_block_tables([f"s{s}" for s in range(len(lens))], g) for g in range(cache.num_groups())]
    return stager.stage(i32(tok), i32(pos), i32(seq), i32(qs), i32(cl), i32(slots), i32([]), tables)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window,rot", [(6, 2, 32, None, 32), (4, 4, 80, 9, 80), (8, 1, 64, None, 32)])
def test_attention_part(dtype, nh, nkv, hd, window, rot):
    from spyinfer_b200.cache import CacheManager
    from spyinfer_b200.config import PartSpec
    from spyinfer_b200.parts import build_part
    H, eps, theta = 88, 1e-5, 5000.0
    spec = PartSpec("attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qk_norm_eps": eps,
                                  "position": PartSpec("rotary_half", {"theta": theta, "rotary_dim": rot}), "window": window,
                                  "scale": None, "prefix": "self_attn."})
    part = build_part(spec, ctx_for(dtype))
    w = bound(part, std=0.15)
    lens = [23, 1, 40]
    cache = CacheManager([part.cache_need()], 8, 32, 4, 512, dtype=dtype, device=torch.device(DEV))
    batch = one_step_batch(cache, lens, torch.device(DEV))
    view = cache.view(0)
    view.block_table = batch.block_tables[0]
    x = torch.randn(sum(lens), H).to(dtype)
    got = part.forward(x.to(DEV), batch, view).float()
    if got.dim() == 3:          # the output projection may hand over its split-K partial products unsummed
        got = got.sum(dim=0)
    got = got.cpu()
    assert batch.status[0].item() == 0
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "rms_norm_eps": eps, "rope_theta": theta}
    off = 0
    for n in lens:
        xs = x[off:off + n].float()
        if rot == hd:
            want = plain_model.attention_mixer(xs, w, "", cfg, list(range(n)), window=window)
        else:   # partial rotation: only the first `rot` elements of each head are rotated
            q = plain_model.rms_norm(plain_model.linear(xs, w["self_attn.q_proj.weight"]).reshape(n, nh, hd), w["self_attn.q_norm.weight"], eps)
            k = plain_model.rms_norm(plain_model.linear(xs, w["self_attn.k_proj.weight"]).reshape(n, nkv, hd), w["self_attn.k_norm.weight"], eps)
            v = plain_model.linear(xs, w["self_attn.v_proj.weight"]).reshape(n, nkv, hd)
            cos, sin = plain_model.rotary_angles(range(n), rot, theta)
            q = torch.cat([plain_model.rotate_half(q[..., :rot], cos, sin), q[..., rot:]], dim=-1)
            k = torch.cat([plain_model.rotate_half(k[..., :rot], cos, sin), k[..., rot:]], dim=-1)
            o = plain_model.causal_attention(q, k, v, range(n), window=window)
            want = plain_model.linear(o.reshape(n, nh * hd), w["self_attn.o_proj.weight"])
        close(got[off:off + n], want, dtype)
        off += n


TOY_DECAY = 0.75


def register_toy_parts():
    """A mixer with a state of its own (a decaying sum of its inputs, one vector per request)
    and the cache need that goes with it.  Defined here, in the test, through the public
    registry only."""
    from spyinfer_b200.config import StateCacheNeed
    from spyinfer_b200.parts import Mixer, register_part
    from spyinfer_b200.weights import WeightDecl

    @register_part("toy_decay_mixer")
    class ToyDecayMixer(Mixer):
        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.hidden = params["hidden_size"]
            self.weight = None

        def weight_decls(self):
            return [WeightDecl("toy.weight", (self.hidden, self.hidden))]

        def bind(self, tensors):
            self.weight = tensors["toy.weight"].float()

        def cache_need(self):
            return StateCacheNeed((self.hidden,), "float32")

        def forward(self, x, batch, cache):
            out = torch.empty_like(x)
            for s in range(batch.num_seqs):
                slot = int(batch.host_state_slot[s])
                state = cache.state[slot].clone()
                for t in range(int(batch.host_q_start[s]), int(batch.host_q_start[s + 1])):
                    state = TOY_DECAY * state + x[t].float()
                    out[t] = (self.weight @ state).to(x.dtype)
                cache.state[slot] = state
            return out

    return ToyDecayMixer


def toy_spec():
    from spyinfer_b200.config import LayerSpec, ModelSpec, PartSpec, RunEntry
    H, V = 48, 97
    norm = lambda name: PartSpec("rms_norm", {"size": H, "eps": 1e-6, "weight": name})
    ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 80, "activation": "silu", "prefix": "mlp."})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": 3, "num_kv_heads": 1, "head_dim": 16, "qk_norm_eps": 1e-6,
                                  "position": PartSpec("rotary_half", {"theta": 10000.0, "rotary_dim": 16}), "window": None, "scale": None,
                                  "prefix": "self_attn."})
    toy = PartSpec("toy_decay_mixer", {"hidden_size": H})
    layers = [LayerSpec("pre_norm", norm("input_layernorm.weight"), m, norm("post_attention_layernorm.weight"), ffn, f"model.layers.{i}.")
              for i, m in enumerate([toy, attn, toy])]
    return ModelSpec(architecture="toy", hidden_size=H, vocab_size=V,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight": "model.embed_tokens.weight"}),
                     layers=layers, run_order=[RunEntry(0), RunEntry(1), RunEntry(2)], final_norm=norm("model.norm.weight"),
                     head=PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True, "weight": "lm_head.weight",
                                               "tied_to": "model.embed_tokens.weight"}), max_position=256)


def plain_toy_logits(w, tokens):
    cfg = {"num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 16, "rms_norm_eps": 1e-6, "rope_theta": 10000.0}
    h = plain_model.embed_tokens(w["model.embed_tokens.weight"], tokens)
    pos = list(range(len(tokens)))
    for i in range(3):
        p = f"model.layers.{i}."
        n = plain_model.rms_norm(h, w[p + "input_layernorm.weight"], 1e-6)
        if i == 1:
            a = plain_model.attention_mixer(n, w, p, cfg, pos)
        else:
            state, rows = torch.zeros(48), []
            for t in range(len(tokens)):
                state = TOY_DECAY * state + n[t]
                rows.append(w[p + "toy.weight"].float() @ state)
            a = torch.stack(rows)
        h = h + a
        n = plain_model.rms_norm(h, w[p + "post_attention_layernorm.weight"], 1e-6)
        h = h + plain_model.feed_forward(n, w, p)
    h = plain_model.rms_norm(h, w["model.norm.weight"], 1e-6)
    return plain_model.linear(h, w["model.embed_tokens.weight"])


def test_toy_mixer_with_state_is_registered_built_and_stepped():
    from spyinfer_b200.config import EngineConfig
    from spyinfer_b200.engine import Model, ModelRunner, StepEntry
    from spyinfer_b200.weights import random_tensors
    register_toy_parts()
    spec = toy_spec()
    cfg = EngineConfig(dtype="float32", max_num_seqs=3, max_model_len=128, kvcache_block_size=8, num_kvcache_blocks=24, max_num_batched_tokens=128)
    model = Model(spec, torch.float32, cfg.device, cfg.max_model_len)
    w = dict(random_tensors(model.weight_decls(), seed=4, std=0.1, norm_std=0.1))
    model.bind({k: v.to(DEV) for k, v in w.items()})
    runner = ModelRunner(model, cfg)
    assert [runner.cache.view(i).kind for i in range(3)] == ["state", "paged", "state"]
    rng = np.random.default_rng(0)
    seqs = {r: rng.integers(0, 97, n).tolist() for r, n in (("x", 19), ("y", 30), ("z", 5))}
    want = {r: plain_toy_logits(w, t) for r, t in seqs.items()}
    # x whole; y in portions beside z's single tokens; then a new request in x's old slot must start from a zero state
    got = runner.step([StepEntry("x", seqs["x"], range(19))]).cpu()
    torch.testing.assert_close(got, want["x"], rtol=1e-4, atol=1e-5)
    runner.finish("x")
    done = {"y": 0, "z": 0}
    sizes = [7, 2, 9, 5, 4, 3]
    rows = {"y": [], "z": []}
    for n in sizes:
        entries = [StepEntry("y", seqs["y"][done["y"]:done["y"] + n], range(n))]
        done["y"] += n
        if done["z"] < 5:
            entries.insert(0, StepEntry("z", seqs["z"][done["z"]:done["z"] + 1], [0]))
            done["z"] += 1
        out = runner.step(entries).cpu()
        off = 0
        for e in entries:
            rows[e.request].append(out[off:off + len(e.tokens)])
            off += len(e.tokens)
    runner.check_status()
    torch.testing.assert_close(torch.cat(rows["y"]), want["y"], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(torch.cat(rows["z"]), want["z"], rtol=1e-4, atol=1e-5)
    runner.finish("y"), runner.finish("z")
    got = runner.step([StepEntry("x2", seqs["x"], range(19))]).cpu()
    torch.testing.assert_close(got, want["x"], rtol=1e-4, atol=1e-5)
    runner.cache.check_invariants()


def test_run_order_names_a_layer_twice_and_reads_another_entrys_cache(tiny_models):
    """Run order [0, 1, 1 reading entry 1's cache, 0]: layer 1 runs twice with the same
    weights; its second run attends to the keys and values its first run stored.  Layer 0
    runs twice with a cache for each run."""
    from spyinfer_b200.config import EngineConfig, RunEntry, config_from_json
    from spyinfer_b200.engine import Model, ModelRunner, StepEntry
    folder, cfg, w = tiny_models["a"]
    spec = config_from_json(cfg).to_spec()
    spec.run_order = [RunEntry(0), RunEntry(1), RunEntry(1, cache_of=1), RunEntry(0)]
    ecfg = EngineConfig(dtype="float32", max_num_seqs=2, max_model_len=64, kvcache_block_size=4, num_kvcache_blocks=40, max_num_batched_tokens=64)
    model = Model(spec, torch.float32, ecfg.device, ecfg.max_model_len)
    model.load(folder)
    runner = ModelRunner(model, ecfg)
    assert len(runner.cache.groups[0].entries) == 3      # entries 0, 1 and 3 own a cache; entry 2 borrows
    tokens = np.random.default_rng(3).integers(0, cfg["vocab_size"], 21).tolist()
    # plain statement of the same run order
    T, pos = len(tokens), list(range(len(tokens)))
    nh, nkv, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    h = plain_model.embed_tokens(w["model.embed_tokens.weight"], tokens)
    kept = {}
    for idx, (layer, reads) in enumerate([(0, None), (1, None), (1, 1), (0, None)]):
        p = f"model.layers.{layer}."
        n = plain_model.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        cos, sin = plain_model.rotary_angles(pos, hd, cfg["rope_theta"])
        q = plain_model.rotate_half(plain_model.rms_norm(plain_model.linear(n, w[p + "self_attn.q_proj.weight"]).reshape(T, nh, hd),
                                                         w[p + "self_attn.q_norm.weight"], eps), cos, sin)
        if reads is None:
            k = plain_model.rotate_half(plain_model.rms_norm(plain_model.linear(n, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd),
                                                             w[p + "self_attn.k_norm.weight"], eps), cos, sin)
            v = plain_model.linear(n, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
            kept[idx] = (k, v)
        else:
            k, v = kept[reads]
        o = plain_model.causal_attention(q, k, v, pos)
        h = h + plain_model.linear(o.reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"])
        n = plain_model.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
        h = h + plain_model.feed_forward(n, w, p)
    want = plain_model.linear(plain_model.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])
    whole = runner.step([StepEntry("w", tokens, range(T))]).cpu()
    torch.testing.assert_close(whole, want, rtol=1e-4, atol=1e-5)
    cut = torch.cat([runner.step([StepEntry("c", tokens[a:b], range(b - a))]).cpu() for a, b in [(0, 9), (9, 11), (11, 12), (12, 21)]])
    torch.testing.assert_close(cut, want, rtol=1e-4, atol=1e-5)
    runner.check_status()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_head_and_block_parts(dtype):
    """Token embedding, tied and untied head, and the pre-norm block arrangement, each alone."""
    from spyinfer_b200.cache import CacheManager
    from spyinfer_b200.config import PartSpec
    from spyinfer_b200.parts import build_block, build_part
    V, H = 331, 72
    ctx = ctx_for(dtype)
    emb = build_part(PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight": "emb.weight"}), ctx)
    w_e = bound(emb, std=0.3)
    ids = torch.tensor([0, 330, 17, 17, 5], dtype=torch.int32, device=DEV)
    h = emb.forward(ids)
    assert h.dtype == torch.float32                     # the residual stream is 32-bit in both paths
    torch.testing.assert_close(h.cpu(), plain_model.embed_tokens(w_e["emb.weight"], ids.tolist()))
    for tied in (True, False):
        head = build_part(PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": tied, "weight": "head.weight", "tied_to": "emb.weight"}), ctx)
        if tied:
            assert head.weight_decls() == [] and head.ignorable == ["head.weight"]
            head.bind({"emb.weight": w_e["emb.weight"].to(DEV)})
            w_h = w_e["emb.weight"]
        else:
            w_h = bound(head, std=0.2, seed=5)["head.weight"]
        x = torch.randn(4, H).to(dtype)
        logits = head.forward(x.to(DEV))
        assert logits.dtype == torch.float32
        close(logits, plain_model.linear(x.float(), w_h), dtype)
    # block: h += attn(norm(h)); h += ffn(norm(h)), the second sum left pending as delta
    nh, nkv, hd, eps = 4, 2, 16, 1e-5
    norm1 = build_part(PartSpec("rms_norm", {"size": H, "eps": eps, "weight": "input_layernorm.weight"}), ctx)
    norm2 = build_part(PartSpec("rms_norm", {"size": H, "eps": eps, "weight": "post_attention_layernorm.weight"}), ctx)
    attn = build_part(PartSpec("attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qk_norm_eps": eps,
                                             "position": PartSpec("rotary_half", {"theta": 1e4, "rotary_dim": hd}), "window": None,
                                             "scale": None, "prefix": "self_attn."}), ctx)
    ffn = build_part(PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 104, "activation": "silu", "prefix": "mlp."}), ctx)
    w = {}
    for i, part in enumerate((norm1, norm2, attn, ffn)):
        w.update(bound(part, std=0.15, seed=10 + i))
    block = build_block("pre_norm", {"mixer_norm": norm1, "mixer": attn, "ffn_norm": norm2, "feed_forward": ffn})
    n = 13
    cache = CacheManager([attn.cache_need()], 4, 16, 2, 64, dtype=dtype, device=torch.device(DEV))
    batch = one_step_batch(cache, [n], torch.device(DEV))
    view = cache.view(0)
    view.block_table = batch.block_tables[0]
    h0 = torch.randn(n, H)
    hidden, delta = block.forward(h0.to(DEV).clone(), None, batch, view)
    delta = delta.float().sum(dim=0) if delta.dim() == 3 else delta.float()
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "rms_norm_eps": eps, "rope_theta": 1e4}
    named = {"model.layers.0." + k: v for k, v in w.items()}
    want = plain_model.decoder_layer(h0, named, 0, cfg, list(range(n)))
    close(hidden + delta, want, dtype)


def register_more_toy_parts():
    """A feed-forward with routing (top-1 of three tiny experts) and a position encoding with
    angles of its own, both defined here and used through the public registry only."""
    from spyinfer_b200.parts import FeedForward, PositionEncoding, register_part
    from spyinfer_b200.weights import WeightDecl

    @register_part("toy_routed_ffn")
    class ToyRoutedFFN(FeedForward):
        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.h, self.i, self.e = params["hidden_size"], params["intermediate_size"], params["experts"]
            self.w = {}

        def weight_decls(self):
            d = [WeightDecl("moe.router.weight", (self.e, self.h))]
            for k in range(self.e):
                d += [WeightDecl(f"moe.experts.{k}.in.weight", (self.i, self.h)), WeightDecl(f"moe.experts.{k}.out.weight", (self.h, self.i))]
            return d

        def bind(self, tensors):
            self.w = {k: v.float() for k, v in tensors.items()}

        def forward(self, x):
            xf = x.float()
            logits = xf @ self.w["moe.router.weight"].t()                      # router logits in 32-bit
            prob = torch.softmax(logits, dim=-1)
            pick = prob.argmax(dim=-1)
            out = torch.zeros_like(xf)
            for k in range(self.e):
                rows = (pick == k).nonzero().squeeze(-1)
                if rows.numel():
                    hid = torch.relu(xf[rows] @ self.w[f"moe.experts.{k}.in.weight"].t())
                    out[rows] = (hid @ self.w[f"moe.experts.{k}.out.weight"].t()) * prob[rows, k:k + 1]
            return out.to(x.dtype)

    @register_part("toy_linear_angles")
    class ToyLinearAngles(PositionEncoding):
        def rotation_table(self):
            r = self.params["rotary_dim"] // 2
            pos = torch.arange(self.ctx.max_model_len, dtype=torch.float32)[:, None]
            angle = pos * (torch.arange(r, dtype=torch.float32)[None, :] + 1.0) * self.params["step"]
            return torch.stack([torch.cos(angle), torch.sin(angle)], dim=-1).contiguous().to(self.ctx.device)


def test_toy_routed_feed_forward_and_toy_position_encoding():
    """Two layers with different feed-forwards and different position encodings, none of them
    known to the package: built from a description, stepped whole and in portions, and compared
    with a plain statement of the same model."""
    from spyinfer_b200.config import EngineConfig, LayerSpec, ModelSpec, PartSpec, RunEntry
    from spyinfer_b200.engine import Model, ModelRunner, StepEntry
    from spyinfer_b200.weights import random_tensors
    register_more_toy_parts()
    H, V, nh, nkv, hd, I, E, step = 64, 113, 4, 1, 32, 48, 3, 0.013
    norm = lambda name: PartSpec("rms_norm", {"size": H, "eps": 1e-6, "weight": name})
    attn = lambda pos: PartSpec("attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qk_norm_eps": None,
                                              "position": pos, "window": None, "scale": 0.2, "prefix": "self_attn."})
    layers = [
        LayerSpec("pre_norm", norm("input_layernorm.weight"), attn(PartSpec("toy_linear_angles", {"rotary_dim": hd, "step": step})),
                  norm("post_attention_layernorm.weight"), PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu",
                                                                                  "prefix": "mlp."}), "model.layers.0."),
        LayerSpec("pre_norm", norm("input_layernorm.weight"), attn(None), norm("post_attention_layernorm.weight"),
                  PartSpec("toy_routed_ffn", {"hidden_size": H, "intermediate_size": I, "experts": E}), "model.layers.1."),
    ]
    spec = ModelSpec(architecture="toy2", hidden_size=H, vocab_size=V,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight": "model.embed_tokens.weight"}),
                     layers=layers, run_order=[RunEntry(0), RunEntry(1)], final_norm=norm("model.norm.weight"),
                     head=PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": False, "weight": "lm_head.weight",
                                               "tied_to": "model.embed_tokens.weight"}), max_position=128)
    cfg = EngineConfig(dtype="float32", max_num_seqs=2, max_model_len=64, kvcache_block_size=8, num_kvcache_blocks=16, max_num_batched_tokens=64)
    model = Model(spec, torch.float32, cfg.device, cfg.max_model_len)
    w = dict(random_tensors(model.weight_decls(), seed=8, std=0.15, norm_std=0.1))
    model.bind({k: v.to(DEV) for k, v in w.items()})
    runner = ModelRunner(model, cfg)
    tokens = np.random.default_rng(1).integers(0, V, 27).tolist()

    # plain statement
    T, pos = len(tokens), list(range(len(tokens)))
    h = plain_model.embed_tokens(w["model.embed_tokens.weight"], tokens)
    for layer in range(2):
        p = f"model.layers.{layer}."
        n = plain_model.rms_norm(h, w[p + "input_layernorm.weight"], 1e-6)
        q = plain_model.linear(n, w[p + "self_attn.q_proj.weight"]).reshape(T, nh, hd)
        k = plain_model.linear(n, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd)
        v = plain_model.linear(n, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
        if layer == 0:
            angle = torch.tensor(pos, dtype=torch.float32)[:, None] * (torch.arange(hd // 2, dtype=torch.float32)[None, :] + 1.0) * step
            q, k = plain_model.rotate_half(q, torch.cos(angle), torch.sin(angle)), plain_model.rotate_half(k, torch.cos(angle), torch.sin(angle))
        o = plain_model.causal_attention(q * (0.2 * math.sqrt(hd)), k, v, pos)          # the part's scale 0.2 replaces 1/sqrt(hd)
        h = h + plain_model.linear(o.reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"])
        n = plain_model.rms_norm(h, w[p + "post_attention_layernorm.weight"], 1e-6)
        if layer == 0:
            h = h + plain_model.feed_forward(n, w, p)
        else:
            prob = torch.softmax(n @ w[p + "moe.router.weight"].float().t(), dim=-1)
            pick = prob.argmax(dim=-1)
            rows = []
            for t in range(T):
                e = int(pick[t])
                hid = torch.relu(w[p + f"moe.experts.{e}.in.weight"].float() @ n[t])
                rows.append((w[p + f"moe.experts.{e}.out.weight"].float() @ hid) * prob[t, e])
            h = h + torch.stack(rows)
    want = plain_model.linear(plain_model.rms_norm(h, w["model.norm.weight"], 1e-6), w["lm_head.weight"])

    whole = runner.step([StepEntry("w", tokens, range(T))]).cpu()
    torch.testing.assert_close(whole, want, rtol=1e-4, atol=2e-5)
    runner.finish("w")
    cut = torch.cat([runner.step([StepEntry("c", tokens[a:b], range(b - a))]).cpu() for a, b in [(0, 10), (10, 12), (12, 13), (13, 27)]])
    torch.testing.assert_close(cut, want, rtol=1e-4, atol=2e-5)
    runner.check_status()


def register_toy_blocks():
    """Two arrangements that the engine does not have, with other roles than the usual four: norms
    after the mixer and after the feed-forward as well ("sandwich": six parts), and a layer that is
    a mixer alone ("mixer_only": two parts, no feed-forward)."""
    from spyinfer_b200.parts import Block, register_block

    @register_block("toy_sandwich")
    class Sandwich(Block):
        required = ("mixer_norm", "mixer", "post_mixer_norm", "ffn_norm", "feed_forward", "post_ffn_norm")

        def __init__(self, parts):
            super().__init__(parts)
            self.mixer.defer_output = self.feed_forward.defer_output = False     # their results are normed, not added

        def forward(self, hidden, delta, batch, cache):
            x = self.mixer_norm.forward_add(hidden, delta)
            a = self.post_mixer_norm.forward(self.mixer.forward(x, batch, cache), out_dtype=torch.float32)
            x = self.ffn_norm.forward_add(hidden, a)
            return hidden, self.post_ffn_norm.forward(self.feed_forward.forward(x), out_dtype=torch.float32)

    @register_block("toy_mixer_only")
    class MixerOnly(Block):
        required = ("mixer_norm", "mixer")

        def forward(self, hidden, delta, batch, cache):
            x = self.mixer_norm.forward_add(hidden, delta)
            return hidden, self.mixer.forward(x, batch, cache)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_arrangements_with_other_roles_are_registered_built_and_stepped(dtype):
    """A layer with six parts and a layer with two, arranged by blocks defined here: the layer
    description carries the further roles, the model builds, declares the weights of and binds
    whatever parts a layer has, and a layer without a feed-forward or with two more norms steps
    through the engine, whole and cut, as the plain statement of the same arrangement does."""
    from spyinfer_b200.config import EngineConfig, LayerSpec, ModelSpec, PartSpec, RunEntry
    from spyinfer_b200.engine import Model, ModelRunner, StepEntry
    from spyinfer_b200.weights import random_tensors
    register_toy_blocks()
    H, V, nh, nkv, hd, eps = 64, 131, 2, 1, 64, 1e-5
    norm = lambda name: PartSpec("rms_norm", {"size": H, "eps": eps, "weight": name})
    attn = PartSpec("attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qk_norm_eps": eps,
                                  "position": PartSpec("rotary_half", {"theta": 1e4, "rotary_dim": hd}), "window": None, "scale": None, "prefix": "self_attn."})
    ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": 96, "activation": "silu", "prefix": "mlp."})
    layers = [LayerSpec("toy_sandwich", mixer_norm=norm("input_layernorm.weight"), mixer=attn, ffn_norm=norm("pre_feedforward_layernorm.weight"),
                        feed_forward=ffn, weight_prefix="model.layers.0.",
                        more={"post_mixer_norm": norm("post_attention_layernorm.weight"), "post_ffn_norm": norm("post_feedforward_layernorm.weight")}),
              LayerSpec("toy_mixer_only", mixer_norm=norm("input_layernorm.weight"), mixer=attn, weight_prefix="model.layers.1.")]
    spec = ModelSpec(architecture="toy", hidden_size=H, vocab_size=V,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight": "model.embed_tokens.weight"}),
                     layers=layers, run_order=[RunEntry(0), RunEntry(1)], final_norm=norm("model.norm.weight"),
                     head=PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": False, "weight": "lm_head.weight",
                                               "tied_to": "model.embed_tokens.weight"}), max_position=256)
    with pytest.raises(ValueError, match="missing.*post_ffn_norm"):
        Model(ModelSpec(**{**spec.__dict__, "layers": [LayerSpec("toy_sandwich", norm("a"), attn, norm("b"), ffn, "model.layers.0.",
                                                                 more={"post_mixer_norm": norm("c")})], "run_order": [RunEntry(0)]}),
              torch.float32, DEV, 64)
    tdtype = torch.float32 if dtype == "float32" else torch.bfloat16
    cfg = EngineConfig(dtype=dtype, max_num_seqs=2, max_model_len=64, kvcache_block_size=16, num_kvcache_blocks=8, max_num_batched_tokens=64)
    model = Model(spec, tdtype, cfg.device, cfg.max_model_len)
    names = {d.name for d in model.weight_decls()}
    assert "model.layers.0.post_feedforward_layernorm.weight" in names and "model.layers.1.mlp.down_proj.weight" not in names
    w = dict(random_tensors(model.weight_decls(), seed=9, std=0.08, norm_std=0.1))
    model.bind({k: v.to(DEV) for k, v in w.items()})
    runner = ModelRunner(model, cfg)
    tokens = np.random.default_rng(1).integers(0, V, 23).tolist()
    cfgd = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "rms_norm_eps": eps, "rope_theta": 1e4}
    pos = list(range(len(tokens)))
    h = plain_model.embed_tokens(w["model.embed_tokens.weight"], tokens)
    p = "model.layers.0."
    a = plain_model.attention_mixer(plain_model.rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p, cfgd, pos)
    h = h + plain_model.rms_norm(a, w[p + "post_attention_layernorm.weight"], eps)
    f = plain_model.feed_forward(plain_model.rms_norm(h, w[p + "pre_feedforward_layernorm.weight"], eps), w, p)
    h = h + plain_model.rms_norm(f, w[p + "post_feedforward_layernorm.weight"], eps)
    p = "model.layers.1."
    h = h + plain_model.attention_mixer(plain_model.rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p, cfgd, pos)
    want = plain_model.linear(plain_model.rms_norm(h, w["model.norm.weight"], eps), w["lm_head.weight"])
    tol = dict(rtol=1e-4, atol=1e-5) if dtype == "float32" else dict(rtol=0.0, atol=0.05 * want.abs().max().item())
    whole = runner.step([StepEntry("w", tokens, range(len(tokens)))]).cpu()
    torch.testing.assert_close(whole, want, **tol)
    cut = torch.cat([runner.step([StepEntry("c", tokens[a:b], range(b - a))]).cpu() for a, b in [(0, 9), (9, 11), (11, 12), (12, 23)]])
    torch.testing.assert_close(cut, want, **tol)
    runner.check_status()


def test_a_whole_architecture_from_this_file_generates_through_the_scheduler_and_survives_preemption(tmp_path):
    """An architecture registered here (its own config.json keys, its own mixer with per-request state
    beside an attention layer) is written as a model folder, read back by name, and generates through
    ``LLMEngine``: with room, and in a pool so small that requests are preempted and recomputed, where
    the state slot of a recomputed request must start from zero again; launching decode steps ahead
    changes nothing.  No file of the framework knows this architecture."""
    import json
    from dataclasses import dataclass

    from spyinfer_b200 import LLMEngine, SamplingParams
    from spyinfer_b200.config import ArchitectureConfig, ConfigError, load_model_config, register_architecture
    from spyinfer_b200.weights import write_model_folder
    register_toy_parts()

    @register_architecture("ToyDecayForCausalLM", model_type="toy_decay")
    @dataclass
    class ToyConfig(ArchitectureConfig):
        decay_layers: int = 2

        @classmethod
        def from_json(cls, data):
            if data.get("decay_layers") != 2:
                raise ConfigError("toy: decay_layers must be 2")
            return cls(decay_layers=2)

        def to_json(self):
            return {"architectures": [self.architecture], "model_type": "toy_decay", "decay_layers": self.decay_layers}

        def to_spec(self):
            return toy_spec()

    write_model_folder(str(tmp_path), ToyConfig(), seed=6, std=0.1, norm_std=0.1)
    assert isinstance(load_model_config(str(tmp_path)), ToyConfig)
    rng = np.random.default_rng(4)
    prompts = [rng.integers(0, 97, n).tolist() for n in (17, 9, 30, 5)]
    sp = SamplingParams(max_new_tokens=20, ignore_eos=True)
    opts = dict(dtype="float32", max_num_seqs=3, max_model_len=128, kvcache_block_size=8, max_num_batched_tokens=24)
    roomy = LLMEngine(str(tmp_path), num_kvcache_blocks=48, **opts)
    want = roomy.generate(prompts, sp)
    from safetensors.torch import load_file
    w = load_file(str(tmp_path / "model.safetensors"))
    for p, o in zip(prompts, want):                                         # greedy tokens of the plain statement of this architecture
        seq = list(p)
        for tok in o[:4]:
            logits = plain_toy_logits(w, seq)[-1]
            assert logits[tok] >= logits.max() - 1e-4
            seq.append(tok)
    for ahead in (True, False):
        tight = LLMEngine(str(tmp_path), num_kvcache_blocks=9, lookahead_decode=ahead, **opts)       # 72 tokens of cache for requests of up to 50
        assert tight.generate(prompts, sp) == want
        assert tight.scheduler.num_preemptions > 0, "the pool was meant to be too small"
        tight.runner.cache.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_interleaved_pairs_and_scaled_frequencies_are_parameters_of_the_rotary_part(dtype):
    """``rotary_interleaved`` (angle j turns the pair (2j, 2j + 1)) with ``frequency_scale`` 4 on one layer and
    ``rotary_half`` with explicit ``inverse_frequencies`` on the other, at head size 128, where the
    bfloat16 path has a kernel of its own for the usual rule and must not take it for the other one."""
    from spyinfer_b200.config import EngineConfig, LayerSpec, ModelSpec, PartSpec, RunEntry
    from spyinfer_b200.engine import Model, ModelRunner, StepEntry
    from spyinfer_b200.weights import random_tensors
    H, V, nh, nkv, hd, I, eps, theta = 128, 211, 2, 1, 128, 96, 1e-6, 5000.0
    given = [0.5 / (j + 1) for j in range(hd // 2)]
    norm = lambda name: PartSpec("rms_norm", {"size": H, "eps": eps, "weight": name})
    attn = lambda pos: PartSpec("attention", {"hidden_size": H, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qk_norm_eps": eps,
                                              "position": pos, "window": None, "scale": None, "prefix": "self_attn."})
    ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu", "prefix": "mlp."})
    layers = [LayerSpec("pre_norm", norm("input_layernorm.weight"), attn(PartSpec("rotary_interleaved", {"theta": theta, "rotary_dim": hd, "frequency_scale": 4.0})),
                        norm("post_attention_layernorm.weight"), ffn, "model.layers.0."),
              LayerSpec("pre_norm", norm("input_layernorm.weight"), attn(PartSpec("rotary_half", {"theta": theta, "rotary_dim": hd, "inverse_frequencies": given})),
                        norm("post_attention_layernorm.weight"), ffn, "model.layers.1.")]
    spec = ModelSpec(architecture="toy3", hidden_size=H, vocab_size=V,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "hidden_size": H, "weight": "model.embed_tokens.weight"}),
                     layers=layers, run_order=[RunEntry(0), RunEntry(1)], final_norm=norm("model.norm.weight"),
                     head=PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "tied": True, "weight": "lm_head.weight",
                                               "tied_to": "model.embed_tokens.weight"}), max_position=128)
    cfg = EngineConfig(dtype=dtype, max_num_seqs=2, max_model_len=64, kvcache_block_size=16, num_kvcache_blocks=8, max_num_batched_tokens=64)
    model = Model(spec, torch.float32 if dtype == "float32" else torch.bfloat16, cfg.device, cfg.max_model_len)
    w = dict(random_tensors(model.weight_decls(), seed=12, std=0.08, norm_std=0.1))
    model.bind({k: v.to(DEV) for k, v in w.items()})
    runner = ModelRunner(model, cfg)
    tokens = np.random.default_rng(2).integers(0, V, 29).tolist()
    T, pos = len(tokens), torch.arange(len(tokens), dtype=torch.float32)

    def turn(x, angle, interleaved):                        # x [T, heads, hd]
        c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
        if interleaved:
            lo, hi = x[..., 0::2], x[..., 1::2]
            return torch.stack([lo * c - hi * s, lo * s + hi * c], dim=-1).flatten(-2)
        return plain_model.rotate_half(x, torch.cos(angle), torch.sin(angle))

    h = plain_model.embed_tokens(w["model.embed_tokens.weight"], tokens)
    for layer in range(2):
        p = f"model.layers.{layer}."
        n = plain_model.rms_norm(h, w[p + "input_layernorm.weight"], eps)
        if layer == 0:
            inv = torch.pow(torch.tensor(theta), -torch.arange(hd // 2, dtype=torch.float32) / (hd // 2)) / 4.0
        else:
            inv = torch.tensor(given, dtype=torch.float32)
        angle = pos[:, None] * inv[None, :]
        q = turn(plain_model.rms_norm(plain_model.linear(n, w[p + "self_attn.q_proj.weight"]).reshape(T, nh, hd), w[p + "self_attn.q_norm.weight"], eps), angle, layer == 0)
        k = turn(plain_model.rms_norm(plain_model.linear(n, w[p + "self_attn.k_proj.weight"]).reshape(T, nkv, hd), w[p + "self_attn.k_norm.weight"], eps), angle, layer == 0)
        v = plain_model.linear(n, w[p + "self_attn.v_proj.weight"]).reshape(T, nkv, hd)
        o = plain_model.causal_attention(q, k, v, list(range(T)))
        h = h + plain_model.linear(o.reshape(T, nh * hd), w[p + "self_attn.o_proj.weight"])
        h = h + plain_model.feed_forward(plain_model.rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p)
    want = plain_model.linear(plain_model.rms_norm(h, w["model.norm.weight"], eps), w["model.embed_tokens.weight"])
    tol = dict(rtol=1e-4, atol=2e-5) if dtype == "float32" else dict(rtol=0.0, atol=0.05 * want.abs().max().item())
    whole = runner.step([StepEntry("w", tokens, range(T))]).cpu()
    torch.testing.assert_close(whole, want, **tol)
    cut = torch.cat([runner.step([StepEntry("c", tokens[a:b], range(b - a))]).cpu() for a, b in [(0, 11), (11, 13), (13, 14), (14, 29)]])
    torch.testing.assert_close(cut, want, **tol)
    runner.check_status()
