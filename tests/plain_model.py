"""Plain, slow restatement of the Qwen3 dense decoder for tests.

Whole sequences, no cache, no batching, one function for each part.  It shares no
code with the package under test: weights come in as a ``{tensor name: torch.Tensor}``
dictionary with the checkpoint's own names, sizes come in as a plain ``dict`` with
config.json's keys.  All arithmetic is done in the dtype of ``compute`` (float32 as
in the reference's CPU path, or float64 when a test wants a tighter oracle).

Every function cites the place in spymaster2h/spyinfer whose formula it restates
(paths relative to that project's root).  The comparison of this file with the
reference's own compiled CPU path is recorded under ``tests/golden``.
"""
from __future__ import annotations

import math

import torch


def embed_tokens(table: torch.Tensor, token_ids, compute=torch.float32) -> torch.Tensor:
    """Row gather without scaling: ``h[t] = E[ids[t]]``.

    src/backends/cpu/cpu_operator.cpp:258-264 (row copy, bf16 widened to fp32);
    src/models/qwen3.hpp:114-119.
    """
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    return table.to(compute)[ids]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * (1/sqrt(mean(x^2) + eps)) * weight`` over the last axis; plain weight, no bias.

    src/backends/cpu/x64/kernels.cpp:168-180.
    """
    w = weight.to(x.dtype)
    mean_sq = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return (1.0 / torch.sqrt(mean_sq + eps)) * x * w


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``y = x @ W^T`` with ``W [out, in]``; no bias is ever bound.

    src/backends/cpu/x64/kernels.cpp:95-166; src/models/qwen3.hpp:138-158.
    """
    return x @ weight.to(x.dtype).t()


def rotary_angles(positions, head_dim: int, theta: float, compute=torch.float32):
    """Table of rotate-half angles: ``freq_j = theta^(-j/(hd/2))``, ``angle = pos * freq_j``.

    src/utils/constant_table.hpp:28-41.  The reference evaluates ``pow`` and the product
    in 32-bit floats; so does this function when ``compute`` is float32.
    """
    half = head_dim // 2
    j = torch.arange(half, dtype=compute)
    freq = torch.pow(torch.tensor(float(theta), dtype=compute), -j / float(half))
    pos = torch.as_tensor(positions, dtype=compute)
    angle = pos[:, None] * freq[None, :]
    return torch.cos(angle), torch.sin(angle)


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Pairs ``(j, j + hd/2)``: ``x'_j = x_j cos - x_{j+r} sin``, ``x'_{j+r} = x_j sin + x_{j+r} cos``.

    ``x`` is ``[T, heads, hd]``; ``cos``/``sin`` are ``[T, hd/2]``.
    src/backends/cpu/cpu_operator.cpp:397-408.
    """
    r = x.shape[-1] // 2
    lo, hi = x[..., :r], x[..., r:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([lo * c - hi * s, lo * s + hi * c], dim=-1)


def causal_attention(q, k, v, positions, window=None) -> torch.Tensor:
    """Softmax attention of one sequence, grouped heads, causal on absolute positions.

    ``q [T, nh, hd]``, ``k, v [T, nkv, hd]`` (T = the whole sequence, position t = t).
    ``kv head = h * nkv // nh``; ``score = (q . k) / sqrt(hd)``; keys after the query's
    position are masked; ``p = exp(score - max) / sum``; ``o = sum p v``.
    src/backends/cpu/cpu_attention.cpp:59 (scale), :96 (head map), :100-110 (mask, score),
    :113-124 (softmax), :126-135 (PV).

    ``window`` (not in the reference, whose layers all see every key) limits a query at
    position p to the keys ``p - window < j <= p``; it is here for the engine's
    windowed-cache tests.
    """
    T, nh, hd = q.shape
    nkv = k.shape[1]
    scale = 1.0 / math.sqrt(float(hd))
    pos = torch.as_tensor(positions, dtype=torch.long)
    out = torch.zeros_like(q)
    for h in range(nh):
        kvh = h * nkv // nh
        scores = (q[:, h, :] @ k[:, kvh, :].t()) * scale  # [T, T]
        key_pos = pos[None, :]
        masked = key_pos > pos[:, None]
        if window is not None:
            masked = masked | (key_pos <= pos[:, None] - int(window))
        scores = scores.masked_fill(masked, float("-inf"))
        scores = scores - scores.max(dim=-1, keepdim=True).values
        p = torch.exp(scores)
        p = p / p.sum(dim=-1, keepdim=True)
        out[:, h, :] = p @ v[:, kvh, :]
    return out


def attention_mixer(x, w, prefix, cfg, positions, window=None):
    """q/k/v projections, per-head q/k RMSNorm, rotate-half RoPE, attention, output projection.

    src/models/qwen3.hpp:136-213 in that order: three linears (138-158), RMSNorm over
    head_dim with one shared weight and the model's eps on q and k, not v (161-180),
    RoPE on q and k (183-194), attention (197-205), o_proj (207-213).  The reference's model has
    bias slots for q, k and v that it never binds (:39, 143, 150, 157); where the weights hold
    ``{q,k,v}_proj.bias`` they are added to the projections (``y = x W^T + b``,
    src/backends/cpu/cpu_operator.cpp:150-186).
    """
    T = x.shape[0]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]

    def projected(name):
        y = linear(x, w[prefix + f"self_attn.{name}_proj.weight"])
        b = w.get(prefix + f"self_attn.{name}_proj.bias")
        return y if b is None else y + b.to(y.dtype)

    q = projected("q").reshape(T, nh, hd)
    k = projected("k").reshape(T, nkv, hd)
    v = projected("v").reshape(T, nkv, hd)
    q = rms_norm(q, w[prefix + "self_attn.q_norm.weight"], cfg["rms_norm_eps"])
    k = rms_norm(k, w[prefix + "self_attn.k_norm.weight"], cfg["rms_norm_eps"])
    cos, sin = rotary_angles(positions, hd, cfg["rope_theta"], compute=x.dtype)
    q = rotate_half(q, cos, sin)
    k = rotate_half(k, cos, sin)
    o = causal_attention(q, k, v, positions, window=window)
    return linear(o.reshape(T, nh * hd), w[prefix + "self_attn.o_proj.weight"])


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` with ``silu(g) = g / (1 + exp(-g))``.

    src/backends/cpu/x64/kernels.cpp:242-247 (scalar tail; the vector lanes use a
    polynomial exp of the same function, :229-240).
    """
    return (gate / (1.0 + torch.exp(-gate))) * up


def feed_forward(x, w, prefix):
    """gate and up projections, SwiGLU, down projection; no biases.

    src/models/qwen3.hpp:233-263.
    """
    g = linear(x, w[prefix + "mlp.gate_proj.weight"])
    u = linear(x, w[prefix + "mlp.up_proj.weight"])
    return linear(swiglu(g, u), w[prefix + "mlp.down_proj.weight"])


def decoder_layer(h, w, layer, cfg, positions, window=None):
    """Pre-norm block: ``h += attn(norm(h))``; ``h += ffn(norm(h))``.

    src/models/qwen3.hpp:127-133 (input norm), 216-221 (residual), 224-230 (post-attention
    norm), 272-277 (residual).
    """
    prefix = f"model.layers.{layer}."
    n = rms_norm(h, w[prefix + "input_layernorm.weight"], cfg["rms_norm_eps"])
    h = h + attention_mixer(n, w, prefix, cfg, positions, window=window)
    n = rms_norm(h, w[prefix + "post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    h = h + feed_forward(n, w, prefix)
    return h


def layer_windows(cfg):
    """Window of each layer, ``None`` for a layer that sees every key.

    The reference reads no window key (src/models/model_config.hpp:27-47): all layers are
    full attention.  The engine under test also takes ``use_sliding_window`` and
    ``sliding_window`` from config.json, with the layers that have the window named either
    by ``layer_types`` (``"sliding_attention"``) or by ``max_window_layers`` (the first
    ``max_window_layers`` layers see every key, the others have the window).  Stated here
    layer by layer, on its own, so that a different reading in the engine shows.
    """
    out = []
    for i in range(cfg["num_hidden_layers"]):
        windowed = False
        if cfg.get("use_sliding_window", False):
            if cfg.get("layer_types") is not None:
                windowed = cfg["layer_types"][i] == "sliding_attention"
            else:
                windowed = i + 1 > cfg["max_window_layers"]
        out.append(cfg["sliding_window"] if windowed else None)
    return out


def forward_logits(w, cfg, token_ids, compute=torch.float32) -> torch.Tensor:
    """Logits ``[T, vocab]`` of one whole sequence.

    src/models/qwen3.hpp:93-281 (forward), 283-308 (final norm and head); the head is the
    embedding table when ``tie_word_embeddings`` (qwen3.hpp:46).
    """
    cfg = dict(cfg)
    cfg.setdefault("head_dim", cfg["hidden_size"] // cfg["num_attention_heads"])
    cfg.setdefault("rope_theta", 1000000.0)
    cfg.setdefault("rms_norm_eps", 1e-6)
    positions = list(range(len(token_ids)))
    h = embed_tokens(w["model.embed_tokens.weight"], token_ids, compute)
    windows = layer_windows(cfg)
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, layer, cfg, positions, window=windows[layer])
    h = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return linear(h, head)


def greedy_generate(w, cfg, prompt, new_tokens: int, compute=torch.float32):
    """Greedy continuation by re-running the whole sequence for each token.

    argmax of the last row's logits, lowest index on ties: src/engine/model_runner.cpp:120-134.
    """
    tokens = list(prompt)
    for _ in range(new_tokens):
        logits = forward_logits(w, cfg, tokens, compute)
        tokens.append(int(torch.argmax(logits[-1]).item()))
    return tokens[len(prompt):]


def softmax_probabilities(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """``softmax(logits / temperature)``: the distribution temperature sampling draws from."""
    z = logits.to(torch.float64) / float(temperature)
    z = z - z.max(dim=-1, keepdim=True).values
    p = torch.exp(z)
    return p / p.sum(dim=-1, keepdim=True)


def top_k_probabilities(logits: torch.Tensor, temperature: float, top_k: int) -> torch.Tensor:
    """``softmax(logits / temperature)`` over the ``top_k`` largest logits (those equal to the
    k-th largest all stay), zero elsewhere.  The reference has no such sampler; this is the
    usual definition, written out for the engine's own option."""
    z = logits.to(torch.float64)
    kth = torch.sort(z, descending=True).values[..., top_k - 1]
    z = torch.where(z >= kth.unsqueeze(-1), z, torch.full_like(z, float("-inf")))
    return softmax_probabilities(z, temperature)


def random_weights(cfg, seed: int, std: float = 0.02, norm_std: float = 0.05):
    """Seeded bf16 weights with the checkpoint's tensor names: linears and embeddings
    ``N(0, std)``, norm weights ``1 + N(0, norm_std)``.  Independent of the package's own
    random-weights mode."""
    g = torch.Generator().manual_seed(seed)
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim", H // nh)
    V = cfg["vocab_size"]

    def lin(*shape):
        return (torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def norm(n):
        return (1.0 + torch.randn(n, generator=g) * norm_std).to(torch.bfloat16)

    w = {"model.embed_tokens.weight": lin(V, H)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        w[p + "input_layernorm.weight"] = norm(H)
        w[p + "self_attn.q_proj.weight"] = lin(nh * hd, H)
        w[p + "self_attn.k_proj.weight"] = lin(nkv * hd, H)
        w[p + "self_attn.v_proj.weight"] = lin(nkv * hd, H)
        w[p + "self_attn.o_proj.weight"] = lin(H, nh * hd)
        w[p + "self_attn.q_norm.weight"] = norm(hd)
        w[p + "self_attn.k_norm.weight"] = norm(hd)
        if cfg.get("attention_bias", False):
            w[p + "self_attn.q_proj.bias"] = lin(nh * hd) * 10.0
            w[p + "self_attn.k_proj.bias"] = lin(nkv * hd) * 10.0
            w[p + "self_attn.v_proj.bias"] = lin(nkv * hd) * 10.0
        w[p + "post_attention_layernorm.weight"] = norm(H)
        w[p + "mlp.gate_proj.weight"] = lin(I, H)
        w[p + "mlp.up_proj.weight"] = lin(I, H)
        w[p + "mlp.down_proj.weight"] = lin(H, I)
    w["model.norm.weight"] = norm(H)
    if not cfg.get("tie_word_embeddings", False):
        w["lm_head.weight"] = lin(V, H)
    return w
