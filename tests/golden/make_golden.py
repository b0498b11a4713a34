#!/usr/bin/env python3
"""Makes the golden logits under tests/golden from the reference's own CPU model code.

It compiles ``reference_harness.cpp`` against the sources of spymaster2h/spyinfer (its CPU
backend needs AVX-512 and the single header nlohmann/json.hpp), writes two tiny seeded
random models with ``tests/plain_model.random_weights``, runs every request whole and
again cut into portions and mixed with other requests, and stores

* ``<name>.json``: config.json's content, seed, weight scales, the prompts, and the largest
  difference between the whole and the cut/mixed run of the reference (0.0: its CPU path
  computes each token independently of the batch);
* ``<name>.logits.f32``: the reference's logits for every prompt token of every request,
  whole runs, requests in order, float32 ``[sum of lengths, vocab]``.

``tests/test_plain_vs_reference.py`` rebuilds the same weights from the seed and compares
``tests/plain_model.forward_logits`` with these files.

usage: python tests/golden/make_golden.py --reference /path/to/spyinfer [--json-include DIR]
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_model  # noqa: E402

CASES = {
    "tiny_a": {
        "config": {
            "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
            "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
            "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
            "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 128,
            "bos_token_id": 1, "eos_token_id": 2,
        },
        "seed": 1234, "std": 0.02, "norm_std": 0.05, "block_size": 4, "prompt_lengths": [5, 9, 13], "portion": 3,
    },
    "tiny_b": {
        "config": {
            "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu",
            "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 8, "num_key_value_heads": 2,
            "head_dim": 32, "intermediate_size": 224, "vocab_size": 384, "rope_theta": 1000000.0,
            "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "max_position_embeddings": 256,
            "bos_token_id": 1, "eos_token_id": 2,
        },
        "seed": 4321, "std": 0.03, "norm_std": 0.1, "block_size": 8, "prompt_lengths": [1, 7, 16, 31], "portion": 5,
    },
}


def make_prompts(case):
    g = torch.Generator().manual_seed(case["seed"] + 1)
    return [torch.randint(0, case["config"]["vocab_size"], (n,), generator=g).tolist() for n in case["prompt_lengths"]]


def step_line(entries, tables, block_size):
    """entries: list of (request index, start, tokens).  One plan line for the harness."""
    tokens, positions, slots, seq_idx, ctx_lens = [], [], [], [], []
    max_blocks = max(len(tables[r]) for r, _, _ in entries)
    flat_tables = []
    for s, (r, start, toks) in enumerate(entries):
        for i, t in enumerate(toks):
            p = start + i
            tokens.append(t)
            positions.append(p)
            slots.append(tables[r][p // block_size] * block_size + p % block_size)
            seq_idx.append(s)
        ctx_lens.append(start + len(toks))
        flat_tables += tables[r] + [-1] * (max_blocks - len(tables[r]))
    fields = [tokens, positions, slots, seq_idx, ctx_lens, [max_blocks], flat_tables]
    return " | ".join(" ".join(str(v) for v in f) for f in fields)


def build_plans(case, prompts):
    bs = case["block_size"]
    tables, nxt = [], 0
    for p in prompts:
        n = (len(p) + bs - 1) // bs
        tables.append(list(range(nxt, nxt + n)))
        nxt += n
    whole = [step_line([(r, 0, p)], tables, bs) for r, p in enumerate(prompts)]
    whole_rows = [(r, i) for r, p in enumerate(prompts) for i in range(len(p))]
    # cut and mixed: every step takes the next portion of every unfinished request, the
    # portion shrinking from `portion` down to one token, entries in rotating order
    mixed, mixed_rows = [], []
    done = [0] * len(prompts)
    step = 0
    while any(d < len(p) for d, p in zip(done, prompts)):
        size = max(1, case["portion"] - step % case["portion"])
        order = [r for r in range(len(prompts)) if done[r] < len(prompts[r])]
        order = order[step % len(order):] + order[:step % len(order)]
        entries = []
        for r in order:
            toks = prompts[r][done[r]:done[r] + size]
            entries.append((r, done[r], toks))
            mixed_rows += [(r, done[r] + i) for i in range(len(toks))]
            done[r] += len(toks)
        mixed.append(step_line(entries, tables, bs))
        step += 1
    return nxt, whole, whole_rows, mixed, mixed_rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the spymaster2h/spyinfer sources")
    ap.add_argument("--json-include", default=None, help="a directory that holds nlohmann/json.hpp")
    args = ap.parse_args()
    inc = args.json_include
    if inc is None:
        hits = glob.glob(os.path.join(sys.prefix, "lib/python*/site-packages/include/cudnn_frontend/thirdparty"))
        inc = hits[0] if hits else "/usr/include"
    ref = args.reference
    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "reference_harness")
        srcs = [os.path.join(HERE, "reference_harness.cpp")]
        for pat in ("src/backends/cpu/*.cpp", "src/backends/cpu/x64/*.cpp", "src/core/*.cpp", "src/utils/context.cpp",
                    "src/utils/safetensors_reader.cpp"):
            srcs += sorted(glob.glob(os.path.join(ref, pat)))
        cmd = ["g++", "-std=c++20", "-O2", "-mavx512f", "-mavx512bw", "-mavx512dq", "-mfma", "-I", os.path.join(ref, "src"), "-I", inc,
               "-o", exe, "-pthread"] + srcs
        print("compiling the reference's CPU path ...", flush=True)
        subprocess.run(cmd, check=True)
        for name, case in CASES.items():
            cfg = case["config"]
            model_dir = os.path.join(tmp, name)
            os.makedirs(model_dir)
            with open(os.path.join(model_dir, "config.json"), "w") as f:
                json.dump(cfg, f)
            weights = plain_model.random_weights(cfg, case["seed"], case["std"], case["norm_std"])
            save_file({k: v.contiguous() for k, v in weights.items()}, os.path.join(model_dir, "model.safetensors"))
            prompts = make_prompts(case)
            blocks, whole, whole_rows, mixed, mixed_rows = build_plans(case, prompts)
            results = {}
            for tag, lines in (("whole", whole), ("mixed", mixed)):
                plan = os.path.join(tmp, f"{name}.{tag}.plan")
                with open(plan, "w") as f:
                    f.write(f"{case['block_size']} {blocks}\n" + "\n".join(lines) + "\n")
                out = os.path.join(tmp, f"{name}.{tag}.f32")
                subprocess.run([exe, model_dir, plan, out], check=True, stdout=subprocess.DEVNULL)
                results[tag] = np.fromfile(out, dtype="<f4").reshape(-1, cfg["vocab_size"])
            by_row = {row: results["mixed"][i] for i, row in enumerate(mixed_rows)}
            cut_diff = max(float(np.abs(by_row[row] - results["whole"][i]).max()) for i, row in enumerate(whole_rows))
            plain = torch.cat([plain_model.forward_logits(weights, cfg, p) for p in prompts]).numpy()
            plain_diff = float(np.abs(plain - results["whole"]).max())
            results["whole"].astype("<f4").tofile(os.path.join(HERE, f"{name}.logits.f32"))
            meta = {k: case[k] for k in ("config", "seed", "std", "norm_std", "block_size")}
            meta.update(prompts=prompts, reference_whole_vs_cut_and_mixed_max_abs_diff=cut_diff,
                        plain_vs_reference_max_abs_diff_when_made=plain_diff,
                        max_abs_logit=float(np.abs(results["whole"]).max()))
            with open(os.path.join(HERE, f"{name}.json"), "w") as f:
                json.dump(meta, f, indent=1)
            print(f"{name}: rows {results['whole'].shape[0]}, whole vs cut/mixed {cut_diff:.3g}, plain vs reference {plain_diff:.3g}")


if __name__ == "__main__":
    main()
