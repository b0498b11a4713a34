#!/usr/bin/env python3
"""Benchmark of the engine's decode step and prefill on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--shape 8b|14b|32b] [--batch B] [--context C] [--impl ours|reference]
    python bench.py --workload mixed [--shape 14b] [--requests 64] [--budget 2048]     (a continuous batch through LLMEngine; its own line)

The model has the layer sizes of Qwen3-8B (36 layers, hidden 4096, 32 query heads, 8 key/value
heads, head size 128, intermediate 12288, vocabulary 151936, untied head) with seeded random
weights in bfloat16.  A "step" is one decode step of a batch of 8 requests at a context of
8192 tokens: the step function on the live batch plus device-side sampling.  The requests'
caches are filled with random keys and values of that length (the step's work does not depend
on their content), so no prefill is timed.  One JSON line is printed:

* ``value``: decoded tokens a second, timed with CUDA events around K steps after W warm-up
  steps; between steps the inputs (weights + cache, > 20 GB) are far larger than L2;
* ``e2e``: the same through the Python entry point ``LLMEngine.step()``: every call copies
  its step's batch arrays from pinned host memory and reads a step's sampled tokens back (the
  engine launches a decode step before it has read the step before, so the tokens a call
  returns are those of the step launched by the call before it; every step's tokens are
  read, once);
* ``prefill``: one step of 2048 prompt tokens of one request; ``frac`` = flops / time / the bf16
  peak of a kernel timed alone (the burst figure), ``frac_sustained`` the same against the rate a
  seconds-long loop of products holds under the power cap;
* ``roofline``: bytes the decode step has to read (every weight it uses once, and the cache
  of the live requests) / its time, against the measured copy bandwidth;
* ``points``: tokens a second of decoding at batch 1 and 64 (same context), and at the context of
  about 640 tokens that the reference workload "prompts of 512, 256 generated tokens" averages;
  ``points_detail`` gives each of them its ``ms_per_step`` and its own ``roofline`` block;
* ``kernels``: each dominant kernel alone at the step's sizes, timed by CUDA events around a loop that
  walks through the layers' own weights (far more than L2 holds): the q|k|v, o, gate|up and down
  products and the output head at the decoding batch, at batch 64 and at 2048 tokens, the decode
  attention at batch 64 and the prompt attention at 2048 tokens, each with microseconds, achieved
  GB/s (decoding: the bytes it has to read and write) or TFLOP/s (prompt) and the fraction of the
  measured copy bandwidth or of the bf16 burst peak;
* ``clocks``: SM clocks and throttle reasons sampled with nvidia-smi during the timed region.

Peaks come from MEASURED_PEAKS.json beside this file when it exists (``hbm_gbs``, ``bf16_tflops``,
``bf16_tflops_sustained``), else 6.65 TB/s and 1.59 PFLOP/s (sustained: 1.4).  ``--gpus N`` with N > 1 prints one line saying that this engine is
single-GPU and exits with 2.  ``--impl reference`` runs the unmodified reference's CUDA decode path on the same shape,
batch, context and steps (see ``reference_arm``) and prints the same line with ``"impl": "reference"``.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": 36,
            "hidden_size": 4096, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
            "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
            "max_position_embeddings": 40960, "eos_token_id": 151645}
# the other two benchmark shapes (same options; --shape picks one, the default is the 8B shape the metric is quoted on)
SHAPES = {
    "8b": {},
    "14b": {"num_hidden_layers": 40, "hidden_size": 5120, "num_attention_heads": 40, "intermediate_size": 17408},
    "32b": {"num_hidden_layers": 64, "hidden_size": 5120, "num_attention_heads": 64, "intermediate_size": 25600},
}


def reference_arm(args) -> int:
    """``--impl reference``: the unmodified reference on its own CUDA backend, same model shape, batch,
    context, page size and number of steps.

    spymaster2h/spyinfer is a C++/xmake project, no Python package, so it is built by hand from its
    own sources (``baseline/build_reference.py``: nvcc and the host compiler over the file list of its
    xmake target, cuBLAS) into ``baseline/_ref`` together with ``baseline/reference_decode.cpp``, which
    drives its stock ``Qwen3::forward`` and ``compute_logits`` on ``CUDABackend`` for decoding steps and
    does with the logits what its ``ModelRunner`` does (copy to the host, widen, argmax).  The model is
    a seeded random bfloat16 checkpoint of the benchmark's shape, written in shards as checkpoints of
    this size are; the reference converts it to float16 at load.  What cannot be had from it: a prompt
    step of 100 or more tokens (its scratch holds 100 rows), hence no ``prefill`` block, and batches of
    100 or more.  If the build fails the line says ``unavailable`` with the compiler's message."""
    import tempfile

    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import build_reference
        exe = build_reference.build(os.environ.get("SPYINFER_REFERENCE", build_reference.DEFAULT_REFERENCE))
    except Exception as e:                                              # noqa: BLE001: whatever stops the build is the reason
        print(json.dumps({"impl": "reference", "unavailable": "the hand build of the reference failed: " + " ".join(str(e).split())[-600:]}))
        return 0
    if args.gpus != 1:
        print(json.dumps({"impl": "reference", "unavailable": "the reference runs on one GPU (devices_[0]); --gpus %d has no meaning for it" % args.gpus}))
        return 0
    import torch

    from spyinfer_b200 import config_from_json
    from spyinfer_b200.weights import write_model_folder

    hbm_gbs, _, _, peak_src = peaks()
    cfg_json = dict(QWEN3_8B)
    cfg_json.update(SHAPES[args.shape])
    full_layers = cfg_json["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg_json["num_hidden_layers"] = layers
    c = config_from_json(cfg_json)
    H, I, V, nh, nkv, hd = c.hidden_size, c.intermediate_size, c.vocab_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim
    weight_bytes = 2 * (layers * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I) + V * H)
    kv_bytes_per_token = 2 * 2 * nkv * hd * layers
    warmup, page, ctx = max(3, args.warmup), 16, args.context
    short = 640 + (args.steps + warmup) // 2
    point_steps = min(args.steps, 10)
    works = [(args.batch, ctx, args.steps)]
    if not args.no_points:
        works += [(1, ctx, point_steps), (64, ctx, point_steps), (1, short, point_steps), (8, short, point_steps), (64, short, point_steps)]
    with tempfile.TemporaryDirectory(prefix="reference_model_") as model_dir:
        write_model_folder(model_dir, c, 0, shard_bytes=3 << 30, device="cuda:0" if torch.cuda.is_available() else "cpu")
        torch.cuda.empty_cache()
        with ClockSampler() as clocks:
            proc = subprocess.run([exe, model_dir, str(page), str(warmup)] + [f"{b}x{n}x{k}" for b, n, k in works], capture_output=True, text=True)
    lines = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")]
    if proc.returncode != 0 or len(lines) != len(works):
        print(json.dumps({"impl": "reference", "unavailable": f"the reference's decode run ended with code {proc.returncode}: "
                          + " ".join((proc.stderr or proc.stdout).split())[-400:]}))
        return 0
    main_run = lines[0]

    def roofline(r):
        nbytes = weight_bytes + kv_bytes_per_token * (r["context"] - r["steps"] // 2) * r["batch"]
        gbs = nbytes / (r["ms_per_step"] / 1e3) / 1e9
        return {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm_gbs, "unit": "GB/s", "frac": round(gbs / hbm_gbs, 4)}

    out = {"impl": "reference",
           "metric": f"decode tokens/s (Qwen3-{args.shape.upper()} shape, bf16, batch {args.batch}, context {ctx})", "value": round(main_run["tokens_per_s"], 1),
           "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (the reference converts the bf16 checkpoint at load)",
           "data": "synthetic: seeded random weights, token ids from the model's own argmax, zeroed cache of the stated context length",
           "config": {"model": f"Qwen3-{args.shape.upper()} shape", "num_layers": layers, "num_layers_full": full_layers, "hidden_size": H,
                      "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": I, "vocab_size": V,
                      "global_batch": args.batch, "seq_len": ctx, "page_size": page, "parallelism": "single GPU",
                      "l2": "inputs (weights and cache) exceed L2 many times", "peaks": peak_src,
                      "api": "Qwen3::forward + compute_logits on CUDABackend, logits to the host and argmax as ModelRunner does; "
                             "LLMEngine takes text through a tokenizer, and execute_model reads freed host memory on CUDA"},
           "gpu_launches": None, "roofline": roofline(main_run), "clocks": clocks.summary(),
           "e2e": {"value": round(main_run["wall_tokens_per_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": main_run["h2d_bytes_per_step"],
                   "d2h_bytes_per_step": main_run["d2h_bytes_per_step"]},
           "prefill": {"unavailable": "a step of 100 or more tokens overruns the reference's scratch (src/models/qwen3.hpp:13, 97)"}}
    if len(lines) > 1:
        names = ["decode_b1", "decode_b64", "decode_b1_ctx640", "decode_b8_ctx640", "decode_b64_ctx640"]
        out["points"] = {n: round(r["tokens_per_s"], 1) for n, r in zip(names, lines[1:])}
        out["points_detail"] = {n: {"value": round(r["tokens_per_s"], 1), "ms_per_step": round(r["ms_per_step"], 4), "batch": r["batch"],
                                    "context": r["context"], "steps": r["steps"], "roofline": roofline(r)} for n, r in zip(names, lines[1:])}
    print(json.dumps(out))
    return 0



def peaks():
    """Copy bandwidth (GB/s), bf16 product rate of a kernel timed alone and of a seconds-long loop under
    the power cap (TFLOP/s), and where they come from: MEASURED_PEAKS.json beside this file when it
    exists (``hbm_gbs``, ``bf16_tflops``, ``bf16_tflops_sustained``), else 6.65 TB/s, 1.59 and 1.4 PFLOP/s."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm, burst, sustained, src = 6650.0, 1590.0, 1400.0, "fallback"
    if os.path.isfile(path):
        try:
            with open(path) as f:
                d = json.load(f)
            hbm = float(d.get("hbm_gbs", hbm))
            burst = float(d.get("bf16_tflops", burst))
            sustained = float(d.get("bf16_tflops_sustained") or burst)
            src = "measured"
        except (ValueError, OSError, TypeError):
            pass
    return hbm, burst, sustained, src


def kernel_rooflines(engine, batches, prompt_tokens, hbm_gbs, bf16_tflops, page):
    """Each dominant kernel alone, at the sizes it has inside the benchmark's steps.

    The products are called exactly as the model's parts call them (same plans, epilogues and
    deferred reductions), through the layers' own ``Linear`` objects, one layer after the other, so
    that every call reads weights that no earlier call left in L2; the attention kernels run on a
    cache of their own of the stated length.  Decoding sizes are read against the copy bandwidth
    (bytes = the weight or the cache read once, plus activations in and out), 2,048 tokens against
    the bf16 peak of a kernel timed alone."""
    import torch

    from spyinfer_b200 import microbench

    model = engine.model
    layers = model.layers
    dev = engine.config.device
    out = {}

    def timed(calls, reps):
        """Microseconds a call.  The calls are captured into a CUDA graph and replayed, as the engine
        replays its decode steps: the time is the device's, without the host's launch cost."""
        for f in calls[:2]:
            f()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for f in calls:
                f()
        graph.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (reps * len(calls))

    def product(name, linears, M, epilogue=None, defer=False, out_dtype=None, reps=3):
        K, N = linears[0].in_features, linears[0].out_features
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        calls = [(lambda lin=lin: lin(x, epilogue=epilogue, defer=defer, out_dtype=out_dtype)) for lin in linears]
        if len(calls) == 1:
            calls = calls * 8               # the head: one matrix, itself ten times L2
        us = timed(calls, reps)
        n_out = N // 2 if epilogue == "swiglu" else N
        nbytes = 2 * N * K + 2 * M * K + M * n_out * (4 if out_dtype == torch.float32 else 2)
        flops = 2.0 * M * N * K
        rec = {"us": round(us, 2)}
        if M <= 256:
            gbs = nbytes / us / 1e3
            rec.update(achieved=round(gbs, 1), unit="GB/s", frac=round(gbs / hbm_gbs, 4))
        else:
            tf = flops / us / 1e6
            rec.update(achieved=round(tf, 1), unit="TFLOP/s", frac=round(tf / bf16_tflops, 4))
        out[name] = rec

    # in the order of the power they draw: the decode attention and the decoding products (the clocks of a decode
    # step: no throttle reason), then the 2,048-token kernels, which run at the power cap and leave lower clocks behind
    spec = layers[0].mixer
    nh, nkv, hd = spec.nh, spec.nkv, spec.hd
    for context in (640, 8192):
        r = microbench.bench_attention(64, context, nh=nh, nkv=nkv, hd=hd, page_size=page, kernel="decode", iters=20, graph=True)
        out[f"attention_decode_b64_ctx{context}"] = {"us": round(r["us"], 2), "achieved": round(r["kv_gbs"], 1), "unit": "GB/s",
                                                      "frac": round(r["kv_gbs"] / hbm_gbs, 4)}
    sizes = [(f"b{b}", b) for b in batches] + [(f"t{prompt_tokens}", prompt_tokens)]
    for tag, M in sizes[:-1]:
        product(f"lm_head_{tag}", [model.head.linear], M, out_dtype=torch.float32)
    def products(tag, M):
        product(f"qkv_{tag}", [l.mixer.qkv for l in layers], M, defer=True)
        product(f"o_{tag}", [l.mixer.o for l in layers], M, defer=True)
        product(f"gate_up_{tag}", [l.feed_forward.gate_up for l in layers], M, epilogue="swiglu")
        product(f"down_{tag}", [l.feed_forward.down for l in layers], M, defer=True)

    for tag, M in sizes[:-1]:
        products(tag, M)
    r = microbench.bench_attention(1, prompt_tokens, q_len=prompt_tokens, nh=nh, nkv=nkv, hd=hd, page_size=page, kernel="tc", iters=20, graph=True)
    out[f"attention_prompt_t{prompt_tokens}"] = {"us": round(r["us"], 2), "achieved": round(r["tflops"], 1), "unit": "TFLOP/s",
                                                  "frac": round(r["tflops"] / bf16_tflops, 4)}
    products(*sizes[-1])
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append(parts)

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[2:]) if v.lower().startswith("active")})
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.samples)}


def mixed_workload(args, model_config, layers, full_layers, page) -> int:
    """A continuous batch as a user runs it: ``--requests`` requests (64) with prompt lengths uniform
    in [64, 2048] and 128 generated tokens each are all submitted to ``LLMEngine`` at once; the
    scheduler admits them, cuts their prompts into portions under ``--budget`` tokens a step beside
    the decode tokens of the requests already running, and the loop calls ``step()`` until all are
    done.  Timed on the host around the whole loop (the device is idle before and after); tokens go
    in and come out on the host.  The first pass is a warm-up (graph captures, first launches), the
    second is reported."""
    import torch

    from spyinfer_b200 import SamplingParams
    from spyinfer_b200.engine import LLMEngine

    n_req, new_tokens = args.requests, 128
    g = torch.Generator().manual_seed(11)
    lengths = torch.randint(64, 2049, (n_req,), generator=g).tolist()
    prompts = [torch.randint(0, model_config.vocab_size, (n,), generator=g).tolist() for n in lengths]
    num_pages = sum((n + new_tokens + page - 1) // page + 1 for n in lengths) + 8
    engine = LLMEngine(model_config=model_config, seed=0, dtype="bfloat16", max_num_seqs=n_req, max_model_len=2048 + new_tokens + 16,
                       kvcache_block_size=page, num_kvcache_blocks=num_pages, max_num_batched_tokens=args.budget)
    sp = SamplingParams(max_new_tokens=new_tokens, ignore_eos=True)
    result = None
    for run in range(2):
        engine.runner.step_events = []
        with ClockSampler() as clocks:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ids = [engine.add_request(p, sp) for p in prompts]
            steps = generated = 0
            first_token_at = {}
            while engine.has_unfinished_requests():
                for rid, _tok, _fin in engine.step():
                    generated += 1
                    first_token_at.setdefault(rid, time.perf_counter() - t0)
                steps += 1
            torch.cuda.synchronize()
            seconds = time.perf_counter() - t0
        assert generated == n_req * new_tokens, (generated, n_req * new_tokens)
        for rid in ids:
            engine.remove_request(rid)
        # the device's share of the time: each step's launches lie between two events on the stream; an event is stamped
        # when the stream reaches it, so the time between one step's last and the next step's first event is time the
        # device waited for the host
        pairs = engine.runner.step_events
        busy_ms = sum(a.elapsed_time(b) for a, b in pairs)
        span_ms = pairs[0][0].elapsed_time(pairs[-1][1])

        ttft = sorted(first_token_at.values())
        result = {"metric": f"generated tokens/s, mixed continuous batch (Qwen3-{args.shape.upper()} shape, bf16, {n_req} requests, prompts 64..2048, "
                            f"{new_tokens} generated each)", "value": round(generated / seconds, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
                  "warmup": 1, "ms_per_step": round(seconds * 1e3 / steps, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                  "dtype": "bf16", "data": "synthetic: seeded random weights and random token ids",
                  "config": {"model": f"Qwen3-{args.shape.upper()} shape", "num_layers": layers, "num_layers_full": full_layers,
                             "requests": n_req, "prompt_tokens_total": sum(lengths), "generated_tokens_total": generated,
                             "max_num_batched_tokens": args.budget, "page_size": page, "parallelism": "single GPU",
                             "timing": "host clock around the whole loop, device idle on both sides"},
                  "total_tokens_per_s": round((sum(lengths) + generated) / seconds, 1), "seconds": round(seconds, 3),
                  "first_token_s": {"median": round(ttft[len(ttft) // 2], 3), "max": round(ttft[-1], 3)},
                  "preemptions": engine.scheduler.num_preemptions, "clocks": clocks.summary(),
                  "device_busy": {"busy_ms": round(busy_ms, 1), "span_ms": round(span_ms, 1), "frac": round(busy_ms / span_ms, 4),
                                  "how": "CUDA events before the first and after the last launch of every step; busy = sum over steps, span = first to last event"}}
    print(json.dumps(result))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the model has (both numbers are reported)")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="Qwen3 layer sizes; the metric is quoted on 8b")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--no-points", action="store_true", help="skip the batch 1/64 and short-context points")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-kernels", action="store_true", help="skip the per-kernel rooflines")
    ap.add_argument("--workload", default="decode", choices=["decode", "mixed"],
                    help="decode: the contract's line (default); mixed: a continuous batch of --requests requests with prompts of 64 to 2,048 "
                         "tokens and 128 generated tokens each through LLMEngine, its own line")
    ap.add_argument("--requests", type=int, default=64, help="mixed workload: number of requests")
    ap.add_argument("--budget", type=int, default=2048, help="mixed workload: max_num_batched_tokens")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(json.dumps({"error": f"this engine runs on one GPU; --gpus {args.gpus} is not supported", "n_gpus": args.gpus}))
        return 2
    warmup = max(3, args.warmup)

    import torch

    from spyinfer_b200 import SamplingParams, config_from_json, kernels
    from spyinfer_b200.engine import LLMEngine, StepEntry

    hbm_gbs, bf16_tflops, bf16_sustained, peak_src = peaks()
    cfg_json = dict(QWEN3_8B)
    cfg_json.update(SHAPES[args.shape])
    full_layers = cfg_json["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg_json["num_hidden_layers"] = layers
    model_config = config_from_json(cfg_json)
    page = 16
    if args.workload == "mixed":
        return mixed_workload(args, model_config, layers, full_layers, page)
    max_batch = max(args.batch, 1 if args.no_points else 64)
    ctx = args.context
    torch.cuda.set_device(0)
    # a batch of 64 at the full context does not fit beside the weights of every shape (32B: 137 GB of
    # cache beside 65 GB of weights): the batch-64 points are then left out, and the line says so
    c0 = model_config
    est_weights = 2 * (layers * (c0.hidden_size * (c0.num_attention_heads + 2 * c0.num_key_value_heads) * c0.head_dim
                                 + c0.num_attention_heads * c0.head_dim * c0.hidden_size + 3 * c0.hidden_size * c0.intermediate_size)
                       + 2 * c0.vocab_size * c0.hidden_size)
    est_cache = lambda b: b * (ctx + 32) * 4 * c0.num_key_value_heads * c0.head_dim * layers
    points_batches = (1, 64)
    if not args.no_points and est_weights + est_cache(64) > 0.92 * torch.cuda.get_device_properties(0).total_memory:
        points_batches = (1,)
        max_batch = max(args.batch, 1)
    total_steps = warmup + args.steps + 8
    pages_per_req = (ctx + page - 1) // page + 1
    num_pages = max_batch * pages_per_req + (args.prefill_tokens + page - 1) // page + 8
    # one more point when the batch-64 points fit: 256 requests of 1,024 keys (the pool of 64 x the context holds them)
    large = (256, 1024) if (not args.no_points and 64 in points_batches and 256 * (1024 // page + 2) <= num_pages) else None
    if large:
        max_batch = max(max_batch, large[0])
    engine = LLMEngine(model_config=model_config, seed=0, dtype="bfloat16", max_num_seqs=max_batch, max_model_len=max(ctx, args.prefill_tokens) + 16,
                       kvcache_block_size=page, num_kvcache_blocks=num_pages, max_num_batched_tokens=max(args.prefill_tokens, max_batch))
    runner, cache = engine.runner, engine.runner.cache
    for g in cache.groups:                      # random cache contents: the decode step's work does not depend on them
        g.pages.normal_(0.0, 1.0)
    c = model_config
    H, I, V, nh, nkv, hd = c.hidden_size, c.intermediate_size, c.vocab_size, c.num_attention_heads, c.num_key_value_heads, c.head_dim
    layer_params = H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * I
    weight_bytes = 2 * (layers * layer_params + V * H)
    kv_bytes_per_token = 2 * 2 * nkv * hd * layers
    vocab = V

    def fake_requests(batch, context, tag):
        """Live requests whose caches hold ``context`` tokens (random content)."""
        rids = [f"{tag}{i}" for i in range(batch)]
        for r in rids:
            cache.add_request(r)
            cache.reserve(r, context)
            cache.commit(r, context)
        return rids

    def release(rids):
        for r in rids:
            runner.finish(r)

    def decode_device(batch, context, steps, warm):
        """Tokens a second of `steps` decode steps timed on the device."""
        start_ctx = context - (steps + warm) - 1
        rids = fake_requests(batch, start_ctx, "d")
        g = torch.Generator().manual_seed(batch)
        toks = torch.randint(0, vocab, (steps + warm, batch), generator=g).tolist()
        sp = [SamplingParams()] * batch
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = 0
        for i in range(steps + warm):
            if i == warm:
                torch.cuda.synchronize()
                launches0 = kernels.launch_count()
                e0.record()
            logits = runner.step([StepEntry(r, [toks[i][j]], [0]) for j, r in enumerate(rids)])
            engine.sampler.sample(logits, sp, [i] * batch)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        runner.check_status()
        release(rids)
        return batch * steps / (ms / 1e3), ms / steps, kernels.launch_count() - launches0

    def decode_e2e(batch, context, steps, warm):
        """The same through the public entry point: requests are submitted with real prompts,
        prefilled by LLMEngine.step() (untimed), then `steps` decode steps are timed, each with
        its host-to-device copy of the batch arrays and its read-back of the sampled tokens."""
        # requests whose prompts finish early decode while the others are still prefilling:
        # leave room for those extra tokens so that nobody finishes inside the timed region
        extra = batch * context // engine.config.max_num_batched_tokens + 4
        prompt_len = context - (steps + warm) - 2 - extra
        g = torch.Generator().manual_seed(1000 + batch)
        sp = SamplingParams(max_new_tokens=steps + warm + 2 + extra, ignore_eos=True)
        ids = [engine.add_request(torch.randint(0, vocab, (prompt_len,), generator=g).tolist(), sp) for _ in range(batch)]
        started = set()
        while len(started) < batch:                      # prompts, in portions under the token budget
            started.update(r for r, _, _ in engine.step())
        n_out = 0
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for i in range(steps + warm):
            if i == warm:
                torch.cuda.synchronize()
                e0.record()
                n_out = 0
            n_out += len(engine.step())
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        for r in ids:
            engine.remove_request(r)
        assert n_out == batch * steps, (n_out, batch, steps)
        h2d = 4 * (4 * batch + 3 * batch + 1 + batch * cache.width)
        return n_out / (ms / 1e3), h2d, 4 * batch + 8     # the sampled tokens and the two words of the status

    def prefill(tokens):
        g = torch.Generator().manual_seed(7)
        toks = torch.randint(0, vocab, (tokens,), generator=g).tolist()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        times = []
        for i in range(6):                       # the first run is a warm-up; the median of the other five is reported
            torch.cuda.synchronize()
            e0.record()
            runner.step([StepEntry(f"p{i}", toks, [tokens - 1])])
            e1.record()
            torch.cuda.synchronize()
            runner.finish(f"p{i}")
            times.append(e0.elapsed_time(e1))
        best = sorted(times[1:])[len(times[1:]) // 2]
        runner.check_status()
        flops = 2.0 * tokens * layers * layer_params + 2.0 * V * H + layers * 4.0 * nh * hd * tokens * (tokens + 1) / 2
        return {"value": round(tokens / (best / 1e3), 1), "tokens": tokens, "ms": round(best, 3),
                "frac": round(flops / (best / 1e3) / (bf16_tflops * 1e12), 4), "peak_tflops": bf16_tflops,
                "frac_sustained": round(flops / (best / 1e3) / (bf16_sustained * 1e12), 4), "peak_tflops_sustained": bf16_sustained}

    with ClockSampler() as clocks:
        value, ms_per_step, launches = decode_device(args.batch, ctx, args.steps, warmup)
    clock_summary = clocks.summary()
    step_bytes = weight_bytes + kv_bytes_per_token * (ctx - args.steps // 2) * args.batch
    achieved = step_bytes / (ms_per_step / 1e3) / 1e9
    out = {
        "metric": f"decode tokens/s (Qwen3-{args.shape.upper()} shape, bf16, batch {args.batch}, context {ctx})", "value": round(value, 1), "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights, random token ids, random cache contents of the stated context length",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "num_layers": layers, "num_layers_full": full_layers, "hidden_size": H,
                   "num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "intermediate_size": I, "vocab_size": V,
                   "global_batch": args.batch, "seq_len": ctx, "page_size": page, "parallelism": "single GPU",
                   "l2": "inputs (weights and cache) exceed L2 many times", "peaks": peak_src},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": hbm_gbs, "unit": "GB/s", "frac": round(achieved / hbm_gbs, 4)},
        "clocks": clock_summary,
    }
    out["prefill"] = prefill(args.prefill_tokens)
    if not args.no_e2e:
        e2e, h2d, d2h = decode_e2e(args.batch, ctx, args.steps, warmup)
        out["e2e"] = {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    if not args.no_points:
        points, detail = {}, {}

        def point(name, b, context):
            tps, ms, _ = decode_device(b, context, args.steps, warmup)
            nbytes = weight_bytes + kv_bytes_per_token * (context - args.steps // 2) * b
            gbs = nbytes / (ms / 1e3) / 1e9
            points[name] = round(tps, 1)
            detail[name] = {"value": round(tps, 1), "ms_per_step": round(ms, 4), "batch": b, "context": context,
                            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": hbm_gbs, "unit": "GB/s", "frac": round(gbs / hbm_gbs, 4)}}

        for b in points_batches:
            point(f"decode_b{b}", b, ctx)
        for b in (1, 8) + points_batches[1:]:
            point(f"decode_b{b}_ctx640", b, 640 + (args.steps + warmup) // 2)
        if large:
            point(f"decode_b{large[0]}_ctx{large[1]}", large[0], large[1] + (args.steps + warmup) // 2)
        out["points"] = points
        out["points_detail"] = detail
    if not args.no_kernels:
        out["kernels"] = kernel_rooflines(engine, sorted({args.batch, 64}), args.prefill_tokens, hbm_gbs, bf16_tflops, page)
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
