"""Timings of single kernels at chosen sizes.

    python -m spyinfer_b200.microbench gemm --m 2048 --n 24576 --k 4096 [--out-dtype float32] [--iters 20] [--graph] [--defer] [--epilogue swiglu]
    python -m spyinfer_b200.microbench attention --batch 8 --context 8192 [--q-len 1] [--split-keys 576] [--kernel tc|mma|decode] [--iters 10]
                                                 [--heads 64 --kv-heads 8 --head-dim 128] [--graph]
    python -m spyinfer_b200.microbench rmsnorm --rows 2048 [--size 4096] [--splits 6]
    python -m spyinfer_b200.microbench step --batch 8 --context 8192 [--layers 4] [--prompt-tokens 2048]      # one step's kernels on the time axis

Defaults are Qwen3-8B's sizes (32 query heads, 8 key/value heads, head size 128, pages of 16).
Timing is by CUDA events around ``iters`` launches after a warm-up (``--graph``: replayed from a CUDA graph, which
kernels of a few microseconds need: eager launches cost the host more than that); the product cycles through
enough weight copies to exceed L2, the attention's cache does so by itself at the default sizes.
"""
from __future__ import annotations

import argparse
import math
import sys

import torch

from . import kernels

DEV = "cuda:0"


def bench_gemm(M: int, N: int, K: int, out_dtype=torch.bfloat16, iters: int = 20, graph: bool = False, defer: bool = False,
               epilogue=None) -> dict:
    """``defer``: the product may leave split-K parts for its consumer, as the model's parts allow it to
    (the time is then without the sum over the parts).  ``epilogue="swiglu"``: rows of gate and up alternate."""
    a = torch.randn(M, K, device=DEV).to(torch.bfloat16)
    copies = max(1, int(300e6 // (N * K * 2)) + 1)
    ws = [(torch.randn(N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16) for _ in range(copies)]
    n_out = N // 2 if epilogue else N
    out = None if defer else torch.empty(M, n_out, device=DEV, dtype=out_dtype)

    def run(i):
        if defer:
            kernels.gemm_tcgen05(a, ws[i % copies], out_dtype=out_dtype, defer=True)
        else:
            kernels.gemm_tcgen05(a, ws[i % copies], out, epilogue=epilogue)

    for i in range(2):
        run(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:   # the launches replayed from a CUDA graph: device time without the host's launch cost
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                run(i)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for i in range(iters):
            run(i)
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    return {"us": ms * 1e3, "tflops": 2.0 * M * N * K / ms / 1e9, "gbs": (N * K * 2 + M * K * 2 + M * n_out * (4 if out_dtype == torch.float32 else 2)) / ms / 1e6}


def bench_attention(batch: int, context: int, q_len: int = 1, split_keys: int = 0, nh: int = 32, nkv: int = 8, hd: int = 128,
                    page_size: int = 16, iters: int = 10, kernel: str = "auto", share: str = "auto", graph: bool = False) -> dict:
    width = (context + page_size - 1) // page_size
    pages = torch.randn(batch * width + 1, 2, nkv, page_size, hd, device=DEV).to(torch.bfloat16)
    bt = torch.randperm(batch * width, device=DEV).view(batch, width).to(torch.int32)
    T = batch * q_len
    q = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV).to(torch.bfloat16)
    pos = torch.cat([torch.arange(context - q_len, context, dtype=torch.int32) for _ in range(batch)]).to(DEV)
    q_start = (torch.arange(batch + 1, dtype=torch.int32) * q_len).to(DEV)
    out = torch.empty(T, nh * hd, device=DEV, dtype=torch.bfloat16)
    max_splits = (context + split_keys - 1) // split_keys if split_keys else 0

    use_tc = kernel == "tc" or (kernel == "auto" and split_keys == 0)

    def run():
        if kernel == "decode":
            kernels.attention_decode(q, nh, hd, out, pages, bt, pos, q_start, batch, 1 / math.sqrt(hd), share=share)
        elif use_tc:
            kernels.attention_tc(q, nh, hd, out, pages, bt, pos, q_start, batch, 1 / math.sqrt(hd))
        else:
            kernels.attention_mma(q, nh, hd, out, pages, bt, pos, q_start, batch, 1 / math.sqrt(hd), split_keys=split_keys, max_splits=max_splits)

    run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:   # the launches replayed from a CUDA graph: device time without the host's launch cost
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(iters):
                run()
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for _ in range(iters):
            run()
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    kv_bytes = batch * context * 2 * nkv * hd * 2
    flops = 4.0 * nh * hd * batch * (q_len * (context - q_len) + q_len * (q_len + 1) / 2)
    return {"us": ms * 1e3, "kv_gbs": kv_bytes / ms / 1e6, "tflops": flops / ms / 1e9}


def bench_rmsnorm(rows: int, size: int, splits: int = 0, iters: int = 20, graph: bool = True) -> dict:
    """The residual norm as a layer runs it: ``h += delta; x = norm(h) * weight`` with a float32 stream ``h``, bfloat16 ``x``
    and a bfloat16 ``delta`` (``splits == 0``) or ``splits`` stacked float32 partial products.  Several copies of the
    buffers are cycled so that a launch does not find the last one's in L2."""
    copies = max(2, int(200e6 // (rows * size * 10)) + 1)
    hs = [torch.randn(rows, size, device=DEV) for _ in range(copies)]
    ds = [torch.randn(splits, rows, size, device=DEV) if splits else torch.randn(rows, size, device=DEV).to(torch.bfloat16) for _ in range(copies)]
    w = torch.ones(size, device=DEV, dtype=torch.bfloat16)
    out = torch.empty(rows, size, device=DEV, dtype=torch.bfloat16)

    def run(i):
        kernels.rmsnorm(hs[i % copies], w, 1e-6, out, delta=ds[i % copies], write_back=True)

    run(0)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if graph:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(iters):
                run(i)
        g.replay()
        torch.cuda.synchronize()
        e0.record()
        g.replay()
        e1.record()
    else:
        e0.record()
        for i in range(iters):
            run(i)
        e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    nbytes = rows * size * (4 + 4 + 2 + (4 * splits if splits else 2))
    return {"us": ms * 1e3, "gbs": nbytes / ms / 1e6}


def step_timeline(batch: int, context: int, layers: int = 4, shape: dict = None, prompt_tokens: int = 0) -> list:
    """The kernels of one step of a model with ``layers`` layers of the given layer sizes (default: Qwen3-8B's), as the
    profiler (CUPTI) saw them on the device: ``(name, start µs, duration µs)`` in the order of their starts.  A decode step
    of ``batch`` requests holding ``context`` keys each, replayed from its graph; with ``prompt_tokens`` a prompt of that
    many tokens instead.  With programmatic dependent launch a kernel starts while the one ahead still runs, so what a
    link of the chain costs is the distance between two kernels' ENDS, which ``print_timeline`` lists."""
    from torch.profiler import ProfilerActivity, profile

    from .config import config_from_json
    from .engine import LLMEngine, StepEntry

    cfg = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "num_hidden_layers": layers, "hidden_size": 4096,
           "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
           "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 40960}
    cfg.update(shape or {})
    page = 16
    tokens = max(context + 16, prompt_tokens + 16)
    engine = LLMEngine(model_config=config_from_json(cfg), seed=0, dtype="bfloat16", max_num_seqs=max(batch, 1), max_model_len=tokens,
                       kvcache_block_size=page, num_kvcache_blocks=max(batch, 1) * (tokens // page + 2) + 8, max_num_batched_tokens=max(prompt_tokens, batch, 16))
    runner, cache = engine.runner, engine.runner.cache
    if prompt_tokens:
        toks = torch.randint(0, 1000, (prompt_tokens,)).tolist()

        def run(i):
            runner.step([StepEntry(f"p{i}", toks, [prompt_tokens - 1])])
            runner.finish(f"p{i}")
    else:
        rids = [f"d{i}" for i in range(batch)]
        for r in rids:
            cache.add_request(r)
            cache.reserve(r, context)
            cache.commit(r, context)

        def run(i):
            runner.step([StepEntry(r, [5 + i], [0]) for r in rids])
    for i in range(5):
        run(i)
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        run(5)
        torch.cuda.synchronize()
    events = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and "mem" not in e.name.lower()]
    events.sort(key=lambda e: e.time_range.start)
    t0 = events[0].time_range.start
    return [(e.name, e.time_range.start - t0, e.time_range.end - e.time_range.start) for e in events]


def print_timeline(events: list) -> None:
    """The second layer's kernels with their starts, durations, ends and the distance of each end from the end before."""
    def short(name):
        name = name.replace("(anonymous namespace)::", "").replace("void ", "")
        return name.split("(")[0][:44]
    firsts = [i for i, e in enumerate(events) if "rmsnorm" in e[0]]
    lo, hi = (firsts[2], firsts[4] + 1) if len(firsts) > 4 else (0, len(events))     # two norms a layer: the second layer, and the norm after it
    prev_end = None
    print(f"{'kernel':46s} {'start':>9s} {'duration':>9s} {'end':>9s} {'after the end before':>21s}")
    for name, start, dur in events[lo:hi]:
        end = start + dur
        print(f"{short(name):46s} {start:9.1f} {dur:9.1f} {end:9.1f} {'' if prev_end is None else format(end - prev_end, '21.1f')}")
        prev_end = end
    print(f"whole step: {events[-1][1] + events[-1][2]:.1f} us, {len(events)} kernels")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, required=True)
    g.add_argument("--n", type=int, required=True)
    g.add_argument("--k", type=int, required=True)
    g.add_argument("--out-dtype", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--iters", type=int, default=20)
    g.add_argument("--graph", action="store_true", help="replay the launches from a CUDA graph (device time without host launch cost)")
    g.add_argument("--defer", action="store_true", help="split-K parts may stay unsummed, as inside the model")
    g.add_argument("--epilogue", default=None, choices=["swiglu"])
    n = sub.add_parser("rmsnorm")
    n.add_argument("--rows", type=int, required=True)
    n.add_argument("--size", type=int, default=4096)
    n.add_argument("--splits", type=int, default=0, help="the delta is a stack of this many float32 partial products (0: one bfloat16 tensor)")
    n.add_argument("--iters", type=int, default=20)
    t = sub.add_parser("step", help="the kernels of one step on the device's time axis")
    t.add_argument("--batch", type=int, default=8)
    t.add_argument("--context", type=int, default=8192)
    t.add_argument("--layers", type=int, default=4)
    t.add_argument("--prompt-tokens", type=int, default=0, help="a prompt of this many tokens instead of a decode step")
    a = sub.add_parser("attention")
    a.add_argument("--batch", type=int, required=True)
    a.add_argument("--context", type=int, required=True)
    a.add_argument("--q-len", type=int, default=1)
    a.add_argument("--split-keys", type=int, default=0, help="mma kernel only: 0: tiles mode; else split mode with this range length")
    a.add_argument("--iters", type=int, default=10)
    a.add_argument("--page-size", type=int, default=16)
    a.add_argument("--heads", type=int, default=32, help="query heads")
    a.add_argument("--kv-heads", type=int, default=8)
    a.add_argument("--head-dim", type=int, default=128)
    a.add_argument("--graph", action="store_true", help="replay the launches from a CUDA graph (device time without host launch cost)")
    a.add_argument("--share", default="auto", choices=["auto", "split", "whole"], help="decode kernel: how the work is dealt out over the blocks")
    a.add_argument("--kernel", default="auto", choices=["auto", "tc", "mma", "decode"],
                   help="auto: tcgen05 for tiles mode, mma.sync for split mode; decode: the persistent tcgen05 decode kernel (q-len 1)")
    args = ap.parse_args(argv)
    kernels.require_cuda()
    if args.what == "gemm":
        r = bench_gemm(args.m, args.n, args.k, getattr(torch, args.out_dtype), args.iters, graph=args.graph, defer=args.defer, epilogue=args.epilogue)
        print(f"gemm M={args.m} N={args.n} K={args.k}: {r['us']:.1f} us, {r['tflops']:.1f} TFLOP/s, {r['gbs']:.1f} GB/s")
    elif args.what == "step":
        print_timeline(step_timeline(args.batch, args.context, args.layers, prompt_tokens=args.prompt_tokens))
        return 0
    elif args.what == "rmsnorm":
        r = bench_rmsnorm(args.rows, args.size, args.splits, args.iters)
        print(f"rmsnorm rows={args.rows} size={args.size} splits={args.splits}: {r['us']:.1f} us, {r['gbs']:.1f} GB/s")
    else:
        r = bench_attention(args.batch, args.context, args.q_len, args.split_keys, nh=args.heads, nkv=args.kv_heads, hd=args.head_dim, page_size=args.page_size,
                            iters=args.iters, kernel=args.kernel, share=args.share, graph=args.graph)
        print(f"attention batch={args.batch} context={args.context} q_len={args.q_len} split_keys={args.split_keys}: {r['us']:.1f} us, "
              f"cache read at {r['kv_gbs']:.1f} GB/s, {r['tflops']:.1f} TFLOP/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
