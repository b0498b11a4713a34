"""Device timelines of the two tcgen05 attention kernels, for the summaries under profiles/.

    SPYINFER_NVCC_FLAGS=-DSPY_TIMELINE python -m spyinfer_b200.timeline decode [--layers 6] [--batch 8] [--context 8192]
    SPYINFER_NVCC_FLAGS=-DSPY_TIMELINE python -m spyinfer_b200.timeline prompt [--tokens 8192]
    SPYINFER_NVCC_FLAGS=-DSPY_TIMELINE python -m spyinfer_b200.timeline prompt-blocks [--tokens 2048]
    SPYINFER_NVCC_FLAGS=-DSPY_TIMELINE python -m spyinfer_b200.timeline chain [--layers 2] [--batch 8] [--context 8192]

With ``-DSPY_TIMELINE`` the kernels stamp the global timer at points of a block's life into a
device array; this program runs them, copies the stamps out and prints, per point, the minimum,
median and maximum over the blocks.  ``decode``: the decode attention of the LAST layer inside
the engine's captured decode graph of a model with Qwen3-8B's layer sizes (so the kernels
ahead of it and behind it are the real ones).  ``prompt``: the prompt attention alone, one
sequence of ``--tokens`` tokens, stamps of every block's tenth key tile.  ``prompt-blocks``: the
same kernel, stamps of each block's life (set-up, Q tile, first scores, loop, output) and how
the blocks follow one another on their SMs.  ``chain``: the
few-token products (one-tile tcgen05 kernel) of one decode step in the order they ran, with
the last layer's decode attention between them, on one time axis.
"""
from __future__ import annotations

import argparse
import ctypes
import sys

import numpy as np
import torch

QWEN3_8B_LAYER = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_act": "silu", "hidden_size": 4096,
                  "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288, "vocab_size": 151936,
                  "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 40960}


def _stamps(module: str, fn: str, blocks: int, points: int = 16) -> np.ndarray:
    from .csrc import build
    lib = build.load(module)
    if not hasattr(lib, fn):
        raise SystemExit(f"{module} was built without -DSPY_TIMELINE: set SPYINFER_NVCC_FLAGS=-DSPY_TIMELINE")
    buf = (ctypes.c_ulonglong * (blocks * points))()
    if getattr(lib, fn)(buf) != 0:
        raise SystemExit(build.last_error(module))
    return np.array(buf, dtype=np.uint64).reshape(blocks, points).astype(np.int64)


def _decode_steps(layers: int, batch: int, context: int, steps: int = 10):
    from . import SamplingParams, config_from_json
    from .engine import LLMEngine, StepEntry
    cfg = dict(QWEN3_8B_LAYER, num_hidden_layers=layers)
    eng = LLMEngine(model_config=config_from_json(cfg), seed=0, dtype="bfloat16", max_num_seqs=batch, max_model_len=context + 64,
                    kvcache_block_size=16, num_kvcache_blocks=batch * ((context + 64) // 16 + 2) + 8, max_num_batched_tokens=2048)
    runner, cache = eng.runner, eng.runner.cache
    for g in cache.groups:
        g.pages.normal_()
    rids = [f"r{i}" for i in range(batch)]
    for r in rids:
        cache.add_request(r)
        cache.reserve(r, context - 20)
        cache.commit(r, context - 20)
    for _ in range(steps):
        logits = runner.step([StepEntry(r, [5], [0]) for r in rids])
        eng.sampler.sample(logits, [SamplingParams()] * batch, [0] * batch)
    torch.cuda.synchronize()


def chain(layers: int, batch: int, context: int) -> None:
    from .csrc import build
    _decode_steps(layers, batch, context)
    lib = build.load("gemm_tcgen05")
    if not hasattr(lib, "spy_gemm_tcgen05_timeline"):
        raise SystemExit("gemm_tcgen05 was built without -DSPY_TIMELINE: set SPYINFER_NVCC_FLAGS=-DSPY_TIMELINE")
    launches, blocks, points = 64, 320, 10
    buf = (ctypes.c_ulonglong * (launches * blocks * points))()
    nxt = ctypes.c_int(0)
    if lib.spy_gemm_tcgen05_timeline(buf, ctypes.byref(nxt)) != 0:
        raise SystemExit(build.last_error("gemm_tcgen05"))
    g = np.array(buf, dtype=np.uint64).reshape(launches, blocks, points).astype(np.int64)
    a = _stamps("attention_decode", "spy_attention_decode_timeline", 256)[:148]
    a = a[a[:, 5] > 0]
    rows = []
    for plane in g:
        n = int(min(plane[0, 9], blocks)) if plane[0, 0] > 0 else 0
        if n:
            rows.append((int(plane[:n, 0].min()), "product", plane[:n], int(plane[0, 9])))
    if not rows:
        raise SystemExit("no stamps: did the step run the one-tile product kernel?")
    rows = sorted(rows, key=lambda r: r[0])[-(4 * layers + 1):]   # the last step's launches: four a layer and the output head
    rows.append((int(a[:, 0].min()), "attention", a, len(a)))
    norms = _stamps("rmsnorm", "spy_rmsnorm_timeline", 128, 8)
    norms = norms[norms[:, 0] >= rows[0][0] - 20_000]
    for start in sorted(set(int(x) for x in norms[:, 0] // 2000)):   # blocks of one launch enter within two microseconds
        group = norms[norms[:, 0] // 2000 == start]
        rows.append((int(group[:, 0].min()), "norm", group, len(group)))
    rows.sort(key=lambda r: r[0])
    t0 = rows[0][0]
    print(f"{layers} layers, batch {batch}, {context} keys: the last step's few-token products (first {blocks} blocks of each) and the last "
          "layer's decode attention; microseconds after the first entry")
    print(f"{'kernel':10s} {'blocks':>6s} {'entry':>15s} {'wait returned':>15s} {'first stage in':>15s} {'last stage in':>15s} {'sums ready':>11s} {'stored':>8s} {'exit':>8s}")

    def span(col):
        col = (col[col > 0] - t0) / 1000.0
        return f"{col.min():6.1f} ..{col.max():6.1f}" if len(col) else " " * 15

    def last(col):
        col = (col[col > 0] - t0) / 1000.0
        return f"{col.max():8.1f}" if len(col) else " " * 8

    for _, kind, t, n in rows:
        if kind == "product":
            print(f"{kind:10s} {n:6d} {span(t[:, 0])} {span(t[:, 2])} {span(t[:, 3])} {span(t[:, 4])} {last(t[:, 5]):>11s} {last(t[:, 6])} {last(t[:, 7])}")
        elif kind == "attention":
            print(f"{kind:10s} {n:6d} {span(t[:, 0])} {span(t[:, 3])} {'first scores':>15s} {span(t[:, 5])} {'':>11s} {last(t[:, 8])} {last(t[:, 10])}")
        else:
            print(f"{kind:10s} {n:6d} {span(t[:, 0])} {span(t[:, 2])} {'row summed':>15s} {span(t[:, 3])} {last(t[:, 4]):>11s} {last(t[:, 5])}")


def decode(layers: int, batch: int, context: int) -> None:
    _decode_steps(layers, batch, context)
    t = _stamps("attention_decode", "spy_attention_decode_timeline", 256)[:148]
    names = ["entry", "prologue done", "first K box requested", "kernel ahead complete (wait returned)", "first Q.K issued", "first scores ready",
             "last probabilities written", "last P.V complete", "partial result written", "segment done", "exit", "merge: arrived last",
             "-", "merge: parts added", "-", "producer: first segment known"]
    busy = t[:, 5] > 0
    t0 = t[busy, 0].min()
    print(f"decode attention of the last of {layers} layers, batch {batch}, {context} keys; {busy.sum()} blocks with work; "
          "ns after the first block's entry: min / median / max")
    for i, n in enumerate(names):
        col = t[busy, i]
        col = col[col >= t0] - t0
        if n != "-" and len(col):
            print(f"  {n:38s} {col.min():8d} {int(np.median(col)):8d} {col.max():8d}")


def prompt(tokens: int) -> None:
    from . import microbench
    r = microbench.bench_attention(1, tokens, tokens, 0, iters=2, kernel="tc")
    print(f"prompt attention, {tokens} tokens: {r['us']:.1f} us, {r['tflops']:.1f} TFLOP/s")
    t = _stamps("attention_tc", "spy_attention_tc_timeline", 1024)
    t = t[(t[:, 0] > 0) & (t[:, 5] > 0) & (t[:, 10] > 0)]
    names = ["scores of tile 10 ready (softmax)", "scores loaded", "maxima exchanged", "exponentials done", "P of tile 10 written",
             "scores of tile 11 ready (softmax)", "MMA: P of tile 10 seen", "MMA: V of tile 10 seen", "MMA: P.V of tile 10 issued",
             "MMA: K of tile 12 seen", "MMA: Q.K of tile 12 issued", "K warp: stage free for tile 13", "K warp: tile 13 requested"]
    print(f"{len(t)} blocks with more than twelve tiles; ns after the block's scores of tile 10 were ready: median (10 % .. 90 %)")
    for i, n in enumerate(names):
        d = (t[:, i] - t[:, 0])[t[:, i] > 0]
        if len(d):
            print(f"  {n:38s} {int(np.median(d)):7d}  ({int(np.percentile(d, 10))} .. {int(np.percentile(d, 90))})")


def prompt_blocks(tokens: int) -> None:
    """Where the work items of the prompt attention spend their lives, and how they follow one another on the SMs."""
    from . import microbench
    r = microbench.bench_attention(1, tokens, tokens, 0, iters=2, kernel="tc")
    print(f"prompt attention, {tokens} tokens: {r['us']:.1f} us, {r['tflops']:.1f} TFLOP/s")
    t = _stamps("attention_tc", "spy_attention_tc_block_life", 1024, 8)
    t = t[(t[:, 0] > 0) & (t[:, 6] > 0)]
    tiles, sm = t[:, 7] & 0xffff, t[:, 7] >> 16
    t0 = t[:, 0].min()
    print(f"{len(t)} work items on {len(set(sm.tolist()))} SMs (one resident block a SM walks through its items); the kernel's span "
          f"(first item's start to last output stored) {(t[:, 6].max() - t0) / 1e3:.1f} us")
    names = [(0, 2, "item read -> Q tile in shared memory (positions read, cp.async)"), (2, 3, "Q tile -> first scores ready"),
             (3, 4, "first scores -> last probabilities written"), (4, 5, "last probabilities -> last P.V complete"),
             (5, 6, "last P.V -> output stored")]
    for a, b, n in names:
        d = t[:, b] - t[:, a]
        print(f"  {n:64s} median {int(np.median(d)):7d} ns  (10 % {int(np.percentile(d, 10))}, 90 % {int(np.percentile(d, 90))})")
    loop = (t[:, 4] - t[:, 3]) / np.maximum(tiles - 1, 1)
    print(f"  per tile inside the loop: median {int(np.median(loop[tiles > 2]))} ns; tiles a block: {int(tiles.min())} .. {int(tiles.max())}, {int(tiles.sum())} in all")
    busy, gaps, ends = [], [], []
    for s_ in sorted(set(sm.tolist())):
        b = t[sm == s_]
        b = b[np.argsort(b[:, 0])]
        busy.append((b[:, 6] - b[:, 0]).sum())
        gaps += (b[1:, 0] - b[:-1, 6]).tolist()
        ends.append(b[:, 6].max() - t0)
    print(f"  per SM: the items' lives sum to median {np.median(busy) / 1e3:.1f} us; gap between an item's output and the next item's start median "
          f"{int(np.median(gaps)) if gaps else 0} ns; last exit {min(ends) / 1e3:.1f} .. {max(ends) / 1e3:.1f} us")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="what", required=True)
    d = sub.add_parser("decode")
    d.add_argument("--layers", type=int, default=6)
    d.add_argument("--batch", type=int, default=8)
    d.add_argument("--context", type=int, default=8192)
    c = sub.add_parser("chain")
    c.add_argument("--layers", type=int, default=2)
    c.add_argument("--batch", type=int, default=8)
    c.add_argument("--context", type=int, default=8192)
    p = sub.add_parser("prompt")
    p.add_argument("--tokens", type=int, default=8192)
    b = sub.add_parser("prompt-blocks")
    b.add_argument("--tokens", type=int, default=2048)
    args = ap.parse_args(argv)
    from . import kernels
    kernels.require_cuda()
    if args.what == "decode":
        decode(args.layers, args.batch, args.context)
    elif args.what == "chain":
        chain(args.layers, args.batch, args.context)
    elif args.what == "prompt-blocks":
        prompt_blocks(args.tokens)
    else:
        prompt(args.tokens)
    return 0


if __name__ == "__main__":
    sys.exit(main())
