"""Trace replay: feeds given token ids through a model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N
              [--page-size P] [--num-pages K] [--max-num-seqs S]
    trace_run --random CONFIG.json --seed N [--weight-std X --norm-std Y] --dtype ... --out DIR --max-tokens N

Steps are read from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch through ``ModelRunner.step`` (the step function that
generation uses, with the same model, cache manager and kernels); nothing is sampled.  For a
step in which something is wanted, ``OUT/<step>.f32`` gets the logits at the wanted places,
in the order of the entries and of ``want``, little-endian float32 ``[wanted, vocab]``.
Requests named in ``end`` give back what they hold after the step.  After every step a line
``done <step>`` is printed and flushed.

The cache pool holds ``--max-tokens`` tokens in pages of ``--page-size`` (16 unless given;
the reference's ``kvcache_block_size``, spymaster2h/spyinfer src/config.hpp:26), so pages
are used again as requests end; ``--num-pages`` (the reference's ``num_kvcache_blocks``,
src/config.hpp:27) sets the number of pages outright instead.  ``--random`` takes a
config.json (a file, or a folder that holds one) and a seed in place of a model folder: the
model folder is written to a temporary place with ``weights.write_model_folder`` (the same
tensors every time for one configuration and seed) and read back by the ordinary loader.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", help="folder with config.json and model.safetensors")
    ap.add_argument("--random", metavar="CONFIG", help="a config.json (or a folder with one): random weights from --seed instead of --model")
    ap.add_argument("--seed", type=int, default=0, help="seed of --random")
    ap.add_argument("--weight-std", type=float, default=0.02, help="--random: standard deviation of matrices and embeddings")
    ap.add_argument("--norm-std", type=float, default=0.05, help="--random: norm weights are 1 + N(0, this)")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time, each request's "
                    "count rounded up to a multiple of 64")
    ap.add_argument("--page-size", type=int, default=16, help="tokens a page (kvcache_block_size)")
    ap.add_argument("--num-pages", type=int, default=None, help="pages of the pool (num_kvcache_blocks); default: what --max-tokens needs")
    ap.add_argument("--max-num-seqs", type=int, default=8, help="most live requests")
    args = ap.parse_args(argv)
    if (args.model is None) == (args.random is None):
        ap.error("give either --model or --random")
    if args.page_size <= 0 or args.max_num_seqs <= 0 or (args.num_pages is not None and args.num_pages <= 0):
        ap.error("--page-size, --num-pages and --max-num-seqs must be positive")

    import torch

    from ..config import EngineConfig, load_model_config
    from .batch import StepEntry
    from .model import Model
    from .runner import ModelRunner

    os.makedirs(args.out, exist_ok=True)
    scratch = None
    if args.random is not None:
        import tempfile

        from ..weights import write_model_folder

        scratch = tempfile.TemporaryDirectory(prefix="trace_run_model_")
        source = args.random if os.path.isdir(args.random) else os.path.dirname(os.path.abspath(args.random))
        if not os.path.isdir(args.random) and os.path.basename(args.random) != "config.json":
            import shutil

            source = os.path.join(scratch.name, "source")       # a configuration under another file name
            os.makedirs(source)
            shutil.copyfile(args.random, os.path.join(source, "config.json"))
        args.model = os.path.join(scratch.name, "model")
        write_model_folder(args.model, load_model_config(source), args.seed, args.weight_std, args.norm_std)
    page_size = args.page_size
    num_pages = args.num_pages
    if num_pages is None:
        # a request's share of --max-tokens is a multiple of 64: whole pages when the page size divides
        # 64, else each live request may need one page more than its share of the sum
        num_pages = max(1, (args.max_tokens + page_size - 1) // page_size) + (0 if 64 % page_size == 0 else args.max_num_seqs)
    model_config = load_model_config(args.model)
    spec = model_config.to_spec()
    config = EngineConfig(dtype=args.dtype, kvcache_block_size=page_size, num_kvcache_blocks=num_pages, max_num_seqs=args.max_num_seqs,
                          max_model_len=max(page_size, num_pages * page_size), max_num_batched_tokens=max(page_size, num_pages * page_size))
    config.clamp_to_model(spec.max_position)
    dtype = torch.bfloat16 if config.dtype == "bfloat16" else torch.float32
    model = Model(spec, dtype, config.device, config.max_model_len)
    model.load(args.model)
    runner = ModelRunner(model, config)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", [])) for e in rec.get("entries", [])]
        logits = runner.step(entries)
        if logits is not None:
            out = logits.to(torch.float32).cpu().numpy().astype("<f4")
            out.tofile(os.path.join(args.out, f"{step}.f32"))
        runner.check_status()
        for rid in rec.get("end", []):
            runner.finish(rid)
        print(f"done {step}", flush=True)
    if scratch is not None:
        scratch.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
