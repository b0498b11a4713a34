"""Trace replay: feeds given token ids through a model step by step and writes logits.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as one batch through ``ModelRunner.step`` (the step function that
generation uses, with the same model, cache manager and kernels); nothing is sampled.  For a
step in which something is wanted, ``OUT/<step>.f32`` gets the logits at the wanted places,
in the order of the entries and of ``want``, little-endian float32 ``[wanted, vocab]``.
Requests named in ``end`` give back what they hold after the step.  After every step a line
``done <step>`` is printed and flushed.  The cache pool holds ``--max-tokens`` tokens (pages
of 16), so pages are used again as requests end.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True, help="most tokens live requests hold at any time")
    args = ap.parse_args(argv)

    import torch

    from ..config import EngineConfig, load_model_config
    from .batch import StepEntry
    from .model import Model
    from .runner import ModelRunner

    os.makedirs(args.out, exist_ok=True)
    page_size = 16
    num_pages = max(1, (args.max_tokens + page_size - 1) // page_size)
    model_config = load_model_config(args.model)
    spec = model_config.to_spec()
    config = EngineConfig(dtype=args.dtype, kvcache_block_size=page_size, num_kvcache_blocks=num_pages, max_num_seqs=8,
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
    return 0


if __name__ == "__main__":
    sys.exit(main())
