"""Command line in the manner of the reference's ``main`` (spymaster2h/spyinfer
main.cpp:16-48, 70-122): ``-m <model_path>``, ``-b <backend_type>``, ``-h``, then a
read-generate-print loop with the commands ``/new`` and ``/exit``.  The reference reads text
and runs it through its tokenizer; this engine's interface is token ids, so a line of input
is a list of token ids (separated by spaces or commas) and the answer is printed as token
ids, streamed as they are generated.  Lines of one conversation are appended to each other;
``/new`` starts a fresh one.

    spyinfer -m /path/to/model [-b cuda] [--dtype bfloat16|float32] [--max-new-tokens N]
             [--temperature X] [--top-k K] [--seed N] [--prompt-tokens 1,2,3 | --prompt-len N] [--stats]
    spyinfer --random CONFIG.json --seed 7 ...        (random weights instead of a checkpoint)
"""
from __future__ import annotations

import argparse
import json
import re
import sys


def _parse_tokens(text: str):
    parts = [p for p in re.split(r"[\s,]+", text.strip()) if p]
    return [int(p) for p in parts]


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="spyinfer", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-m", "--model", dest="model", help="model folder (config.json and safetensors)")
    ap.add_argument("-b", "--backend", dest="backend", default="cuda", help="backend type; only \"cuda\" exists in this engine")
    ap.add_argument("--random", metavar="CONFIG_JSON", help="a config.json; the model gets seeded random weights")
    ap.add_argument("--seed", type=int, default=0, help="seed of random weights and of temperature sampling")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "bf16", "float32", "fp32"])
    ap.add_argument("--prompt-tokens", help="run this one prompt (comma-separated ids) and exit")
    ap.add_argument("--prompt-len", type=int, default=None, help="run one prompt of this many seeded random token ids and exit")
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-k", type=int, default=0, help="with a temperature: draw among the k most likely tokens only (0: all)")
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--max-num-batched-tokens", type=int, default=None)
    ap.add_argument("--max-num-seqs", type=int, default=None)
    ap.add_argument("--chunk-size", type=int, default=None, help="most prompt tokens of one request in a step")
    ap.add_argument("--max-model-len", type=int, default=None)
    ap.add_argument("--kvcache-block-size", "--page-size", dest="kvcache_block_size", type=int, default=None, help="tokens a cache page holds")
    ap.add_argument("--num-kvcache-blocks", "--num-pages", dest="num_kvcache_blocks", type=int, default=None,
                    help="pages of the cache pool (default: from free device memory)")
    ap.add_argument("--stats", action="store_true", help="print engine counters at the end")
    return ap


def main(argv=None) -> int:
    ap = build_parser()
    args = ap.parse_args(argv)
    if (args.model is None) == (args.random is None):
        print("Usage: spyinfer -m <model_path> [-b <backend_type>]   (or --random CONFIG.json)", file=sys.stderr)
        print("Use -h for help", file=sys.stderr)
        return 1
    if args.backend != "cuda":
        print(f"Invalid backend type: {args.backend}", file=sys.stderr)
        print("Available backends: cuda", file=sys.stderr)
        return 1

    from ..config import config_from_json
    from ..sampling import SamplingParams
    from .llm_engine import LLMEngine

    params = {"dtype": args.dtype}
    for key in ("max_num_batched_tokens", "max_num_seqs", "chunk_size", "max_model_len", "kvcache_block_size", "num_kvcache_blocks"):
        if getattr(args, key) is not None:
            params[key] = getattr(args, key)
    print("Using CUDA backend", flush=True)
    if args.model is not None:
        engine = LLMEngine(args.model, backend_type=args.backend, **params)
    else:
        with open(args.random) as f:
            engine = LLMEngine(model_config=config_from_json(json.load(f)), seed=args.seed, backend_type=args.backend, **params)
    sampling = SamplingParams(temperature=args.temperature, seed=args.seed, top_k=args.top_k, max_new_tokens=args.max_new_tokens, ignore_eos=args.ignore_eos)

    def run(tokens):
        rid = engine.add_request(tokens, sampling)
        while not engine.is_request_finished(rid):
            for r, tok, _ in engine.step():
                if r == rid:
                    print(tok, end=" ", flush=True)
        print(flush=True)
        out = engine.get_output_tokens(rid)
        engine.remove_request(rid)
        return out

    if args.prompt_tokens is not None:
        run(_parse_tokens(args.prompt_tokens))
    elif args.prompt_len is not None:
        import random
        rng = random.Random(args.seed)
        run([rng.randrange(engine.model.spec.vocab_size) for _ in range(max(1, args.prompt_len))])
    else:
        history = []
        while True:
            print("\nUser: ", end="", flush=True)
            line = sys.stdin.readline()
            if not line or line.strip() == "/exit":
                break
            if line.strip() == "/new":
                history = []
                print("Starting new conversation.", flush=True)
                continue
            try:
                new = _parse_tokens(line)
            except ValueError:
                print("expected token ids separated by spaces or commas, /new or /exit", flush=True)
                continue
            if not new:
                continue
            print("Assistant: ", end="", flush=True)
            try:
                history = run(history + new)
            except ValueError as e:
                print(f"\nrequest refused: {e}", flush=True)
    if args.stats:
        print(json.dumps(engine.stats()), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
