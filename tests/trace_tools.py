"""Builders of replay traces and the subprocess driver of ``bin/trace_run`` for tests.

A trace is a list of steps ``{"step", "entries": [{"id", "tokens", "want"}], "end"}``.  The
builders below cut the same requests in different ways; ``run_trace`` replays a trace with
the real program and returns ``{(request, position): logits row}``.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class TraceBuilder:
    def __init__(self):
        self.steps: List[dict] = []
        self.rows: List[List[Tuple[str, int]]] = []  # per step: (request, position) of each wanted row
        self.progress: Dict[str, int] = {}

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end: Sequence[str] = ()):
        """entries: (request id, tokens, wanted places among them)."""
        recs, rows = [], []
        for rid, tokens, want in entries:
            start = self.progress.get(rid, 0)
            recs.append({"id": rid, "tokens": [int(t) for t in tokens], "want": [int(w) for w in want]})
            rows += [(rid, start + int(w)) for w in want]
            self.progress[rid] = start + len(tokens)
        self.steps.append({"step": len(self.steps), "entries": recs, "end": list(end)})
        self.rows.append(rows)
        for rid in end:
            self.progress.pop(rid, None)

    # ---- the ways of cutting one request --------------------------------------------------
    def whole(self, rid: str, tokens):
        self.step([(rid, tokens, range(len(tokens)))], end=[rid])

    def tail_one_by_one(self, rid: str, tokens, tail: int = 32):
        head = max(1, len(tokens) - tail)
        self.step([(rid, tokens[:head], range(head))])
        for i in range(head, len(tokens)):
            self.step([(rid, tokens[i:i + 1], [0])], end=[rid] if i == len(tokens) - 1 else [])
        if head == len(tokens):
            self.steps[-1]["end"] = [rid]
            self.progress.pop(rid, None)

    def portions(self, rid: str, tokens, sizes: Sequence[int]):
        i, k = 0, 0
        while i < len(tokens):
            n = min(sizes[k % len(sizes)], len(tokens) - i)
            last = i + n == len(tokens)
            self.step([(rid, tokens[i:i + n], range(n))], end=[rid] if last else [])
            i += n
            k += 1


def mixed_trace(builder: TraceBuilder, requests: Dict[str, Sequence[int]], prompt_lens: Dict[str, int], rng, max_live: int = 4,
                portion_sizes: Sequence[int] = (7, 5, 3, 2)):
    """Continuous batching by hand: up to ``max_live`` requests at a time; each feeds its
    "prompt" (the first ``prompt_lens[r]`` tokens) in portions of changing size and the rest one
    token a step; entries of a step are shuffled; a request now and then sits a step out.
    Finished requests end, so their pages go to the requests that start next."""
    waiting = list(requests)
    live: List[str] = []
    done = {r: 0 for r in requests}
    k = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        entries, ending = [], []
        order = list(live)
        rng.shuffle(order)
        for r in order:
            if len(order) > 1 and rng.random() < 0.15:
                continue  # left out of this step, goes on later
            toks = requests[r]
            if done[r] < prompt_lens[r]:
                n = min(portion_sizes[k % len(portion_sizes)], prompt_lens[r] - done[r])
                k += 1
            else:
                n = 1
            entries.append((r, toks[done[r]:done[r] + n], range(n)))
            done[r] += n
            if done[r] == len(toks):
                ending.append(r)
        if not entries:
            continue
        builder.step(entries, end=ending)
        for r in ending:
            live.remove(r)


def peak_tokens(builder: TraceBuilder, round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to ``round_to``."""
    held: Dict[str, int] = {}
    peak = 0
    for st in builder.steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for r in st["end"]:
            held.pop(r, None)
    return peak


def peak_pages(builder: TraceBuilder, page_size: int) -> int:
    """The most pages of ``page_size`` tokens that live requests hold at any time: the smallest pool the
    trace can run in, so that every page a request gives back is needed again."""
    held: Dict[str, int] = {}
    peak = 0
    for st in builder.steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((n + page_size - 1) // page_size for n in held.values()))
        for r in st["end"]:
            held.pop(r, None)
    return peak


def run_trace(model_dir: str, dtype: str, builder: TraceBuilder, out_dir: str, max_tokens: int, vocab: int, timeout: float = 600.0,
              env=None, options: Sequence[str] = (), model_args: Sequence[str] = ()) -> Dict[Tuple[str, int], np.ndarray]:
    """``options``: further options of the program (``--page-size`` and the like); ``model_args``
    replaces ``--model model_dir`` (for ``--random``)."""
    os.makedirs(out_dir, exist_ok=True)
    text = "".join(json.dumps(s) + "\n" for s in builder.steps)
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), *(model_args or ["--model", model_dir]), "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens), *[str(o) for o in options]]
    proc = subprocess.run(cmd, input=text, capture_output=True, text=True, timeout=timeout, env=env)
    if proc.returncode != 0:
        raise RuntimeError(f"trace_run exited with {proc.returncode}\nstdout:\n{proc.stdout[-2000:]}\nstderr:\n{proc.stderr[-4000:]}")
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == [s["step"] for s in builder.steps], "a 'done <step>' line is missing"
    out: Dict[Tuple[str, int], np.ndarray] = {}
    for st, rows in zip(builder.steps, builder.rows):
        path = os.path.join(out_dir, f"{st['step']}.f32")
        if not rows:
            assert not os.path.exists(path), f"step {st['step']} wanted nothing but wrote a file"
            continue
        data = np.fromfile(path, dtype="<f4").reshape(len(rows), vocab)
        for key, row in zip(rows, data):
            assert key not in out, f"{key} was asked for twice"
            out[key] = row
    return out
