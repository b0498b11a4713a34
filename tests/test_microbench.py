"""The measuring commands that the summaries under profiles/ cite run and print their line."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run(*args):
    proc = subprocess.run([sys.executable, "-m", "spyinfer_b200.microbench", *[str(a) for a in args]], cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return proc.stdout


def test_microbench_commands_run():
    assert "TFLOP/s" in run("gemm", "--m", 8, "--n", 512, "--k", 512, "--iters", 3, "--graph", "--defer")
    assert "TFLOP/s" in run("gemm", "--m", 300, "--n", 512, "--k", 512, "--iters", 3, "--epilogue", "swiglu")
    assert "cache read at" in run("attention", "--batch", 3, "--context", 300, "--kernel", "decode", "--iters", 2, "--graph", "--heads", 10, "--kv-heads", 2, "--head-dim", 64)
    assert "cache read at" in run("attention", "--batch", 1, "--context", 300, "--q-len", 300, "--kernel", "tc", "--iters", 2)
    assert "GB/s" in run("rmsnorm", "--rows", 64, "--size", 1024, "--splits", 3, "--iters", 3)
    out = run("step", "--batch", 2, "--context", 100, "--layers", 1)
    assert "whole step" in out and "attention_decode_kernel" in out
