"""Builds the reference project (spymaster2h/spyinfer) unmodified, by hand, into ``baseline/_ref``.

The reference is a C++20 project built by xmake (its ``xmake.lua``, target "main" with
``backend=cuda``); it is no Python package, so ``pip install`` cannot take it, and xmake is not
on this image.  This script does what that target does, with the compilers that are: every
``src/backends/cuda/**.cpp|.cu``, ``src/backends/cpu/**.cpp``, ``src/core/**.cpp`` and the
``src/utils`` files the model needs are compiled from the reference's tree as they are
(``-DUSE_CUDA``, C++20, AVX-512 flags for the CPU backend's files only, sm_100a for the kernels)
and linked with ``reference_decode.cpp`` (the benchmark's driver, this repository's own file) and
cuBLAS into ``baseline/_ref/reference_decode``.  The engine (``src/engine``), the tokenizer and
``main.cpp`` are left out: the driver calls the model directly (see its header for why).

    python baseline/build_reference.py [--reference /path/to/spyinfer] [--force]

Prints the path of the binary, or the compiler's message and exit code 1.
"""
from __future__ import annotations

import argparse
import glob
import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
DEFAULT_REFERENCE = "/root/reference"


def json_include() -> str:
    """A directory that holds nlohmann/json.hpp (the reference's only outside header)."""
    for pat in (os.path.join(sys.prefix, "lib/python*/site-packages/include/cudnn_frontend/thirdparty"), "/usr/include", "/usr/local/include"):
        for d in glob.glob(pat):
            if os.path.isfile(os.path.join(d, "nlohmann", "json.hpp")):
                return d
    raise FileNotFoundError("nlohmann/json.hpp was not found on this machine")


def sources(ref: str):
    pats = ["src/backends/cuda/*.cpp", "src/backends/cuda/*.cu", "src/backends/cuda/*/*.cu", "src/backends/cpu/*.cpp", "src/backends/cpu/x64/*.cpp",
            "src/core/*.cpp", "src/utils/context.cpp", "src/utils/safetensors_reader.cpp"]
    out = []
    for p in pats:
        out += sorted(glob.glob(os.path.join(ref, p)))
    return out


def build(ref: str = DEFAULT_REFERENCE, force: bool = False) -> str:
    exe = os.path.join(OUT, "reference_decode")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.isdir(os.path.join(ref, "src")):
        if os.path.isfile(exe) and not force:
            return exe                      # built where the sources are; the binary travels with the repository's folder
        raise FileNotFoundError(f"the reference's sources are not at {ref} and no binary built from them is at {exe}")
    srcs = sources(ref) + [os.path.join(HERE, "reference_decode.cpp")]
    stamp = hashlib.sha256()
    for s in srcs:
        with open(s, "rb") as f:
            stamp.update(s.encode() + f.read())
    stamp_file = exe + ".hash"
    if not force and os.path.isfile(exe) and os.path.isfile(stamp_file) and open(stamp_file).read() == stamp.hexdigest():
        return exe
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    inc = ["-I", os.path.join(ref, "src"), "-I", json_include()]
    common = ["-std=c++20", "-O2", "-DUSE_CUDA"]

    def compile_one(src: str) -> str:
        obj = os.path.join(OUT, "obj", hashlib.sha1(src.encode()).hexdigest()[:12] + "_" + os.path.basename(src) + ".o")
        host_flags = ["-mavx512f", "-mavx512bw", "-mavx512dq", "-mfma"] if "/backends/cpu/" in src else []
        if src.endswith(".cu"):
            cmd = [nvcc, "-c", src, "-o", obj, *common, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", *inc]
        else:
            cmd = [nvcc, "-c", src, "-o", obj, *common, *inc] + (["-Xcompiler", ",".join(host_flags)] if host_flags else [])
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=8) as pool:
        objs = list(pool.map(compile_one, srcs))
    libdir = os.path.join(os.path.dirname(os.path.dirname(os.path.realpath(nvcc))), "lib64")
    cmd = [nvcc, "-o", exe, *objs, "-lcublas", "-lcublasLt", "-lpthread", "-Xlinker", f"-rpath={libdir}"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")
    with open(stamp_file, "w") as f:
        f.write(stamp.hexdigest())
    return exe


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    args = ap.parse_args()
    try:
        print(build(args.reference, args.force))
    except (RuntimeError, FileNotFoundError) as e:
        print(str(e)[-4000:], file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
