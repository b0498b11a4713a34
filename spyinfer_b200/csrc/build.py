"""Builds and loads the native modules: the CUDA kernels and the host-side engine core.

Every ``<module>.cu`` in this folder becomes one shared library with a C interface, built
with nvcc for sm_100a and loaded with ctypes; ``engine_core.cpp`` (the cache's bookkeeping,
the scheduler's decisions and the batch assembly, no CUDA) is built with the host compiler.  A module is built the first time something
asks for it (or all at once by ``build_all``), into ``_build/`` beside the sources when that
folder can be written, else into a per-user folder under the system's temporary folder.  A
library is reused when the hash of its sources, the shared header and the flags is the one
it was built from; time stamps are not trusted.  While nvcc runs, a line is printed to
standard error now and then.  There is no fallback: without nvcc, or when a build fails, the
caller gets an error with the compiler's output.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Dict, Iterable, List

HERE = os.path.dirname(os.path.abspath(__file__))
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-shared",
              "-Xcompiler", "-fvisibility=default"]
HOST_MODULES = ["engine_core"]                 # plain C++, built with the host compiler
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=default"]
MODULES = ["embedding", "rmsnorm", "qk_rope_store", "attention_generic", "attention_mma", "attention_tc", "attention_decode", "gemm_simt", "gemm_tcgen05", "swiglu", "sampling"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()
_dir_lock = threading.Lock()


class KernelBuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise KernelBuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin): the CUDA kernels cannot be built, "
                           "and this engine has no other path")


_build_dir_cached = None


def _build_dir() -> str:
    """Decided once per process: ``_build/`` beside the sources if it can be written, else a
    per-user folder under the temporary folder."""
    global _build_dir_cached
    if _build_dir_cached is not None:
        return _build_dir_cached
    with _dir_lock:
        if _build_dir_cached is None:
            local = os.path.join(HERE, "_build")
            try:
                os.makedirs(local, exist_ok=True)
                fd, probe = tempfile.mkstemp(prefix=".probe", dir=local)
                os.close(fd)
                os.remove(probe)
                _build_dir_cached = local
            except OSError:
                d = os.path.join(tempfile.gettempdir(), f"spyinfer_b200_build_{os.getuid()}")
                os.makedirs(d, exist_ok=True)
                _build_dir_cached = d
    return _build_dir_cached


def _cxx() -> str:
    for cand in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), shutil.which("clang++")):
        if cand and shutil.which(cand):
            return shutil.which(cand)
    raise KernelBuildError("no C++ compiler was found (looked at $CXX, g++, c++, clang++): the engine core cannot be built")


def _extra_flags() -> List[str]:
    """More nvcc flags from the environment (``SPYINFER_NVCC_FLAGS``), e.g. ``-DNAME`` switches for experiments."""
    return os.environ.get("SPYINFER_NVCC_FLAGS", "").split()


def _source_hash(module: str) -> str:
    h = hashlib.sha256()
    if module in HOST_MODULES:
        h.update(" ".join(HOST_FLAGS).encode())
        with open(os.path.join(HERE, module + ".cpp"), "rb") as f:
            h.update(f.read())
        return h.hexdigest()
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS + _extra_flags()).encode())
    for name in sorted(os.listdir(HERE)):
        if name.endswith(".cuh") or name.endswith(".h") or name == module + ".cu":
            with open(os.path.join(HERE, name), "rb") as f:
                h.update(name.encode())
                h.update(f.read())
    return h.hexdigest()


def library_path(module: str) -> str:
    return os.path.join(_build_dir(), f"libspy_{module}.so")


def _is_current(module: str) -> bool:
    so = library_path(module)
    stamp = so + ".hash"
    if not (os.path.isfile(so) and os.path.isfile(stamp)):
        return False
    with open(stamp) as f:
        return f.read().strip() == _source_hash(module)


def _compile(module: str) -> None:
    host = module in HOST_MODULES
    src = os.path.join(HERE, module + (".cpp" if host else ".cu"))
    if not os.path.isfile(src):
        raise KernelBuildError(f"no native module {module!r} ({src} does not exist)")
    so = library_path(module)
    tmp = f"{so}.{os.getpid()}.tmp"
    if host:
        cmd = [_cxx()] + HOST_FLAGS + ["-o", tmp, src]
    else:
        cmd = [_nvcc()] + ARCH_FLAGS + NVCC_FLAGS + _extra_flags() + ["-I", HERE, "-o", tmp, src]
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    t0 = time.time()
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    done = threading.Event()

    def ticker():
        while not done.wait(15.0):
            print(f"[spyinfer_b200] still compiling {os.path.basename(src)} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    out, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        if os.path.exists(tmp):
            os.remove(tmp)
        raise KernelBuildError(f"the compiler failed on {os.path.basename(src)}:\n$ {' '.join(cmd)}\n{out}")
    os.replace(tmp, so)
    with open(so + ".hash", "w") as f:
        f.write(_source_hash(module))
    print(f"[spyinfer_b200] compiled {os.path.basename(src)} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def ensure_built(modules: Iterable[str]) -> None:
    """Builds, in parallel, those of ``modules`` whose library is missing or out of date."""
    todo = [m for m in dict.fromkeys(modules) if not _is_current(m)]
    if not todo:
        return
    print(f"[spyinfer_b200] compiling {len(todo)} native module(s) (CUDA kernels for sm_100a, host core): {', '.join(todo)}", file=sys.stderr, flush=True)
    with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 1)) as pool:
        for f in [pool.submit(_compile, m) for m in todo]:
            f.result()


def build_all() -> List[str]:
    ensure_built(MODULES + HOST_MODULES)
    return [library_path(m) for m in MODULES + HOST_MODULES]


def load(module: str) -> ctypes.CDLL:
    """The loaded library of one module, built first if need be."""
    lib = _loaded.get(module)
    if lib is not None:
        return lib
    with _lock:
        lib = _loaded.get(module)
        if lib is None:
            ensure_built([module])
            try:
                lib = ctypes.CDLL(library_path(module))
            except OSError as e:
                raise KernelBuildError(f"cannot load {library_path(module)}: {e}") from None
            err = getattr(lib, f"spy_{module}_last_error")
            err.restype = ctypes.c_char_p
            _loaded[module] = lib
    return lib


def last_error(module: str) -> str:
    return getattr(load(module), f"spy_{module}_last_error")().decode(errors="replace")
