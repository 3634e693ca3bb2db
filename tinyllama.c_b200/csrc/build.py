"""Builds and loads the CUDA kernel library (sm_100a only).

The reference builds its kernels with ``nvcc -O3 -arch=native`` from a Makefile
(src/Makefile:34).  Here the library is compiled on first use, in the source tree,
with plain ``nvcc`` (no framework headers, so a file takes seconds), and loaded with
``ctypes``.  There is no fallback: if it cannot be built or loaded, importing the
kernels raises.
"""
from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time

_HERE = os.path.dirname(os.path.abspath(__file__))
_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
          "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
LIB_NAME = "libtinyllama_c_b200.so"
_lock = threading.Lock()
_lib = None


class KernelBuildError(RuntimeError):
    pass


def sources():
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"),
                 os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc"),
                 "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise KernelBuildError("nvcc not found (looked at $NVCC, PATH, $CUDA_HOME/bin, /usr/local/cuda/bin); "
                           "the CUDA kernels of tinyllama.c_b200 cannot be built and there is no fallback")


def _fingerprint() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(_HERE)):
        if name.endswith((".cu", ".cuh", ".h")):
            h.update(name.encode())
            with open(os.path.join(_HERE, name), "rb") as f:
                h.update(f.read())
    h.update(" ".join(_FLAGS).encode())
    return h.hexdigest()[:16]


def _build_dir() -> str:
    d = os.path.join(_HERE, "_build")
    try:
        os.makedirs(d, exist_ok=True)
        probe = os.path.join(d, f".w{os.getpid()}")
        with open(probe, "w"):
            pass
        os.remove(probe)
        return d
    except OSError:
        d = os.path.join(tempfile.gettempdir(), f"tinyllama_c_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[tinyllama.c_b200] {msg}", file=sys.stderr, flush=True)


def build(force: bool = False, verbose: bool = True) -> str:
    """Compiles every .cu file of this folder into one shared library; returns its path."""
    bdir = _build_dir()
    fp = _fingerprint()
    lib = os.path.join(bdir, LIB_NAME)
    stamp = os.path.join(bdir, "fingerprint")
    if not force and os.path.isfile(lib) and os.path.isfile(stamp) and open(stamp).read().strip() == fp:
        return lib
    nvcc = _nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {bdir} (first call only)")
    t0 = time.time()

    def compile_one(name: str) -> str:
        obj = os.path.join(bdir, name[:-3] + ".o")
        cmd = [nvcc, *_FLAGS, "-I", _HERE, "-c", os.path.join(_HERE, name), "-o", obj]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {name}:\n{p.stdout}\n{p.stderr}")
        if verbose:
            _say(f"  compiled {name} ({time.time() - t0:.0f}s)")
        return obj

    done = threading.Event()

    def heartbeat():
        while not done.wait(10.0):
            _say(f"  still compiling ... {time.time() - t0:.0f}s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        hb.start()
    try:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
            objs = list(ex.map(compile_one, srcs))
        tmp = lib + f".tmp{os.getpid()}"
        p = subprocess.run([nvcc, "-shared", "-o", tmp, *objs], capture_output=True, text=True)
        if p.returncode != 0:
            raise KernelBuildError(f"link failed:\n{p.stdout}\n{p.stderr}")
        os.replace(tmp, lib)
        with open(stamp, "w") as f:
            f.write(fp)
    finally:
        done.set()
    if verbose:
        _say(f"built {LIB_NAME} in {time.time() - t0:.0f}s")
    return lib


def load() -> ctypes.CDLL:
    """The loaded kernel library (built first if its sources changed)."""
    global _lib
    with _lock:
        if _lib is None:
            path = build()
            try:
                _lib = ctypes.CDLL(path)
            except OSError as e:
                raise KernelBuildError(f"cannot load {path}: {e}") from e
    return _lib
