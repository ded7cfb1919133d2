"""Build and load the CUDA kernel library.

The ``.cu`` files of this folder are compiled with nvcc for sm_100a into one shared
library, ``_build/librocml_b200.so`` beside them, and loaded with ctypes.  The build runs
at the first use when the library is absent or older than its sources, prints a line per
file while it works, and needs neither network nor a home directory.  There is no other
implementation behind it: without the library (and without nvcc to make it) every kernel
call fails with ``ExtensionMissing``.
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

from ..errors import ExtensionMissing

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_NAME = "librocml_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]
_lock = threading.Lock()
_lib = None


def sources():
    return sorted(f for f in os.listdir(_HERE) if f.endswith(".cu"))


def _headers():
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def _fingerprint() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in sources() + _headers():
        h.update(f.encode())
        with open(os.path.join(_HERE, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise ExtensionMissing(
        "the CUDA kernel library is not built and nvcc was not found (looked at $NVCC, PATH and "
        "/usr/local/cuda/bin/nvcc); this library has no other implementation to fall back to"
    )


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
        # a read-only checkout: build where this user may write
        d = os.path.join(tempfile.gettempdir(), f"rocml_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _say(msg: str) -> None:
    print(f"[rocml_b200 build] {msg}", file=sys.stderr, flush=True)


def build(verbose: bool = True, force: bool = False) -> str:
    """Compile what is stale; return the library's path."""
    out_dir = _build_dir()
    lib_path = os.path.join(out_dir, _LIB_NAME)
    stamp = os.path.join(out_dir, "fingerprint.txt")
    fp = _fingerprint()
    if not force and os.path.isfile(lib_path) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == fp:
                return lib_path
    nvcc = _nvcc()
    srcs = sources()
    if verbose:
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first use only)")
    t0 = time.time()

    def compile_one(src):
        obj = os.path.join(out_dir, src[:-3] + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", _HERE, "-c", os.path.join(_HERE, src), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise ExtensionMissing(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _say(f"  {src} done ({time.time() - t0:.0f} s)")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
        objs = list(pool.map(compile_one, srcs))
    tmp = lib_path + f".tmp{os.getpid()}"
    r = subprocess.run([nvcc, "-shared", "-o", tmp, *objs, "-lcudart"], capture_output=True, text=True)
    if r.returncode != 0:
        raise ExtensionMissing(f"linking {_LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, lib_path)
    with open(stamp, "w") as f:
        f.write(fp)
    if verbose:
        _say(f"built {_LIB_NAME} in {time.time() - t0:.0f} s")
    return lib_path


def library() -> ctypes.CDLL:
    """The loaded kernel library (built first when needed)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = build()
                try:
                    _lib = ctypes.CDLL(path)
                except OSError as e:
                    raise ExtensionMissing(f"cannot load {path}: {e}") from e
    return _lib


def library_path() -> str:
    return os.path.join(_build_dir(), _LIB_NAME)
