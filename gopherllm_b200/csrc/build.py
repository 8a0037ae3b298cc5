"""Compiles the CUDA sources of this folder for sm_100a and loads them.

Each ``.cu`` file becomes one shared library under ``csrc/_build`` (or, where
the package folder cannot be written, under a per-user temporary folder),
compiled by nvcc on first use and whenever the source, a header or the flags
change.  A library may be specialised by preprocessor definitions (a head size
for the attention kernels); each set of definitions is a library of its own, so
a model compiles what its sizes need and nothing else.  Libraries are loaded
with ctypes: the launchers are plain C functions.
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
from typing import Dict, Iterable, Optional, Tuple

_HERE = os.path.dirname(os.path.abspath(__file__))
_ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
# no --use_fast_math: expf, erff and division stay exact
_BASE_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-shared",
               "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
_lock = threading.Lock()
_loaded: Dict[str, ctypes.CDLL] = {}


class BuildError(RuntimeError):
    pass


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand):
            return cand
    raise BuildError("nvcc not found: the CUDA kernels of gopherllm_b200 cannot be compiled "
                     "(set NVCC or put /usr/local/cuda/bin on PATH)")


def _headers() -> Iterable[str]:
    return sorted(f for f in os.listdir(_HERE) if f.endswith((".cuh", ".h")))


def _digest(source: str, defines: Tuple[str, ...]) -> str:
    h = hashlib.sha256()
    for name in [source, *_headers()]:
        with open(os.path.join(_HERE, name), "rb") as f:
            h.update(name.encode() + b"\0" + f.read() + b"\0")
    h.update(" ".join(_ARCH_FLAGS + _BASE_FLAGS + list(defines)).encode())
    return h.hexdigest()[:16]


def _build_dirs() -> Iterable[str]:
    yield os.path.join(_HERE, "_build")
    yield os.path.join(tempfile.gettempdir(), f"gopherllm_b200_build_{os.getuid()}")


def _lib_name(source: str, defines: Tuple[str, ...]) -> str:
    stem = os.path.splitext(source)[0]
    tag = "".join("_" + d.replace("=", "").replace("GL_", "").lower() for d in defines)
    return f"libgl_{stem}{tag}"


def library_path(source: str, defines: Tuple[str, ...] = (), build: bool = True,
                 verbose: bool = True) -> str:
    """Path of the up-to-date library for ``source`` (+ -D definitions), compiling it if needed."""
    digest = _digest(source, defines)
    name = _lib_name(source, defines)
    for d in _build_dirs():
        so, stamp = os.path.join(d, name + ".so"), os.path.join(d, name + ".hash")
        if os.path.isfile(so) and os.path.isfile(stamp):
            with open(stamp) as f:
                if f.read().strip() == digest:
                    return so
    if not build:
        raise BuildError(f"{name}.so is not built")
    last_err: Optional[Exception] = None
    for d in _build_dirs():
        try:
            os.makedirs(d, exist_ok=True)
            probe = os.path.join(d, f".w{os.getpid()}_{threading.get_ident()}")
            with open(probe, "w"):
                pass
            os.remove(probe)
        except OSError as e:
            last_err = e
            continue
        so, stamp = os.path.join(d, name + ".so"), os.path.join(d, name + ".hash")
        tmp = os.path.join(d, f"{name}.{os.getpid()}_{threading.get_ident()}.tmp.so")
        cmd = [_nvcc(), *_ARCH_FLAGS, *_BASE_FLAGS, *[f"-D{x}" for x in defines],
               "-I", _HERE, "-o", tmp, os.path.join(_HERE, source)]
        if verbose:
            print(f"[gopherllm_b200] compiling {source}{' ' + ' '.join(defines) if defines else ''} "
                  f"for sm_100a ...", file=sys.stderr, flush=True)
        t0 = time.time()
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"nvcc failed on {source}:\n{' '.join(cmd)}\n{proc.stderr[-4000:]}")
        os.replace(tmp, so)
        with open(stamp, "w") as f:
            f.write(digest)
        if verbose:
            print(f"[gopherllm_b200] built {name}.so in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)
        return so
    raise BuildError(f"no writable build folder for {name}.so: {last_err}")


def load(source: str, defines: Tuple[str, ...] = ()) -> ctypes.CDLL:
    """The loaded library for ``source``; compiled first if it is missing or stale."""
    key = _lib_name(source, defines)
    with _lock:
        lib = _loaded.get(key)
        if lib is None:
            lib = ctypes.CDLL(library_path(source, defines))
            _loaded[key] = lib
        return lib


def build_all(head_dims: Iterable[int] = (), verbose: bool = True) -> None:
    """Compile every library (the per-head-size ones for ``head_dims``), several at a time."""
    from . import catalog
    jobs = list(catalog.all_libraries(head_dims))
    errors = []

    def work(job):
        try:
            library_path(job[0], job[1], verbose=verbose)
        except Exception as e:  # collected and raised below
            errors.append(e)

    threads = []
    width = max(1, min(len(jobs), os.cpu_count() or 1))
    pending = list(jobs)
    while pending or threads:
        while pending and len(threads) < width:
            t = threading.Thread(target=work, args=(pending.pop(0),))
            t.start()
            threads.append(t)
        threads[0].join()
        threads.pop(0)
    if errors:
        raise errors[0]
