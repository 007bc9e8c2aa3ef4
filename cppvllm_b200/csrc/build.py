"""Compiles the package's CUDA sources for sm_100a with nvcc and loads the shared libraries through ctypes.

Each *library* is a named group of ``.cu`` files next to this module.  A library is compiled the first time
it is asked for (so a model compiles only the kernels it needs), into ``_build/`` next to the sources, or
into a per-user folder under the system's temporary directory when the package folder cannot be written.
A stamp file with a hash of the sources and flags decides whether a rebuild is needed.  While nvcc runs, a
line goes to stderr every few seconds, so a first call that compiles does not look hung.

The sources include no PyTorch header: launchers take raw pointers and a stream, which keeps a cold build
to a few seconds per file.  If nvcc is missing or a compilation fails the error is raised; nothing falls
back to another implementation.
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
from typing import Dict, List

_HERE = os.path.dirname(os.path.abspath(__file__))

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]

# library name -> source files
LIBRARIES: Dict[str, List[str]] = {
    "core": ["elementwise.cu", "qk_rope_kv.cu", "attention_general.cu", "sampling.cu", "selftest.cu"],
    "attn_bf16": ["attention_bf16.cu"],
    "gemv_bf16": ["gemv_bf16.cu"],
    "gemm_bf16": ["gemm_tcgen05.cu"],
    "attn_tcgen05": ["attention_tcgen05.cu"],
    # host code only (the cache manager and the scheduler); nvcc hands it to the host compiler
    "runtime": ["cache_runtime.cpp", "scheduler_runtime.cpp"],
}

_HEADERS = ["common.cuh", "sm100.cuh", "tensor_map.cuh", "attention_bf16.h", "runtime.hpp"]
_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


class BuildError(RuntimeError):
    pass


def _find_nvcc() -> str:
    for cand in (os.environ.get("CUDACXX"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.isfile(cand) and os.access(cand, os.X_OK):
            return cand
    raise BuildError("nvcc not found (looked at $CUDACXX, PATH and /usr/local/cuda/bin): the CUDA kernels "
                     "cannot be compiled and there is no other implementation to fall back to")


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
        d = os.path.join(tempfile.gettempdir(), f"cppvllm_b200_build_{os.getuid()}")
        os.makedirs(d, exist_ok=True)
        return d


def _digest(name: str) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for f in _HEADERS + LIBRARIES[name]:
        with open(os.path.join(_HERE, f), "rb") as fh:
            h.update(f.encode())
            h.update(fh.read())
    return h.hexdigest()


def _say(msg: str) -> None:
    print(f"[cppvllm_b200] {msg}", file=sys.stderr, flush=True)


def library_path(name: str) -> str:
    return os.path.join(_build_dir(), f"libcvb_{name}.so")


def build_library(name: str, verbose: bool = True) -> str:
    """Compile library `name` if its stamp is stale; return the path of the .so."""
    if name not in LIBRARIES:
        raise BuildError(f"unknown kernel library '{name}'; known: {sorted(LIBRARIES)}")
    out_dir = _build_dir()
    so = os.path.join(out_dir, f"libcvb_{name}.so")
    stamp = so + ".stamp"
    digest = _digest(name)
    if os.path.isfile(so) and os.path.isfile(stamp):
        with open(stamp) as f:
            if f.read().strip() == digest:
                return so
    nvcc = _find_nvcc()
    t0 = time.time()
    if verbose:
        _say(f"compiling kernel library '{name}' for sm_100a ({len(LIBRARIES[name])} files) ...")
    procs = []
    objs = []
    for src in LIBRARIES[name]:
        obj = os.path.join(out_dir, f"{name}__{os.path.splitext(src)[0]}.{os.getpid()}.o")
        objs.append(obj)
        cmd = [nvcc] + NVCC_FLAGS + ["-I", _HERE, "-c", os.path.join(_HERE, src), "-o", obj]
        procs.append((src, cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    last = time.time()
    pending = list(procs)
    logs = {}
    while pending:
        for item in list(pending):
            src, cmd, p = item
            if p.poll() is not None:
                logs[src] = (p.returncode, p.stdout.read())
                pending.remove(item)
        if pending:
            time.sleep(0.2)
            if verbose and time.time() - last > 5:
                _say(f"  still compiling ({', '.join(s for s, _, _ in pending)}; {time.time() - t0:.0f} s)")
                last = time.time()
    failed = {s: log for s, (rc, log) in logs.items() if rc != 0}
    if failed:
        for o in objs:
            if os.path.exists(o):
                os.remove(o)
        text = "\n".join(f"--- {s} ---\n{log}" for s, log in failed.items())
        raise BuildError(f"nvcc failed for kernel library '{name}':\n{text}")
    tmp_so = so + f".{os.getpid()}.tmp"
    link = [nvcc, "-shared", "-o", tmp_so] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    for o in objs:
        if os.path.exists(o):
            os.remove(o)
    if r.returncode != 0:
        raise BuildError(f"linking kernel library '{name}' failed:\n{r.stdout}")
    os.replace(tmp_so, so)            # atomic: a concurrent process sees the old or the new file, never half
    with open(stamp + f".{os.getpid()}", "w") as f:
        f.write(digest)
    os.replace(stamp + f".{os.getpid()}", stamp)
    if verbose:
        _say(f"kernel library '{name}' ready in {time.time() - t0:.1f} s: {so}")
    return so


def load_library(name: str) -> ctypes.CDLL:
    """The library `name`, built if need be.  CVB_LIBRARY_<NAME> in the environment names a file to load instead (a build
    of the same sources with other flags, for instance the host runtime compiled with sanitizers)."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            override = os.environ.get(f"CVB_LIBRARY_{name.upper()}")
            lib = ctypes.CDLL(override if override else build_library(name))
            _loaded[name] = lib
        return lib


def build_all(verbose: bool = True) -> List[str]:
    return [build_library(n, verbose=verbose) for n in LIBRARIES]
